"""The distributed-tensor engine on a GPU: a tensor worker per proc executes the controller's
operator stream on its device, named streams are CUDA streams joined by borrows, and
``Tensor.reduce`` runs on this package's NVLink kernels through a communicator whose
buffers were exchanged over actor messages (no ``torch.distributed`` on that path).  One
GPU here, so the mesh has one proc; tests/multigpu_tensor_engine.py repeats the reduce
checks on 2-8 GPUs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dm():
    from monarch_b200 import tensor_engine as te
    from monarch_b200.actor import this_host
    pm = this_host().spawn_procs(per_host={"gpus": 1})
    mesh = te.spawn_tensor_engine(pm, use_cuda=True)
    yield mesh
    mesh.exit()
    pm.stop().get()


def _launches(dm):
    """Kernels of this library launched inside the worker process so far."""
    from monarch_b200 import tensor_engine as te

    def count(_t):
        from monarch_b200.ops import kernels as K
        return K.launch_count
    return te.call_on_shard_and_fetch(count, torch.zeros(1, device="cuda"), shard={"gpus": 0}).get()


def test_ops_run_on_the_device_and_match_torch(dm):
    from monarch_b200 import tensor_engine as te
    with dm.activate():
        a = torch.arange(12, dtype=torch.float32, device="cuda").reshape(3, 4)
        b = 2 * a + 1
        c = (b @ b.t()).relu().sum()
        w = torch.ones(4, 4, dtype=torch.bfloat16, device="cuda")
        d = (a.to(torch.bfloat16) @ w).float()
        where = te.call_on_shard_and_fetch(lambda t: str(t.device), b, shard={"gpus": 0}).get()
        got_b, got_c, got_d = te.inspect(b), te.inspect(c), te.inspect(d)
    assert where.startswith("cuda")
    ra = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    rb = 2 * ra + 1
    assert torch.equal(got_b, rb)
    assert got_c.item() == (rb @ rb.t()).relu().sum().item()
    assert torch.allclose(got_d, ra.sum(1, keepdim=True).expand(3, 4))


def test_reduce_variants_use_the_nvlink_kernels(dm):
    from monarch_b200 import tensor_engine as te
    with dm.activate():
        before = _launches(dm)
        x = torch.arange(6, dtype=torch.float32, device="cuda").reshape(1, 6) + 1
        r_sum = te.inspect(x.reduce("gpus", "sum"))
        r_avg = te.inspect(x.reduce("gpus", "avg"))
        r_max = te.inspect(x.to(torch.bfloat16).reduce("gpus", "max"))
        r_stack = te.inspect(x.reduce("gpus", "stack"))
        r_rs = te.inspect(x.reduce("gpus", "sum", scatter=True))
        r_a2a = te.inspect(x.reduce("gpus", "stack", scatter=True))
        y = x.clone()
        y.reduce_("gpus", "sum")
        r_in = te.inspect(y)
        o = torch.zeros(1, 6, device="cuda")
        x.reduce("gpus", "sum", out=o)
        r_out = te.inspect(o)
        after = _launches(dm)
    ref = torch.arange(6, dtype=torch.float32).reshape(1, 6) + 1
    assert torch.equal(r_sum, ref) and torch.equal(r_avg, ref) and torch.equal(r_in, ref)
    assert torch.equal(r_max.float(), ref) and torch.equal(r_out, ref)
    assert r_stack.shape == (1, 1, 6) and torch.equal(r_stack[0], ref)
    assert r_rs.shape == (6,) and torch.equal(r_rs, ref[0])
    assert r_a2a.shape == (1, 6) and torch.equal(r_a2a, ref)
    # launched by the tensor worker: one kernel per small all-reduce (it stages, handshakes and
    # combines), stage + reduce or stage + gather for the other five collectives
    assert after - before >= 11, (before, after)


def test_borrow_between_two_cuda_streams(dm):
    from monarch_b200 import tensor_engine as te
    side = te.Stream("side")
    with dm.activate():
        x = torch.ones(1 << 20, device="cuda")
        for _ in range(8):
            x = x * 1.0 + 1.0            # work in flight on the main stream
        y, borrow = side.borrow(x, mutable=True)
        with side.activate():
            y.add_(2)
            z = y.reduce("gpus", "sum")  # a collective on the side stream: its own communicator
        borrow.drop()
        got = te.inspect(x)
        with side.activate():
            got_z = te.inspect(z)
    assert got[0].item() == 11 and got[-1].item() == 11
    assert got_z[0].item() == 11


def test_to_mesh_and_fetch_shard(dm):
    from monarch_b200 import tensor_engine as te
    with dm.activate():
        f = (dm.rank("gpus") + 3).to(torch.float32).cuda() * torch.ones(2, 2, device="cuda")
        g = f.to_mesh(dm)
        g.add_(1)
        assert te.fetch_shard(f, gpus=0).get().tolist() == [[3.0, 3.0], [3.0, 3.0]]
        assert te.fetch_shard(g, gpus=0).get().tolist() == [[4.0, 4.0], [4.0, 4.0]]


def _udf_collectives(x, pg):
    """Worker-side code written against torch.distributed: the group it receives runs on the
    package's NVLink kernels (backend name "mb200"), not on NCCL."""
    import torch.distributed as dist
    assert pg.getBackendName() == "mb200" and not dist.is_initialized()
    out = x.clone()
    dist.all_reduce(out, group=pg)
    gathered = torch.empty(pg.size() * x.numel(), device=x.device, dtype=x.dtype)
    dist.all_gather_into_tensor(gathered, x.reshape(-1), group=pg)
    mx = x.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=pg)
    dist.broadcast(mx, 0, group=pg)
    dist.barrier(group=pg)
    return out + gathered.view(pg.size(), *x.shape).sum(0) + mx


def test_user_defined_function_gets_a_process_group_over_the_nvlink_kernels(dm):
    from monarch_b200 import tensor_engine as te
    fn = te.remote(_udf_collectives, propagate=lambda x, pg: x)
    with dm.activate():
        pg = dm.process_group("gpus")
        x = torch.arange(4, dtype=torch.float32, device="cuda") + 1
        got = te.inspect(fn(x, pg))
    assert got.tolist() == [3.0, 6.0, 9.0, 12.0]
