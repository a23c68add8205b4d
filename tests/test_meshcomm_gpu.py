"""The mesh communicator's kernels on one GPU: a group of one rank runs the same stage /
reduce / gather kernels (the wait sees the rank's own flag), which pins down staging
layout, chunking, dtype handling and ragged sizes against plain PyTorch.  Groups of 2-8
ranks are checked by tests/multigpu_meshcomm.py (needs as many GPUs)."""
import pytest
import torch

from monarch_b200.parallel.meshcomm import MeshComm, plan_chunks


def test_plan_chunks_covers_and_aligns():
    assert plan_chunks(0, 64) == [(0, 0)]
    for n, cap in ((1, 64), (64, 64), (65, 64), (1000, 48), (4096, 1 << 20)):
        ch = plan_chunks(n, cap)
        assert ch[0][0] == 0 and sum(s for _, s in ch) == n
        assert all(o % 16 == 0 and 0 < s <= cap for o, s in ch)
        assert all(ch[i][0] + ch[i][1] == ch[i + 1][0] for i in range(len(ch) - 1))


@pytest.fixture(scope="module")
def comm():
    from monarch_b200.ops import ipc
    dev = torch.device("cuda", 0)
    cap = 1 << 16                      # small on purpose: forces the chunked paths
    local = MeshComm.allocate_local(dev, cap)
    c = MeshComm.from_exports(0, [ipc.export_handle(local)], local, dev, cap)
    c.one_shot_bytes = 1 << 12         # both all-reduce algorithms get exercised
    return c


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64,
                                   torch.int32, torch.int64])
@pytest.mark.parametrize("n", [1, 7, 1024, 100_003])
def test_all_reduce_of_one_rank_is_the_identity(comm, dtype, n):
    from monarch_b200.ops import kernels as K
    x = (torch.randn(n, device="cuda") * 10).to(dtype)
    for op in ("sum", "avg", "product", "min", "max"):
        if op == "avg" and not dtype.is_floating_point:
            continue
        y = comm.all_reduce(x, op)
        torch.cuda.synchronize()
        K.check_status("cuda")
        assert y.shape == x.shape and y.dtype == dtype
        assert torch.equal(y, x), (op, dtype, n)
    if not dtype.is_floating_point and dtype in (torch.int32, torch.int64):
        for op in ("band", "bor", "bxor"):
            assert torch.equal(comm.all_reduce(x, op), x), (op, dtype, n)
    z = x.clone()
    assert comm.all_reduce(z, "sum", out=z) is z
    torch.cuda.synchronize()
    assert torch.equal(z, x)


@pytest.mark.gpu
def test_copy_collectives_and_ragged_shapes(comm):
    from monarch_b200.ops import kernels as K
    x = torch.randn(1, 333, 7, device="cuda").to(torch.bfloat16)
    assert torch.equal(comm.all_gather(x[0]), x)
    assert torch.equal(comm.all_to_all(x), x)
    assert torch.equal(comm.reduce_scatter(x, "sum"), x[0])
    assert torch.equal(comm.broadcast(x, 0), x)
    assert torch.equal(comm.reduce(x, 0, "max"), x)
    big = torch.randn(1, 70_001, device="cuda")          # several passes through the staging
    assert torch.equal(comm.reduce_scatter(big, "sum"), big[0])
    assert torch.equal(comm.all_to_all(big), big)
    assert torch.equal(comm.all_gather(big[0]), big)
    u8 = torch.randint(0, 255, (1, 1001), device="cuda", dtype=torch.uint8)
    assert torch.equal(comm.all_gather(u8[0]), u8)       # copies take any dtype
    view = torch.randn(64, 64, device="cuda")[:, 1:9]    # non-contiguous, misaligned start
    assert torch.equal(comm.all_reduce(view, "sum"), view)
    comm.barrier()
    torch.cuda.synchronize()
    K.check_status("cuda")
    with pytest.raises(TypeError):
        comm.all_reduce(u8, "sum")
    with pytest.raises(ValueError):
        comm.reduce_scatter(torch.zeros(3, 4, device="cuda"), "sum")
