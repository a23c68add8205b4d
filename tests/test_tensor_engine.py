"""Distributed tensors driven from one controller: op dispatch, shape propagation, rank
tensors, collectives (reduce variants over mesh dims), remote functions, error poisoning,
coalescing, streams/borrows.  CPU ranks with gloo.  Modelled on the reference's
test_tensor_engine.py / test_remote_functions.py / test_coalescing.py."""
import pytest
import torch

from monarch_b200 import tensor_engine as te
from monarch_b200.actor import this_host


@pytest.fixture(scope="module")
def dm():
    pm = this_host().spawn_procs(per_host={"gpus": 4})
    mesh = te.spawn_tensor_engine(pm, use_cuda=False)
    yield mesh.split(gpus=("host", "gpu"), gpu=2)
    mesh.exit()
    pm.stop().get()


def test_ops_are_dispatched_and_fetched(dm):
    with dm.activate():
        a = torch.ones(3, 4)
        b = 2 * a + 1
        assert isinstance(b, te.Tensor) and b.shape == (3, 4) and b.dtype == torch.float32
        assert te.inspect(b).tolist() == [[3.0] * 4] * 3
        c = (b @ b.t()).sum()
        assert c.shape == () and te.inspect(c).item() == 9 * 4 * 9
        b.add_(1)                      # in-place ops alias their input
        assert te.inspect(b)[0, 0].item() == 4
        assert te.fetch_shard(b, host=1, gpu=1).get()[0, 0].item() == 4


def test_rank_tensors_and_mesh_reshaping(dm):
    assert dm.sizes == {"hosts": 1, "host": 2, "gpu": 2}
    with dm.activate():
        r = dm.rank("host") * 10 + dm.rank("gpu")
        got = [[te.inspect(r, host=h, gpu=g).item() for g in range(2)] for h in range(2)]
        assert got == [[0, 1], [10, 11]]
    flat = dm.flatten("all")
    with flat.activate():
        assert te.inspect(flat.rank("all"), all=3).item() == 3


def test_reduce_variants(dm):
    with dm.activate():
        x = (dm.rank("host") * 2 + dm.rank("gpu") + 1).to(torch.float32) * torch.ones(2, 3)
        assert te.inspect(x.reduce("gpu", "sum"), host=1)[0, 0].item() == 3 + 4
        assert te.inspect(x.reduce(("host", "gpu"), "sum"))[0, 0].item() == 10
        assert te.inspect(x.reduce("host", "max"), gpu=1)[0, 0].item() == 4
        assert te.inspect(x.reduce("gpu", "avg"), host=0)[0, 0].item() == 1.5
        st = x.reduce("gpu", "stack")           # all-gather adds an outer dim
        assert st.shape == (2, 2, 3)
        assert te.inspect(st, host=1)[:, 0, 0].tolist() == [3.0, 4.0]
        rs = x.reduce("gpu", "sum", scatter=True)  # reduce-scatter keeps slice i on member i
        assert rs.shape == (3,) and te.inspect(rs, host=0, gpu=1).tolist() == [3.0] * 3
        a2a = x.reduce("gpu", "stack", scatter=True)
        assert a2a.shape == (2, 3)
        assert te.inspect(a2a, host=0, gpu=0)[:, 0].tolist() == [1.0, 2.0]
        y = x.clone()
        y.reduce_("gpu", "sum")
        assert te.inspect(y, host=0)[0, 0].item() == 3
        with pytest.raises(ValueError):
            torch.ones(5).reduce("gpu", "sum", scatter=True)
        with pytest.raises(KeyError):
            x.reduce("nope", "sum")


def test_remote_functions_and_errors(dm):
    @te.remote(propagate=lambda x, k: x.sum(0))
    def colsum(x, k):
        return x.sum(0) * k

    @te.remote(propagate=lambda x: x)
    def nope(x):
        raise ValueError("nope")

    with dm.activate():
        a = torch.ones(4, 2)
        assert te.inspect(colsum(a, 3)).tolist() == [12.0, 12.0]
        bad = nope(a)
        worse = bad * 2 + 1              # dependants inherit the failure
        with pytest.raises(te.RemoteException, match="nope") as ei:
            te.inspect(worse)
        assert ei.value.dependent_of is not None and "ValueError" in ei.value.exc_text
        # the workers stay alive and later commands work
        assert te.inspect(a.sum()).item() == 8
        got = te.call_on_shard_and_fetch(lambda t: t.shape, a, shard={"host": 1}).get()
        assert tuple(got) == (4, 2)


def test_controller_history_tracks_failures_and_progress(dm):
    """The native controller history learns of a failure from the error port and poisons,
    on the controller's books, the failed command's results, the commands already issued
    that read them, and commands issued later -- no round trip to the workers."""
    import time

    @te.remote(propagate=lambda x: x)
    def boom(x):
        raise ValueError("boom")

    client = dm.client
    with dm.activate():
        a = torch.ones(3)
        good = a + 1
        bad = boom(a)
        dep = bad * 2                     # issued before the failure is known
        te.inspect(good)                  # the workers have passed `boom` by now
        deadline = time.monotonic() + 10
        while client.known_failure(bad) is None and time.monotonic() < deadline:
            time.sleep(0.01)
        f = client.known_failure(bad)
        assert f is not None and "boom" in f.exc_text
        assert client.known_failure(dep) is not None          # forward pass over live commands
        later = dep - 1                                           # issued after: inherits at once
        assert client.history.ref_failed(later.ref) == client.history.ref_failed(bad.ref)
        assert client.known_failure(good) is None
        # deleting the tensors forgets their poison
        ref = bad.ref
        del bad, dep, later
        client.flush()
        client._send_deletes()
        assert client.history.ref_failed(ref) == -1
    # progress: a ping answered by every rank retires what they have passed
    h = client.history
    before = h.live_invocations()
    client._last_ping = -1e9
    client.operation_timeout, saved = 60.0, client.operation_timeout
    try:
        deadline = time.monotonic() + 10
        client._watch()
        while client._ping is not None and time.monotonic() < deadline:
            time.sleep(0.01)
            client._watch()
    finally:
        client.operation_timeout = saved
    assert client._ping is None and h.min_completed() > 0
    assert h.live_invocations() < max(before, 1)


def test_remote_inspect_propagation(dm):
    @te.remote(propagate="inspect")
    def weird(x):
        return torch.zeros(x.shape[0] + 1, 2, dtype=torch.float64)

    with dm.activate():
        out = weird(torch.ones(3))
        assert out.shape == (4, 2) and out.dtype == torch.float64


def test_coalescing_batches_messages(dm):
    from monarch_b200 import _native as N
    with dm.activate():
        warm = torch.ones(2) + 1
        te.inspect(warm)
        before = N.metrics_counter("cast.messages")
        with te.coalescing():
            x = torch.ones(8)
            for _ in range(20):
                x = x + 1
        sent = N.metrics_counter("cast.messages") - before
        assert sent <= 2, sent            # one cast for the whole block
        assert te.inspect(x)[0].item() == 21


def test_streams_and_borrows(dm):
    comm = te.Stream("comm")
    with dm.activate():
        x = torch.ones(4)
        y, borrow = comm.borrow(x, mutable=True)
        with pytest.raises(RuntimeError, match="borrowed"):
            x + 1                          # origin stream may not touch it meanwhile
        with comm.activate():
            y.add_(2)
        borrow.drop()
        assert te.inspect(x)[0].item() == 3
        with pytest.raises(RuntimeError, match="dropped"):
            y + 1


def test_slice_mesh_and_to_mesh(dm):
    with dm.activate():
        f = (dm.rank("host") * 2 + dm.rank("gpu")).to(torch.float32) * 10
    top = dm.slice(host=0)
    bottom = dm.slice(host=1)
    with bottom.activate():
        moved = f.slice_mesh(host=0).to_mesh(bottom)
        assert te.inspect(moved + 1, gpu=1).item() == 11
    with top.activate():
        assert te.inspect(f.slice_mesh(host=0), gpu=0).item() == 0


def test_no_mesh_escapes_dispatch(dm):
    with dm.activate():
        with te.no_mesh():
            local = torch.ones(2) * 3
        assert not isinstance(local, te.Tensor) and local.tolist() == [3.0, 3.0]


def test_compile_records_once_and_replays(dm):
    calls = []

    @te.compile
    def step(w, x, scale):
        calls.append(1)
        h = (x @ w).relu()
        w.add_(h.sum(0, keepdim=True).t().expand_as(w) * scale)
        return h.sum(), h

    with dm.activate():
        w = torch.ones(3, 3)
        x = torch.arange(6, dtype=torch.float32).reshape(2, 3)
        with te.no_mesh():
            ref_w = torch.ones(3, 3)
            ref_x = torch.arange(6, dtype=torch.float32).reshape(2, 3)
        for it in range(3):
            s, h = step(w, x, 0.5)
            with te.no_mesh():
                ref_h = (ref_x @ ref_w).relu()
                ref_w = ref_w + ref_h.sum(0, keepdim=True).t().expand_as(ref_w) * 0.5
            assert te.inspect(s).item() == ref_h.sum().item(), it
            assert torch.equal(te.inspect(h), ref_h)
        assert torch.equal(te.inspect(w), ref_w)
        assert len(calls) == 1          # traced once, replayed twice
        step(w, torch.ones(4, 3), 0.5)  # new input shape -> new trace
        assert len(calls) == 2


# ------------------------------------------------------------------------------- pipes --
def _counting_loader(pipe, n, width):
    """Worker side of a pipe: a generator; each worker yields batches marked with its
    coordinates."""
    tag = pipe.ranks["host"] * 10 + pipe.ranks["gpu"]
    for i in range(n):
        yield {"x": torch.full((2, width), float(tag + 100 * i)), "i": torch.tensor(i)}


def _echo_loader(pipe):
    """Worker side that talks back: doubles whatever the controller sends."""
    while True:
        v = pipe.recv()
        pipe.send(v["t"] * 2 + v["k"])


def _broken_loader(pipe):
    yield torch.zeros(1)
    raise ValueError("loader broke")


def test_pipe_generator_feeds_distributed_tensors(dm):
    @te.remote_generator(_counting_loader, max_messages=2)
    def loader(pipe, n, width):
        for _ in range(n):
            yield {"x": torch.zeros(2, width), "i": torch.tensor(0)}

    with dm.activate():
        p = loader(3, 5)
        b0 = p.recv()
        b1 = p.recv()
        assert isinstance(b0["x"], te.Tensor) and b0["x"].shape == (2, 5)
        assert te.inspect(b0["x"], host=1, gpu=1)[0, 0].item() == 11
        assert te.inspect(b1["x"], host=0, gpu=1)[1, 4].item() == 101
        assert te.inspect(b1["i"]).item() == 1
        s = (b0["x"] + b1["x"]).reduce(("host", "gpu"), "sum")   # usable like any tensor
        assert te.inspect(s)[0, 0].item() == (0 + 1 + 10 + 11) * 2 + 400
        p.recv()
        with pytest.raises(StopIteration):
            p.recv()          # the propagation generator ends with the worker's


def test_pipe_send_reaches_the_generator(dm):
    @te.remote_generator(_echo_loader)
    def echo(pipe):
        while True:
            v = pipe.recv()
            yield v["t"] * 2 + v["k"]

    with dm.activate():
        p = echo()
        t = dm.rank("gpu").to(torch.float32) * torch.ones(3)
        p.send({"t": t, "k": 5})
        out = p.recv()
        assert out.shape == (3,)
        assert te.inspect(out, host=0, gpu=1).tolist() == [7.0] * 3
        p.drop()


def test_pipe_failure_poisons_the_received_tensors(dm):
    @te.remote_generator(_broken_loader)
    def broken(pipe):
        while True:
            yield torch.zeros(1)

    with dm.activate():
        p = broken()
        ok = p.recv()
        assert te.inspect(ok).item() == 0
        bad = p.recv()
        with pytest.raises(te.RemoteException, match="loader broke"):
            te.inspect(bad)
        assert te.inspect(ok + 1).item() == 1     # workers stay alive


# ---------------------------------------------------------------------------- watchdog --
def _sleep_on(rank_t, which, seconds):
    import time
    if int(rank_t.item()) == which:
        time.sleep(seconds)
    return rank_t + 0


def test_progress_watchdog_names_the_stuck_ranks(dm):
    client = dm.client
    saved = (client.operation_timeout, client.progress_interval, client.fail_on_worker_timeout)
    client.operation_timeout, client.progress_interval = 0.8, 0.1
    sleepy = te.remote(_sleep_on, propagate=lambda t, w, s: t)
    flat = dm.flatten("all")
    try:
        with flat.activate():
            r = flat.rank("all")
            n0 = len(client.stalls)
            out = sleepy(r, 2, 3.0)
            assert te.inspect(out, all=2).item() == 2          # waits through the stall
            assert len(client.stalls) == n0 + 1
            assert client.stalls[-1]["ranks"] == [2]
            # with fail_on_worker_timeout the wait itself raises, naming the ranks
            client.fail_on_worker_timeout = True
            out = sleepy(r, 1, 3.0)
            with pytest.raises(te.WorkerTimeoutError) as ei:
                te.inspect(out, all=1)
            assert ei.value.ranks == [1]
    finally:
        client._failed = None
        client.operation_timeout, client.progress_interval, client.fail_on_worker_timeout = saved
    import time
    time.sleep(3.0)     # let the sleeper finish before the fixture tears the mesh down
    with flat.activate():
        assert te.inspect(flat.rank("all") + 1, all=3).item() == 4


# ------------------------------------------------------------------- process groups ----
def _hand_written_allreduce(t, pg):
    import torch.distributed as dist
    out = t.clone()
    dist.all_reduce(out, group=pg)
    return out * dist.get_world_size(pg)


def test_remote_process_group_in_a_remote_function(dm):
    fn = te.remote(_hand_written_allreduce, propagate=lambda t, pg: t)
    with dm.activate():
        pg = dm.process_group("gpu")
        assert pg.size() == 2 and isinstance(pg, te.RemoteProcessGroup)
        x = (dm.rank("host") * 2 + dm.rank("gpu") + 1).to(torch.float32) * torch.ones(3)
        y = fn(x, pg)
        # host 0 holds 1 and 2, host 1 holds 3 and 4; summed over "gpu", times group size 2
        assert te.inspect(y, host=0, gpu=1).tolist() == [6.0] * 3
        assert te.inspect(y, host=1, gpu=0).tolist() == [14.0] * 3
        with pytest.raises(KeyError):
            dm.process_group("nope")


def test_coalescing_keeps_program_order_across_meshes(dm):
    """A block that alternates between the whole mesh and a sub-mesh is sent as runs of
    consecutive messages, so a sub-mesh read sits between the two whole-mesh writes it was
    written between."""
    sub = dm.slice(host=0)
    with dm.activate():
        a = torch.ones(3)
        with te.coalescing():
            a.add_(10)                      # whole mesh
            b = a.slice_mesh(host=0)        # same data, seen from the sub-mesh
            with sub.activate():
                c = b + 0                   # sub-mesh read: must see 11
            a.add_(10)                      # whole mesh again
        assert te.inspect(c, gpu=1).tolist() == [11.0] * 3
        assert te.inspect(a, host=0, gpu=0).tolist() == [21.0] * 3


def test_reading_values_on_the_controller_is_a_clear_error(dm):
    with dm.activate():
        t = torch.ones(3)
        with pytest.raises(RuntimeError, match="fetch_shard"):
            t.sum().item()
        with pytest.raises(RuntimeError, match="fetch_shard"):
            bool(t.sum() > 2)
        assert te.inspect(t.sum()).item() == 3.0      # the way to do it


# ------------------------------------------- compile scenarios of the reference's tests --
def _bogus_matmul(x, y):
    return x @ y


def test_compiled_blocks_with_closures_formals_errors_and_borrows(dm):
    """python/tests/test_coalescing.py of the reference: repeat_simple, repeat_formals,
    repeat_error_inside, repeat_inner_borrow, nested_coalescing."""
    with dm.activate():
        a = torch.zeros(())

        @te.compile
        def bump():
            nonlocal a
            z = torch.ones(())
            a += z                       # a tensor of the enclosing scope, mutated in place
            return z

        z = None
        for _ in range(3):
            z = bump()
        assert te.inspect(a).item() == 3 and te.inspect(z).item() == 1

        w = torch.rand(3, 4)

        @te.compile
        def affine(p, q):
            return 2 * p + q

        @te.compile
        def affine_closed(q):
            return 2 * w + q

        for fn, args in ((affine, (w,)), (affine_closed, ())):
            for _ in range(3):
                q = torch.rand(3, 4)
                lz, lw, lq = te.inspect((fn(*args, q), w, q))
                assert torch.allclose(lz, 2 * lw + lq)

        bogus = te.remote(_bogus_matmul, propagate=lambda x, y: x)

        @te.compile
        def broken():
            s = torch.ones(())
            return bogus(s, s)           # fails on the workers, inside the recording

        with pytest.raises(te.RemoteException):
            te.inspect(broken())
        assert te.inspect(a).item() == 3          # the workers carry on

        other = te.Stream("other_for_compile")
        with other.activate():
            b = torch.ones(())
        acc = torch.zeros(())

        @te.compile
        def add_borrowed():
            nonlocal acc
            c, borrow = te.get_active_stream().borrow(b)
            with borrow:
                acc += c

        for _ in range(3):
            add_borrowed()
        assert te.inspect(acc).item() == 3

        with te.coalescing():
            t = torch.zeros(3, 4)
            with te.coalescing():
                for _ in range(9):
                    t = t + torch.ones(3, 4)
        assert te.inspect(t)[0, 0].item() == 9


# ------------------------- hand-written collectives in remote functions (reference tests) --
def _udf_all_reduce(t, group=None):
    import torch.distributed as dist
    out = t.clone()
    dist.all_reduce(out, group=group)
    return out


def _udf_barrier(group=None):
    import torch.distributed as dist
    dist.barrier(group=group)
    return torch.ones(())


def _append_processed(s):
    return s + " processed"


def test_process_groups_over_dims_and_sub_meshes(dm):
    """python/tests/test_remote_functions.py of the reference: comms_full_mesh,
    comms_by_dimension, comms_sub_mesh, barrier, fetch_preprocess."""
    all_reduce = te.remote(_udf_all_reduce, propagate=lambda t, group=None: t)
    barrier = te.remote(_udf_barrier, propagate=lambda group=None: torch.ones(()))

    def myrank():
        return (dm.rank("host") + 1) * 2 + dm.rank("gpu") + 1       # 3 4 / 5 6

    with dm.activate():
        x = torch.ones((3, 4)) * myrank()
        full = all_reduce(x, group=dm.process_group(("host", "gpu")))
        got = te.fetch_shard(full).get(timeout=60)
        assert got.shape == (3, 4) and got.eq(18).all().item()
        by_gpu = all_reduce(x, group=dm.process_group(("gpu",)))
        assert te.fetch_shard(by_gpu).get(timeout=60)[0, 0].item() == 7
        assert te.fetch_shard(by_gpu, host=1, gpu=1).get(timeout=60)[0, 0].item() == 11
        by_host = all_reduce(x, group=dm.process_group(("host",)))
        assert te.fetch_shard(by_host).get(timeout=60)[0, 0].item() == 8
        assert te.fetch_shard(by_host, host=0, gpu=1).get(timeout=60)[0, 0].item() == 10
        # the worker function itself can serve as the shape rule: on fakes the group is a
        # stand-in whose collectives do nothing
        itself = te.remote(_udf_all_reduce, propagate=_udf_all_reduce)
        again = itself(x, group=dm.process_group(("host", "gpu")))
        assert te.fetch_shard(again).get(timeout=60)[0, 0].item() == 18
        done = barrier(group=dm.process_group(("host", "gpu")))
        assert te.fetch_shard(done).get(timeout=60).item() == 1.0
        assert te.call_on_shard_and_fetch(te.remote(_append_processed),
                                          "an argument").get(timeout=30) == "an argument processed"
    # a part of the mesh: the parent's rank tensors and process groups serve it
    for h, expect in ((1, 11), (0, 7)):
        with dm.slice(host=h).activate():
            x = torch.ones((3, 4)) * myrank()
            r = all_reduce(x, group=dm.process_group(("gpu",)))
            assert te.fetch_shard(r).get(timeout=60)[0, 0].item() == expect


def _udf_mutating_prop(t, *args, **kwargs):
    t.add_(1)          # "the worker function writes its first argument"
    return t


def _udf_broadcast(tensor, src=None, group=None):
    import torch.distributed as dist
    dist.broadcast(tensor, src=src, group=group)
    return tensor


def _udf_all_to_all_single(out, inp, group=None):
    import torch.distributed as dist
    dist.all_to_all_single(out, inp, group=group)
    return out


def _udf_all_gather(tensor_list, tensor, group=None):
    import torch.distributed as dist
    dist.all_gather(tensor_list, tensor, group=group)
    return tensor_list


def _udf_reduce_scatter_tensor(out, inp, group=None):
    import torch.distributed as dist
    dist.reduce_scatter_tensor(out, inp, group=group)
    return out


def _udf_inner_that_fails():
    raise Exception("Failed to execute the inner function")


def _udf_outer_that_calls_inner():
    _udf_inner_that_fails()
    return torch.zeros(1)


def _udf_returns_exception():
    return Exception("is a valid value to return")


def _udf_fails_in_place(t):
    raise ValueError("cannot fill")


def test_collectives_that_write_their_arguments(dm):
    """Remote functions that change their arguments in place, told by a propagation function
    that does the same to the fakes (reference: test_remote_function_broadcast,
    _all_to_all_single, _all_gather, _reduce_scatter_tensor_sum, test_tensor_dtype_complex,
    _failure_message_contains_traceback, test_return_exception)."""
    import itertools
    broadcast = te.remote(_udf_broadcast, propagate=_udf_mutating_prop)
    a2a_single = te.remote(_udf_all_to_all_single, propagate=_udf_mutating_prop)
    rs_tensor = te.remote(_udf_reduce_scatter_tensor, propagate=_udf_mutating_prop)
    all_gather = te.remote(_udf_all_gather,
                           propagate=lambda tl, *a, **k: [torch.zeros_like(t) for t in tl])
    shards = list(itertools.product(range(2), repeat=2))
    with dm.activate():
        pg = dm.process_group(("host", "gpu"))
        for src in (0, 3):
            rank = 2 * dm.rank("host") + dm.rank("gpu")
            broadcast(rank, src=src, group=pg)                      # result ignored: in place
            assert [te.inspect(rank, host=h, gpu=g).item() for h, g in shards] == [src] * 4
        t_in, t_out = torch.arange(4, dtype=torch.float64), torch.empty(4, dtype=torch.float64)
        a2a_single(t_out, t_in, group=pg)
        for h, g in shards:
            assert te.inspect(t_out, host=h, gpu=g).eq(2 * h + g).all().item()
        rank = 2 * dm.rank("host") + dm.rank("gpu")
        outs = all_gather(list(torch.zeros(8).chunk(4)), rank * torch.ones(2), group=pg)
        assert [x[0].item() for x in te.inspect(outs, host=1, gpu=0)] == [0, 1, 2, 3]
        out = torch.zeros(2, dtype=torch.int64)
        rs_tensor(out, torch.arange(8, dtype=torch.int64), group=pg)
        for h, g in shards:
            r = 2 * h + g
            assert te.inspect(out, host=h, gpu=g).tolist() == [8 * r, 8 * r + 4]
        # complex views pass through the same functions
        t = torch.rand(2)
        tl = [torch.rand(2) for _ in range(4)]
        tl[1] = torch.view_as_complex(tl[1])
        te.inspect(all_gather(tl, torch.view_as_complex(t), group=pg))
        # a failure names the frames of the worker's stack
        x = te.remote(_udf_outer_that_calls_inner, propagate=lambda: torch.zeros(1))()
        with pytest.raises(te.RemoteException) as ei:
            te.inspect(x)
        assert "_udf_outer_that_calls_inner" in str(ei.value)
        assert "_udf_inner_that_fails" in str(ei.value)
        # an exception object is a value like any other
        v = te.call_on_shard_and_fetch(te.remote(_udf_returns_exception)).get(timeout=30)
        assert isinstance(v, Exception)
        # a function that was to write its argument and failed leaves the argument failed
        y = torch.zeros(3)
        te.remote(_udf_fails_in_place, propagate=_udf_mutating_prop)(y)
        with pytest.raises(te.RemoteException, match="cannot fill"):
            te.inspect(y + 1)


def _udf_copies(n, t):
    return [t + i for i in range(n)]


def test_cached_propagation_probes_once_per_signature(dm):
    """python/tests/test_remote_functions.py::test_cached_remote_function of the reference."""
    fn = te.remote(_udf_copies, propagate="cached")
    with dm.activate():
        x, y = torch.ones(3, 4), torch.rand(3, 4)
        a, _, _ = fn(3, x)
        b, _, c = fn(3, x)
        _, _, _ = fn(3, y)              # same shapes and dtype: answered from the table
        t0, t1 = fn(2, x)               # another plain value: probed again
        s = t0 + t1
        assert a.shape == (3, 4) and s.shape == (3, 4)
        assert fn.cache_hits == 2 and len(fn._cache) == 2
        assert te.inspect(a).eq(1.0).all().item() and te.inspect(c).eq(3.0).all().item()
        assert te.inspect(s).eq(3.0).all().item()
        z = fn(1, torch.ones(2, dtype=torch.int64))[0]
        assert z.dtype == torch.int64 and len(fn._cache) == 3


def _udf_fails_on_one_rank(x, y, rank, fail_rank=None):
    if fail_rank is not None and int(rank.item()) != fail_rank:
        return x + y
    return x @ y               # 3x4 @ 3x4: raises


def test_failure_on_one_rank_of_a_distributed_tensor(dm):
    """python/tests/test_remote_functions.py::test_distributed_error of the reference: the
    rank whose input failed still takes part in collectives, fetching any shard of a tensor
    that failed somewhere raises, and unrelated work goes on."""
    bogus = te.remote(_udf_fails_on_one_rank, propagate=lambda x, y, r, fail_rank=None: x + y)
    with dm.activate():
        x, y = torch.rand(3, 4), torch.rand(3, 4)
        rank = dm.rank("host") * 2 + dm.rank("gpu")
        z = bogus(x, y, rank, fail_rank=1)
        a = (x + y).reduce("gpu")
        assert te.fetch_shard(a).get(timeout=60).shape == (3, 4)
        with pytest.raises(te.RemoteException, match="_udf_fails_on_one_rank"):
            te.fetch_shard(z).get(timeout=60)              # shard of rank 0, failure of rank 1
        rz = z.reduce("gpu")                               # rank 1 joins with a stand-in
        with pytest.raises(te.RemoteException, match="_udf_fails_on_one_rank"):
            te.fetch_shard(rz).get(timeout=60)
        ok = te.fetch_shard(2 * x, host=0, gpu=1).get(timeout=60)
        assert ok.shape == (3, 4)
        # the other pair of ranks reduced among themselves, but the tensor as a whole failed
        with pytest.raises(te.RemoteException):
            te.fetch_shard(rz, host=1, gpu=0).get(timeout=60)
        dm.client.drain_errors()


# -------------------------------------------------------- one host thread per stream --
import threading as _threading  # noqa: E402

_GATE = _threading.Event()       # lives in every worker process (this module is imported there)


def _wait_for_gate(x):
    if not _GATE.wait(30):
        raise RuntimeError("nobody opened the gate: the streams share one host thread")
    _GATE.clear()
    return x + 1


def _open_gate(x):
    _GATE.set()
    return x * 2


def test_user_functions_of_two_streams_run_on_separate_host_threads(dm):
    """A function on the main stream blocks on the host until a function on a second
    stream releases it: possible only because every stream has its own OS thread in the
    worker (monarch_tensor_worker/src/stream.rs:542-588 in the reference)."""
    wait = te.remote(_wait_for_gate, propagate=lambda x: x)
    release = te.remote(_open_gate, propagate=lambda x: x)
    side = te.Stream("gatekeeper")
    with dm.activate():
        x = torch.ones(2)
        waited = wait(x)                       # main stream: parks its thread on the host
        after = waited + 1                     # queued behind it on the same stream
        with side.activate():
            z = torch.ones(2)
            opened = release(z)                # side stream: runs meanwhile
            assert te.inspect(opened).tolist() == [2.0, 2.0]
        assert te.inspect(after).tolist() == [3.0, 3.0]


def test_null_device_workers_execute_nothing_but_keep_shapes():
    """The switch that stands in for the reference's mock_cuda: programs run end to end,
    results have the right shapes and dtypes, nothing is computed (values are zeros)."""
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    mesh = te.spawn_tensor_engine(pm, use_cuda=False, null_device=True)
    try:
        with mesh.activate():
            a = torch.ones(3, 4)
            b = (2 * a + 1) @ torch.ones(4, 5, dtype=torch.float64).float()
            got = te.inspect(b, gpus=1)
            assert got.shape == (3, 5) and got.dtype == torch.float32 and got.eq(0).all()
            s = b.reduce("gpus", "stack")
            assert te.inspect(s).shape == (2, 3, 5)
            r = torch.ones(2, 6).reduce("gpus", "sum", scatter=True)
            assert te.inspect(r).shape == (6,)
            side = te.Stream("null-side")
            y, borrow = side.borrow(a)
            with side.activate():
                z = y + 1
                assert te.inspect(z).shape == (3, 4)
            borrow.drop()
    finally:
        mesh.exit()
        pm.stop().get()
