"""Controller-side semantics of distributed tensors: the scenarios of the reference's
python/tests/test_controller.py on a 2x2 CPU mesh."""
import re

import pytest
import torch

from monarch_b200 import tensor_engine as te
from monarch_b200.actor import this_host


@pytest.fixture(scope="module")
def mesh():
    pm = this_host().spawn_procs(per_host={"gpus": 4})
    m = te.spawn_tensor_engine(pm, use_cuda=False).split(gpus=("host", "gpu"), gpu=2)
    yield m
    m.exit()
    pm.stop().get()


def test_mutation_while_borrowed(mesh):
    """test_mutate / test_dropped_trace: the origin may not write a borrowed tensor, a
    read-only borrow may not be written through, a dropped borrow names where it went."""
    with mesh.activate():
        x = torch.rand(3, 4)
        x.abs_()
        s = te.Stream("other")
        b, drop = s.borrow(x)
        with pytest.raises(te.BorrowError, match="would be mutated"):
            x.abs_()
        with s.activate():
            _ = b.add(b)
            with pytest.raises(te.BorrowError, match="read-only borrow"):
                b.abs_()
        drop.drop()
        x.abs_()
        b, drop = s.borrow(x, mutable=True)
        with s.activate():
            b.abs_()
        drop.drop()
        x.abs_()
        te.inspect(x)
        with s.activate():
            with pytest.raises(te.BorrowError) as ei:
                b + 1                      # the message survives operator forms too
        assert re.match(".*tensor.*is dropped at.*drop.drop().*", str(ei.value), flags=re.DOTALL)


def test_movement_between_sub_meshes(mesh):
    """test_movement, test_to_mesh_stream, test_to_mesh_cow, test_to_mesh_aliasing."""
    sm0, sm1 = mesh.slice(host=0), mesh.slice(host=1)
    with sm0.activate():
        x = torch.rand(3, 4)
        moved = x.to_mesh(sm1)
        want = te.inspect(x, gpu=1)
    with sm1.activate():
        assert torch.equal(te.inspect(moved, gpu=1), want)
    with mesh.activate():
        a = torch.rand(3, 4)
        b = a.slice_mesh(host=0)
        _ = b.to_mesh(sm0)
        c = b.to_mesh(sm1)
    with sm1.activate():
        te.inspect(c)
    other = te.Stream("other")
    with sm0.activate():
        t2 = torch.rand(3, 4).to_mesh(sm1, stream=other)
    with sm1.activate(), other.activate():
        te.inspect(t2 + t2)
    with mesh.activate():                  # to the same mesh: a value of its own
        t = torch.zeros(())
        same = t.to_mesh(mesh)
        t.add_(1)
        assert te.inspect(same).item() == 0 and te.inspect(t).item() == 1
    p2p = te.Stream("p2p_stream")
    ppmesh = mesh.flatten("all").split(all=("dp", "pp"), pp=2)
    stages = [ppmesh.slice(pp=i) for i in range(2)]
    with stages[0].activate():
        x = torch.randn(3, 3)
        xb, x_borrow = p2p.borrow(x)
        with p2p.activate():
            y_p2p = xb.to_mesh(stages[1])
    with stages[1].activate():
        x_borrow.drop()
        y, y_borrow = te.get_active_stream().borrow(y_p2p)
        te.inspect(y)
        y_borrow.drop()


def test_to_mesh_broadcasts_along_missing_dims(mesh):
    """test_broadcast_one / test_broadcast_two: from a slice to the whole mesh."""
    for dim in ("host", "gpu"):
        subset = mesh.slice(**{dim: 1})
        with subset.activate():
            x = torch.rand(3)
            y = x.to_mesh(mesh)
            a = te.inspect(x)
        with mesh.activate():
            b = te.inspect(y.reduce(dim, reduction="stack"))
        assert torch.equal(a.expand(2, -1), b)
    one = mesh.slice(host=1, gpu=1)
    with one.activate():
        x = torch.rand(3)
        y = x.to_mesh(mesh)
        a = te.inspect(x)
    with mesh.activate():
        b = te.inspect(y.reduce("host", reduction="stack").reduce("gpu", reduction="stack"))
    assert torch.equal(a.expand(2, 2, -1), b)
    with pytest.raises(ValueError, match="different sizes"):
        with mesh.slice(gpu=0).activate():
            torch.rand(3).to_mesh(mesh.flatten("all"))


def test_autograd_over_meshes(mesh):
    """test_autograd, test_mesh_semantics, test_autograd_multi_mesh."""
    from monarch_b200.gradient_generator import grad_function, grad_generator
    with mesh.activate():
        x = torch.rand(3, 4, requires_grad=True)
        y = torch.rand(4, 3, requires_grad=True)
        z = torch.rand(3, requires_grad=True)
        foo = (x @ y + z).sum()
    with te.no_mesh():                     # backward runs on the meshes of the forward
        grads = list(grad_generator(foo, [z, y, x]))
    with mesh.activate():
        assert [tuple(te.fetch_shard(g).get(timeout=60).shape) for g in grads] == \
            [(3,), (4, 3), (3, 4)]

    host0, host1 = mesh.slice(host=0), mesh.slice(host=1)
    with host0.activate():
        x = torch.randn(5)
    y = x * 5                              # tensors carry their mesh: no activation needed
    with host1.activate():
        a = torch.randn(5)
        b = a * 5
        x.cos()                            # a tensor of another mesh computes on its own
    y.cos()
    with host1.activate():
        te.inspect(b.cos())

    @grad_function
    def to_mesh(t, m):
        origin = t.mesh

        def backward(grad_t):
            return grad_t.to_mesh(origin), None

        return t.to_mesh(m), backward

    with host0.activate():
        x = torch.rand(3, 4, requires_grad=True)
        y = torch.rand(4, 3, requires_grad=True)
        t = to_mesh(x @ y, host1)
    with host1.activate():
        z = torch.rand(3, requires_grad=True)
        foo = (t + z).sum()
    meshes = []
    for r in grad_generator(foo, [z, y, x]):
        with r.mesh.activate():
            te.fetch_shard(r).get(timeout=60)
        meshes.append(r.mesh._ndslice)
    assert meshes == [host1._ndslice, host0._ndslice, host0._ndslice]


def test_generator_states(mesh):
    """test_random_state: states are values; per-rank seeds give per-rank streams."""
    from monarch_b200 import random as mrandom
    assert mesh.size(["host", "gpu"]) == 4
    with mesh.activate():
        mrandom.make_deterministic()
        a = mrandom.get_state()
        te.inspect(a)
        first = torch.rand(1)
        mrandom.set_state(a)
        second = torch.rand(1)
        f, s = te.inspect((first, second))
        assert torch.equal(f, s)
        seed = mesh.rank(["host", "gpu"]) + 4
        s2, s3 = mrandom.new_state(seed), mrandom.new_state(seed)
        draws = []
        for state in (s2, s3):
            mrandom.set_state(state)
            r = torch.rand(1)
            for d in ("host", "gpu"):
                r = r.reduce(d, reduction="stack")
            draws.append(te.inspect(r))
        mrandom.set_state(a)
        assert torch.equal(te.inspect(torch.rand(1)), f)      # new_state disturbed nothing
    assert torch.equal(draws[0], draws[1])
    assert draws[0].flatten().unique().numel() == 4           # every rank its own numbers


def test_trees_of_tensors(mesh):
    """test_reduce_pytree, test_to_mesh_pytree, test_slice_mesh_pytree, test_torch_tensor,
    test_torch_op_with_optional_tensors."""
    with mesh.activate():
        assert te.inspect(torch.tensor([1, 2, 4])).tolist() == [1, 2, 4]
        x = torch.rand(3, 4)
        te.inspect(torch.nn.LayerNorm(4, bias=True, elementwise_affine=True)(x))
        te.inspect(torch.nn.LayerNorm(4, bias=False, elementwise_affine=False)(x))
        d = {"a": mesh.rank(("gpu", "host")) + torch.zeros((1,)),
             "b": mesh.rank(("gpu", "host")) + torch.ones((1,))}
        _ = te.reduce_(d, dims=("gpu", "host"), reduction="sum")
        r = te.reduce(d, dims=("gpu", "host"), reduction="sum")
        got = [te.inspect(t).item() for t in (d["a"], d["b"], r["a"], r["b"])]
    assert got == [6.0, 10.0, 24.0, 40.0]
    host0, host1 = mesh.slice(host=0), mesh.slice(host=1)
    with host0.activate():
        moved = te.to_mesh({"a": torch.zeros((1,)), "b": torch.ones((1,))}, host1)
    with host1.activate():
        moved["a"].add_(1)
        moved["b"].add_(1)
        assert (te.inspect(moved["a"]).item(), te.inspect(moved["b"]).item()) == (1.0, 2.0)
    with mesh.activate():
        d = {"a": mesh.rank("host") + torch.zeros((1,)), "b": mesh.rank("host") + torch.ones((1,))}
        parts = [te.slice_mesh(d, host=h) for h in range(2)]
    for h, sub, want in ((0, host0, (0.0, 2.0)), (1, host1, (2.0, 4.0))):
        t = te.to_mesh(parts[h], sub)
        with sub.activate():
            _ = te.reduce_(t, dims=("gpu",), reduction="sum")
            assert (te.inspect(t["a"]).item(), te.inspect(t["b"]).item()) == want


def test_argument_errors_are_raised_on_the_controller(mesh):
    """test_errors, test_sub_mesh_process_grop, test_dim1_mesh, test_fetch."""
    import itertools
    with mesh.activate():
        y = torch.rand(3, 4)
        with pytest.raises(ValueError, match="WRONG_MESH"):
            with mesh.slice(host=0).activate():
                torch.rand(3, 4) + y
        other = te.Stream("other")
        t = torch.rand(10)
        with pytest.raises(TypeError, match="WRONG_STREAM"):
            with other.activate():
                t.reduce("host", "sum")
        h, g = mesh.rank("host"), mesh.rank("gpu")
        for hi, gi in itertools.product(range(2), range(2)):
            a, b = te.fetch_shard((h, g), {"host": hi, "gpu": gi}).get(timeout=60)
            assert (a.item(), b.item()) == (hi, gi)
    h0 = mesh.slice(host=0)
    assert h0.process_group(("gpu",)) != h0.process_group(("gpu",))
    with mesh.split(host=("oh", "ih"), ih=1).activate():       # a dim of size one
        got = te.inspect(torch.ones(3, 4))
    assert torch.equal(got, torch.ones(3, 4))


def test_reduce_forms(mesh):
    """test_reduce and test_reduce_out."""
    import itertools
    with mesh.activate():
        x = 24 * mesh.rank("host") + 12 * mesh.rank("gpu") + torch.arange(12).reshape(3, 4)
        y = x.reduce("gpu", "sum")
        g = x.reduce("gpu", "stack")
        with pytest.raises(TypeError, match="When scattering"):
            x.reduce("gpu", "sum", scatter=True)
        x = x.reshape(2, 6)
        all_to_all = x.reduce("gpu", "stack", scatter=True)
        reduce_scatter = x.reduce("gpu", "sum", scatter=True)
        every = x.reduce((), "sum")                             # () is every dim
        every_named = x.reduce(("gpu", "host"), "sum")
        for kw in ({"reduction": "sum", "scatter": True}, {"reduction": "stack"},
                   {"reduction": "stack", "scatter": True}):
            with pytest.raises(ValueError, match="is not valid for multiple dimensions"):
                x.reduce((), **kw)
        yl, gl, el, enl = (te.inspect(t) for t in (y, g, every, every_named))
        assert te.inspect(all_to_all).shape == (2, 6) and te.inspect(reduce_scatter).shape == (6,)
    xs = {(h, g): 24 * h + 12 * g + torch.arange(12).reshape(3, 4)
          for h, g in itertools.product(range(2), range(2))}
    assert torch.equal(yl, xs[0, 0] + xs[0, 1])
    assert torch.equal(gl, torch.stack([xs[0, 0], xs[0, 1]]))
    total = sum(xs.values()).reshape(el.shape)
    assert torch.equal(el, total) and torch.equal(enl, total)
    split = mesh.split(host=("oh", "ih"), ih=1)
    with split.activate():
        x = 24 * split.rank("oh") + 12 * split.rank("gpu") + torch.arange(12).reshape(3, 4)
        inner = te.inspect(x.reduce(("ih", "gpu"), "sum"))
        outer = te.inspect(x.reduce(("oh", "gpu"), "sum"))
    assert torch.equal(inner, xs[0, 0] + xs[0, 1]) and torch.equal(outer, total.reshape(3, 4))

    with mesh.activate():
        inp, wrong, out = torch.rand(2, 4), torch.rand(2, 4), torch.rand(4)
        with pytest.raises(ValueError, match="Reduce expects the shape to be"):
            inp.reduce("host", reduction="sum", scatter=True, out=wrong)
        fresh = inp.reduce("host", reduction="sum", scatter=True)
        before, want = te.inspect(out), te.inspect(fresh)
        into = inp.reduce("host", reduction="sum", scatter=True, out=out)
        assert into is out
        after = te.inspect(out)
    assert not torch.equal(before, want) and torch.equal(after, want)
