"""The tensor worker's native executor core: operator calls against the ref environment,
error poisoning of dependents, recordings with rebinding and Python fallbacks."""
import pytest
import torch

from monarch_b200.tensor_engine.worker import Ref, _load_core

mod = _load_core()
pytestmark = pytest.mark.skipif(mod is None, reason="native worker core is not built")


def _core():
    return mod.WorkerCore(3, Ref)


def test_call_op_resolves_refs_and_stores_results():
    c = _core()
    c.set(1, torch.arange(6.0).reshape(2, 3))
    c.set(2, torch.ones(3, 2))
    assert c.call_op(10, [3], [], "aten.mm.default", (Ref(1), Ref(2)), {}, 0) is None
    assert torch.equal(c.get(3), torch.arange(6.0).reshape(2, 3) @ torch.ones(3, 2))
    # keyword and scalar arguments, tensor lists, in-place ops
    assert c.call_op(11, [4], [], "aten.add.Tensor", (Ref(3), Ref(3)), {"alpha": 2}, 0) is None
    assert torch.equal(c.get(4), c.get(3) * 3)
    assert c.call_op(12, [5], [], "aten.cat.default", ([Ref(3), Ref(4)], 0), {}, 0) is None
    assert c.get(5).shape == (4, 2)
    assert c.call_op(13, [], [3], "aten.mul_.Scalar", (Ref(3), 0.5), {}, 0) is None
    assert torch.equal(c.get(3), torch.tensor([[1.5, 1.5], [6.0, 6.0]]))
    assert len(c) == 5 and c.live_bytes() > 0
    c.erase([4, 5])
    assert not c.contains(4) and c.pop(99) is None


def test_failures_poison_results_and_dependents():
    c = _core()
    c.set(1, torch.ones(2, 3))
    c.set(2, torch.ones(2, 3))
    err = c.call_op(20, [3], [], "aten.mm.default", (Ref(1), Ref(2)), {}, 0)
    assert err is not None and err[0] == 20 and err[1] == 3 and err[5] == -1
    assert "mm" in err[2] and "RuntimeError" in err[3]
    v = c.get(3)
    assert v[0] == "__remote_error__"
    dep = c.call_op(21, [4], [], "aten.relu.default", (Ref(3),), {}, 0)
    assert dep[5] == 20 and dep[0] == 21          # inherited from seq 20, nothing new
    assert c.get(4)[0] == "__remote_error__"


def test_recording_replays_natively_with_rebinding():
    c = _core()
    msgs = [("call", 1, [Ref(12)], [], ("op", "aten.mul.Tensor"), (Ref(10), Ref(10)), {}, 0),
            ("noop", "python side"),
            ("call", 2, [Ref(13)], [], ("op", "aten.sum.default"), (Ref(12),), {}, 0)]
    c.define_recording(7, msgs)
    assert c.has_recording(7)
    seen = []
    c.set(100, torch.full((3,), 2.0))
    n = c.call_recording(7, {10: 100, 12: 101, 13: 102}, lambda i, b: seen.append((i, b[10])),
                         None)
    assert n == 2 and seen == [(1, 100)]
    assert c.get(102).item() == 12.0 and not c.contains(13)
    c.set(200, torch.full((2,), 3.0))
    c.call_recording(7, {10: 200, 12: 201, 13: 202}, lambda i, b: None, None)
    assert c.get(202).item() == 18.0
