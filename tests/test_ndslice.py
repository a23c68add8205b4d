"""ndslice: slices, shapes, selection grammar, routing (C++ with bindings).
Modelled on the reference's ndslice unit/property tests and python/tests/_monarch/test_ndslice.py."""
import itertools
import pickle
import random

import pytest

from monarch_b200 import _native as N
from monarch_b200.actor.shape import Extent, MeshTrait, Point, Shape


def test_row_major_and_indexing():
    s = N.Slice.new_row_major([2, 3, 4])
    assert s.sizes == [2, 3, 4] and s.strides == [12, 4, 1] and len(s) == 24
    for i, c in enumerate(itertools.product(range(2), range(3), range(4))):
        assert s.nditem(list(c)) == i
        assert s.coordinates(i) == list(c)
        assert s.index(i) == i and s[i] == i
    with pytest.raises(ValueError):
        s.nditem([2, 0, 0])
    with pytest.raises(ValueError):
        s.coordinates(24)


def test_strided_slice_and_select():
    s = N.Slice(1, [2, 3], [6, 2])
    assert s.ranks() == [1, 3, 5, 7, 9, 11]
    assert s.index(9) == 4 and s.coordinates(9) == [1, 1]
    assert not s.contains(2)
    sub = s.select(1, 1, 3, 1)
    assert sub.ranks() == [3, 5, 9, 11]
    assert s.at(0, 1).ranks() == [7, 9, 11]
    with pytest.raises(ValueError):
        N.Slice(0, [2, 2], [1, 1])  # overlapping


def test_from_list_roundtrip():
    for ranks in ([0, 1, 2, 3], [0, 2, 4, 9, 10, 11], [5]):
        got = sorted(r for s in N.Slice.from_list(ranks) for r in s.ranks())
        assert got == sorted(ranks)
    assert N.Slice.from_list([]) == []


def test_pickle_and_eq():
    s = N.Slice(3, [2, 2], [4, 1])
    assert pickle.loads(pickle.dumps(s)) == s
    assert hash(s) == hash(N.Slice(3, [2, 2], [4, 1]))


@pytest.mark.parametrize("text,expected", [
    ("*", list(range(24))),
    ("0", list(range(12))),
    ("1,*,0", [12, 16, 20]),
    ("*,1:3,0:4:2", [4, 6, 8, 10, 16, 18, 20, 22]),
    ("0,0,0|1,2,3", [0, 23]),
    ("*,*,1:3 & *,1,*", [5, 6, 17, 18]),
    ("(0|1),0,0", [0, 12]),
    (":,2:,3", [11, 23]),
])
def test_selection_grammar(text, expected):
    s = N.Slice.new_row_major([2, 3, 4])
    assert N.Selection.from_string(text).eval(s) == expected


def test_selection_errors_and_any():
    s = N.Slice.new_row_major([4, 4])
    with pytest.raises(ValueError):
        N.Selection.from_string("1,,")
    with pytest.raises(ValueError):
        N.Selection.from_string("0:4:0")
    got = N.Selection.from_string("?,?").eval(s)
    assert len(got) == 1 and 0 <= got[0] < 16
    assert N.Selection.from_string("?,?").eval(s) == got  # deterministic for a seed


def _random_selection(rng, dims, depth=0):
    if depth == len(dims):
        return None
    n = dims[depth]
    kind = rng.choice(["all", "idx", "range"])
    if kind == "all":
        head = "*"
    elif kind == "idx":
        head = str(rng.randrange(n))
    else:
        a = rng.randrange(n)
        b = rng.randrange(a, n + 1)
        head = f"{a}:{b}:{rng.choice([1, 2])}"
    rest = _random_selection(rng, dims, depth + 1)
    return head if rest is None else f"{head},{rest}"


def test_routing_delivers_exactly_the_evaluated_set():
    """Property: the cast tree reaches every selected rank exactly once, and nobody else."""
    rng = random.Random(0)
    for _ in range(200):
        dims = [rng.randint(1, 4) for _ in range(rng.randint(1, 4))]
        offset = rng.randint(0, 5)
        base = N.Slice.new_row_major(dims)
        sl = N.Slice(offset, dims, base.strides)
        parts = [_random_selection(rng, dims) for _ in range(rng.randint(1, 3))]
        text = rng.choice(["|", "&"]).join(f"({p})" for p in parts)
        sel = N.Selection.from_string(text)
        want = sel.eval(sl)
        delivered, hops, fanout = N.simulate_cast(sel, sl)
        assert sorted(delivered) == sorted(want), (text, dims)
        assert len(set(delivered)) == len(delivered)
        assert all(h <= len(dims) for h in hops.values())


def test_reshape_with_limit_bounds_fanout():
    sl = N.Slice.new_row_major([64, 3])
    r = N.reshape_with_limit(sl, 8)
    assert sorted(r.ranks()) == sorted(sl.ranks()) and max(r.sizes) <= 8
    _, _, fanout_flat = N.simulate_cast(N.Selection.all(), N.Slice.new_row_major([192]))
    _, hops, fanout = N.simulate_cast(N.Selection.all(), N.reshape_with_limit(
        N.Slice.new_row_major([192]), 8))
    assert fanout_flat == 191 and fanout <= 3 * 7 and max(hops.values()) <= 3


def test_view_and_contiguity():
    s = N.Slice.new_row_major([4, 6])
    v = s.view([2, 2, 6])
    assert v.ranks() == s.ranks()
    assert s.is_contiguous() and not s.select(1, 0, 6, 2).is_contiguous()
    with pytest.raises(ValueError):
        s.view([5, 5])


class _M(MeshTrait):
    def __init__(self, shape):
        self.s = shape

    @property
    def _ndslice(self):
        return self.s.ndslice

    @property
    def _labels(self):
        return tuple(self.s.labels)

    def _new_with_shape(self, shape):
        return _M(shape)


def test_mesh_trait_slice_split_flatten_rename():
    m = _M(Shape(["host", "gpu"], N.Slice.new_row_major([4, 8])))
    assert m.size() == 32 and m.size("gpu") == 8 and m.sizes == {"host": 4, "gpu": 8}
    a = m.slice(host=1)
    assert a._labels == ("gpu",) and a._ndslice.ranks() == list(range(8, 16))
    b = m.slice(gpu=slice(2, 6))
    assert b.sizes == {"host": 4, "gpu": 4} and b._ndslice.ranks()[:4] == [2, 3, 4, 5]
    sp = m.split(host=("dp", "pp"), gpu=("tp",), pp=2)
    assert sp.sizes == {"dp": 2, "pp": 2, "tp": 8} and sp._ndslice.ranks() == list(range(32))
    assert sp.slice(dp=1, pp=0)._ndslice.ranks() == list(range(16, 24))
    assert m.rename(host="dp")._labels == ("dp", "gpu")
    assert m.flatten("all").sizes == {"all": 32}
    with pytest.raises(ValueError):
        b.flatten("x")
    with pytest.raises(ValueError):
        m.split(host=("a", "b"))
    with pytest.raises(ValueError):
        m.split(host=("a", "b"), a=3)
    with pytest.raises(KeyError):
        m.size("nope")


def test_point_and_extent():
    ext = Extent(["hosts", "gpus"], [1, 2])
    p = Point(1, ext)
    assert p["gpus"] == 1 and p["hosts"] == 0 and p.rank == 1 and p.size("gpus") == 2
    assert str(p) == "{'hosts': 0/1, 'gpus': 1/2}"
    assert dict(p) == {"hosts": 0, "gpus": 1}
    assert pickle.loads(pickle.dumps(p)) == p
    with pytest.raises(ValueError):
        Point(2, ext)


def test_shape_at_and_select_follow_the_reference_vectors():
    """Golden values of the reference's shape tests (python/tests/test_actor_shape.py)."""
    from monarch_b200.actor.shape import Shape
    sh = Shape(["batch", "height", "width"], N.Slice(0, [2, 3, 4], [12, 4, 1]))
    r = sh.at("batch", 1)
    assert (r.labels, list(r.ndslice.sizes), list(r.ndslice.strides), r.ndslice.offset) == \
        (["height", "width"], [3, 4], [4, 1], 12)
    r = sh.at("height", 2)
    assert (r.labels, list(r.ndslice.sizes), list(r.ndslice.strides), r.ndslice.offset) == \
        (["batch", "width"], [2, 4], [12, 1], 8)
    r = sh.at("width", 3)
    assert (list(r.ndslice.sizes), list(r.ndslice.strides), r.ndslice.offset) == ([2, 3], [12, 4], 3)
    rc = Shape(["rows", "cols"], N.Slice.new_row_major([4, 6]))
    r = rc.select("rows", slice(1, 3))
    assert (r.labels, list(r.ndslice.sizes), r.ndslice.offset) == (["rows", "cols"], [2, 6], 6)
    r = rc.select("cols", slice(0, 6, 2))
    assert (list(r.ndslice.sizes), list(r.ndslice.strides)) == ([4, 3], [6, 2])
    r = sh.select("width", slice(1, 4)).at("batch", 0)
    assert (r.labels, list(r.ndslice.sizes)) == (["height", "width"], [3, 3])
    r = sh.at("height", 1).select("width", slice(2, 4))
    assert (r.labels, list(r.ndslice.sizes)) == (["batch", "width"], [2, 2])
    # errors are ValueErrors (as in the reference) and the usual Python lookup errors
    with pytest.raises(ValueError):
        rc.at("nonexistent", 0)
    with pytest.raises(KeyError):
        rc.at("nonexistent", 0)
    with pytest.raises(ValueError):
        rc.at("rows", 5)
    with pytest.raises(IndexError):
        rc.at("rows", 5)
    assert rc.at("rows", -1).ndslice.offset == 18        # Python-style negative indices
