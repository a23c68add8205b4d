"""Property tests (hypothesis): slice index algebra, selection routing == evaluation,
fan-out-limited reshapes, channel framing over both read paths, message flattening.
Modelled on the reference's proptest suites (ndslice/src/strategy.rs, selection/test_utils.rs,
hyperactor/src/channel/net/framed.rs, serde_multipart)."""
import pickle

import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

from monarch_b200 import _native as N
from monarch_b200.actor.pickle import flatten, unflatten

_cfg = settings(max_examples=80, deadline=None,
                suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])

dims_st = st.lists(st.integers(1, 5), min_size=1, max_size=4)


@st.composite
def slices(draw):
    dims = draw(dims_st)
    base = N.Slice.new_row_major(dims)
    return N.Slice(draw(st.integers(0, 7)), dims, base.strides)


@st.composite
def selection_text(draw, dims, depth=0):
    if depth == len(dims):
        return None
    n = dims[depth]
    kind = draw(st.sampled_from(["all", "idx", "range"]))
    if kind == "all":
        head = "*"
    elif kind == "idx":
        head = str(draw(st.integers(0, n - 1)))
    else:
        a = draw(st.integers(0, n - 1))
        b = draw(st.integers(a, n))
        head = f"{a}:{b}:{draw(st.sampled_from([1, 2, 3]))}"
    rest = draw(selection_text(dims, depth + 1))
    return head if rest is None else f"{head},{rest}"


@_cfg
@given(slices())
def test_slice_index_location_roundtrip(sl):
    ranks = sl.ranks()
    assert len(ranks) == len(set(ranks)) == len(sl)
    for i, r in enumerate(ranks):
        assert sl.index(r) == i
        coords = sl.coordinates(r)
        assert sl.nditem(coords) == r
        assert all(0 <= c < n for c, n in zip(coords, sl.sizes))
    clone = pickle.loads(pickle.dumps(sl))
    assert clone == sl and clone.ranks() == ranks


@_cfg
@given(st.data())
def test_cast_routing_reaches_exactly_the_selected_ranks(data):
    sl = data.draw(slices())
    dims = list(sl.sizes)
    parts = [data.draw(selection_text(dims)) for _ in range(data.draw(st.integers(1, 3)))]
    text = data.draw(st.sampled_from(["|", "&"])).join(f"({p})" for p in parts)
    sel = N.Selection.from_string(text)
    want = sel.eval(sl)
    delivered, hops, _ = N.simulate_cast(sel, sl)
    assert sorted(delivered) == sorted(want), text
    assert len(set(delivered)) == len(delivered)          # nobody hears it twice
    assert all(h <= len(dims) for h in hops.values())     # one hop per dimension at most


@_cfg
@given(st.integers(1, 400), st.integers(2, 16))
def test_reshape_with_limit_keeps_ranks_and_bounds_every_dim(n, limit):
    sl = N.Slice.new_row_major([n])
    r = N.reshape_with_limit(sl, limit)
    assert r.ranks() == sl.ranks()
    # a dimension stays above the limit only when it has no divisor the limit allows
    for size in r.sizes:
        assert size <= limit or all(size % d for d in range(2, limit + 1)), (n, limit, r.sizes)


frame_st = st.tuples(
    st.binary(min_size=0, max_size=200),
    st.lists(st.one_of(st.binary(min_size=0, max_size=300),
                       st.integers(60_000, 200_000).map(lambda n: bytes([n % 251]) * n)),
             min_size=0, max_size=4))


@pytest.fixture(scope="module")
def unix_pair():
    rx = N.channel_serve_any("unix")
    tx = N.channel_dial(rx.addr)
    yield tx, rx
    tx.close()
    rx.close()


@settings(max_examples=40, deadline=None,
          suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture,
                                 HealthCheck.data_too_large, HealthCheck.large_base_example])
@given(st.lists(frame_st, min_size=1, max_size=12))
def test_frames_arrive_intact_and_in_order(unix_pair, frames):
    """Small frames are read in one piece and split, large ones part by part in place: a
    mixed stream must come out exactly as it went in."""
    tx, rx = unix_pair
    for head, parts in frames:
        tx.post(head, parts)
    for head, parts in frames:
        got = rx.recv(10000)
        assert got is not None
        assert got[0] == head and list(got[1]) == parts


leaf_st = st.one_of(st.integers(), st.text(max_size=20), st.none(), st.floats(allow_nan=False),
                    st.binary(max_size=64),
                    st.integers(65_536, 70_000).map(lambda n: b"z" * n),
                    st.integers(1, 3000).map(lambda n: torch.arange(n, dtype=torch.float32)))


@settings(max_examples=60, deadline=None, suppress_health_check=list(HealthCheck))
@given(st.recursive(leaf_st, lambda ch: st.one_of(st.lists(ch, max_size=4),
                                                  st.dictionaries(st.text(max_size=5), ch,
                                                                  max_size=4),
                                                  st.tuples(ch, ch)), max_leaves=12))
def test_flatten_unflatten_roundtrip(obj):
    """Large tensors, bytes and bytearrays leave the pickle as parts; whatever the nesting,
    the message comes back equal."""
    body, parts = flatten(obj)
    # parts may be views of the sender's memory: the wire would copy them
    back = unflatten(body, [bytes(p) for p in parts])
    assert _same(back, obj)


def _same(a, b):
    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and \
            a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    if isinstance(a, (list, tuple)):
        return type(a) is type(b) and len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, dict):
        return isinstance(b, dict) and a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    return a == b and type(a) is type(b)
