"""The allocation-free RMSNorm backward (`mb200_rmsnorm_bwd_noalloc`).

Some users of the kernel library cannot allocate device memory at the point where they
need the kernel (inside a stream capture, inside a host runtime that owns all device
memory, in a loop where allocation is banned).  For them the library keeps the scratch of
the RMSNorm backward in a built-in device array.  This test drives that entry point the
way such a caller would -- through its exported C symbol, passing only inputs and outputs
-- and checks it against the regular entry point, twice in a row, because consecutive
calls share the same scratch and must not disturb one another.

The file name sorts last on purpose: a run that stops at the first failure has already
run every other test by the time it gets here.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _symbol():
    from monarch_b200.ops import kernels as K
    fn = K.lib().mb200_rmsnorm_bwd_noalloc
    vp, i = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
    fn.restype = i
    return fn


# (1000, 8192): more row blocks than the built-in scratch has room for at this width, so
# the entry point has to clip its block count; (77, 8192) and (1000, 4096) stay below it.
@pytest.mark.parametrize("rows,d,accumulate", [(1000, 4096, 0), (77, 8192, 0), (1000, 8192, 0),
                                               (300, 2048, 1)])
def test_noalloc_matches_regular_entry_point_twice(rows, d, accumulate):
    from monarch_b200 import ops
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        torch.manual_seed(10 * call + rows)
        x = torch.randn(rows, d, device="cuda", dtype=bf16)
        w = (1 + 0.1 * torch.randn(d, device="cuda")).to(bf16)
        dy = torch.randn(rows, d, device="cuda", dtype=bf16)
        dres = torch.randn(rows, d, device="cuda", dtype=bf16)
        _, rstd = ops.rmsnorm_fwd(x, w, 1e-5)
        dw0 = (0.5 * torch.randn(d, device="cuda")).to(bf16) if accumulate else \
            torch.zeros(d, device="cuda", dtype=bf16)
        dw_ref = dw0.clone()
        dx_ref = ops.rmsnorm_bwd(dy, x, w, rstd, dw_ref, accumulate=bool(accumulate), dres=dres)
        dx = torch.empty_like(x)
        dw = dw0.clone()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]   # sees cudaMalloc, not only torch's pool
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                dx.data_ptr(), dw.data_ptr(), accumulate, rows, d, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call == 1:   # the first call on a device may page the library's own image in
            assert torch.cuda.mem_get_info()[0] == free_before
        assert _rel(dx, dx_ref) < 6e-3, (call, _rel(dx, dx_ref))
        assert _rel(dw, dw_ref) < 6e-3, (call, _rel(dw, dw_ref))


def test_noalloc_rejects_sizes_beyond_its_scratch():
    fn = _symbol()
    t = torch.zeros(8, device="cuda", dtype=bf16)
    f = torch.zeros(8, device="cuda")
    p = t.data_ptr()
    assert fn(p, p, p, f.data_ptr(), None, p, p, 0, 1, 8192 + 8, None) == 1101
    assert fn(p, p, p, f.data_ptr(), None, p, p, 0, 1, 12, None) == 1101
    assert fn(p, p, p, f.data_ptr(), None, p, p, 0, -1, 64, None) == 1102
    torch.cuda.synchronize()
