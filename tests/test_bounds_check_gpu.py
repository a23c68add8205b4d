"""The bounds-checked kernel library (``MB200_KERNEL_LIB=checked``): collectives look every
peer access up in a table of registered ranges; an access outside them is not performed and
is reported through the status word.  The "wrong" pointer used here points at valid memory
of this process that merely was not registered, so nothing can fault in either build."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import torch
    from monarch_b200.ops import ipc, kernels as K
    from monarch_b200.parallel.meshcomm import MeshComm
    assert K.CHECKED and K.lib().mb200_bounds_enabled() == 1
    dev = torch.device("cuda", 0)
    cap = 1 << 16
    local = MeshComm.allocate_local(dev, cap)
    comm = MeshComm.from_exports(0, [ipc.export_handle(local)], local, dev, cap)
    x = torch.arange(1000, device=dev, dtype=torch.float32)
    # registered ranges: everything works as in the regular build
    assert torch.equal(comm.all_reduce(x, "sum"), x)
    assert torch.equal(comm.all_gather(x)[0], x)
    torch.cuda.synchronize(); K.check_status(dev)
    # a stale "peer" pointer: valid memory, but not a range the communicator registered
    stray = torch.zeros_like(local)
    comm.ptrs[0] = stray.data_ptr()
    comm._at_cache.clear()                    # (pointer arrays are cached per offset)
    y = comm.all_reduce(x, "sum")
    torch.cuda.synchronize()
    st = K.status_word(dev)
    assert int(st[0].item()) == 4, st.tolist()
    addr = (int(st[3].item()) << 32) | (int(st[2].item()) & 0xffffffff)
    assert stray.data_ptr() <= addr < stray.data_ptr() + stray.numel(), hex(addr)
    assert y.eq(0).all()                      # the refused loads read as zeros
    try:
        K.check_status(dev)
        raise SystemExit("no error raised")
    except K.KernelError as e:
        assert "bounds" in str(e), e
    # the word is cleared and the device keeps working
    comm.ptrs[0] = local.data_ptr()
    comm._at_cache.clear()
    st[2:].zero_()
    # (the aborted collective left its epoch published on the stray buffer: start afresh)
    comm2_buf = MeshComm.allocate_local(dev, cap)
    comm2 = MeshComm.from_exports(0, [ipc.export_handle(comm2_buf)], comm2_buf, dev, cap)
    assert torch.equal(comm2.all_reduce(x, "max"), x)
    torch.cuda.synchronize(); K.check_status(dev)
    print("BOUNDS OK")
""")


def test_checked_library_refuses_unregistered_peer_access():
    env = dict(os.environ, MB200_KERNEL_LIB="checked", PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-c", SCRIPT], env=env, cwd=ROOT, capture_output=True,
                       text=True, timeout=280)
    assert p.returncode == 0 and "BOUNDS OK" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]
