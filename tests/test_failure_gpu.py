"""The device-side timeout path, exercised without faulting anything: a bounded wait on a
flag that nobody sets runs out, the kernel records a status code and returns, the host
reads the code, clears it, and the device keeps working.  Also: a training step whose
kernels reported a failed wait must raise instead of returning a loss."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _withheld_flag_wait(limit_ms=5):
    """Launch a bounded wait on a flag that stays 0; returns after it has given up."""
    from monarch_b200.ops import kernels as K
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = K.status_word("cuda")
    K.check(K.lib().mb200_wait_flag(flag.data_ptr(), 1, limit_ms, st.data_ptr(), K.stream_ptr()),
            "wait_flag")
    return flag, st


def test_withheld_flag_times_out_reports_and_clears():
    from monarch_b200.ops import kernels as K
    torch.cuda.synchronize()
    K.status_word("cuda").zero_()
    flag, st = _withheld_flag_wait()
    torch.cuda.synchronize()                      # returns: the wait was bounded
    assert int(st[0].item()) == 2                 # kStatusFlagTimeout
    with pytest.raises(K.KernelError, match="flag timed out"):
        K.check_status("cuda")
    assert int(st[0].item()) == 0                 # the sticky word was cleared
    # the context is intact: a satisfied wait and an ordinary kernel run normally
    flag.fill_(1)
    K.check(K.lib().mb200_wait_flag(flag.data_ptr(), 1, 5, st.data_ptr(), K.stream_ptr()),
            "wait_flag")
    from monarch_b200 import ops
    x = torch.randn(8, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    y, _ = ops.rmsnorm_fwd(x, w, 1e-5)
    torch.cuda.synchronize()
    K.check_status("cuda")
    assert torch.isfinite(y.float()).all()


def test_sticky_status_makes_later_waits_give_up_at_once():
    from monarch_b200.ops import kernels as K
    K.status_word("cuda").zero_()
    _withheld_flag_wait(5)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    _withheld_flag_wait(500)                      # would spin for 0.5 s on a clean status
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 100
    with pytest.raises(K.KernelError):
        K.check_status("cuda")


def test_trainer_step_raises_when_a_kernel_wait_ran_out(tmp_path):
    from monarch_b200.ops import kernels as K
    from monarch_b200.parallel.trainer import Trainer
    K.status_word("cuda").zero_()
    tr = Trainer("tiny", seq_len=128, micro_batch=2, parallelism="single", device="cuda:0")
    tok = torch.randint(0, tr.cfg.vocab, (2, 128))
    assert tr.step(tok, tok) > 0
    _withheld_flag_wait()                         # stands for a collective whose peer stalled
    with pytest.raises(K.KernelError):
        tr.step(tok, tok)
    assert tr.step(tok, tok) > 0                  # cleared: training goes on
    # the non-blocking entry point learns of it one call later, checkpoints refuse at once
    _withheld_flag_wait()
    dev_tok = tok.cuda()
    tr.step_device(dev_tok, dev_tok)
    torch.cuda.synchronize()
    with pytest.raises(K.KernelError):
        tr.step_device(dev_tok, dev_tok)
    _withheld_flag_wait()
    with pytest.raises(K.KernelError):
        tr.save_checkpoint(str(tmp_path / "ck"))
    tr.save_checkpoint(str(tmp_path / "ck"))
