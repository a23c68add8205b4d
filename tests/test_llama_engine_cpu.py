"""The explicit forward/backward engine must reproduce autograd on the stock-torch
model (same weights, fp32 CPU reference ops)."""
import pytest
import torch

from monarch_b200.models import (PRESETS, LlamaEngine, LocalParamStore, ParamLayout, TorchLlama,
                                 load_hf_state_dict, to_hf_state_dict)


def _fp32_store(cfg, layout):
    st = LocalParamStore(layout, "cpu", seed=1, init_std=0.05)
    # run the CPU reference in fp32 so the comparison is tight
    st.params = st.master.clone()
    st.grads = torch.zeros_like(st.master)
    return st


@pytest.mark.parametrize("preset,ckpt", [("tiny", True), ("tiny", False), ("tiny-tied", True),
                                         ("tiny", 1)])
def test_engine_matches_autograd(preset, ckpt):
    cfg = PRESETS[preset]
    layout = ParamLayout(cfg)
    st = _fp32_store(cfg, layout)
    if ckpt is True or ckpt is False:
        eng = LlamaEngine(cfg, st, seq_len=16, checkpoint=ckpt)
    else:   # recompute only the first `ckpt` layers, keep the activations of the rest
        eng = LlamaEngine(cfg, st, seq_len=16, checkpoint=True, recompute_layers=ckpt)
        assert eng.recompute_layers == ckpt < cfg.n_layers
    torch.manual_seed(0)
    tokens = torch.randint(0, cfg.vocab, (2, 16))
    targets = torch.randint(0, cfg.vocab, (2, 16))
    loss = eng.forward_backward(tokens, targets)

    ref = TorchLlama(cfg).float()
    ref.load_state_dict(to_hf_state_dict(cfg, layout, st.params), strict=True)
    ref_loss = ref(tokens, targets)
    ref_loss.backward()
    assert torch.allclose(loss, ref_loss, atol=1e-5), (loss, ref_loss)

    gsd = to_hf_state_dict(cfg, layout, st.grads)
    for name, p in ref.named_parameters():
        g = gsd[name]
        assert torch.allclose(g, p.grad, atol=2e-5, rtol=1e-4), (
            name, (g - p.grad).abs().max().item())


def test_state_dict_roundtrip():
    cfg = PRESETS["tiny"]
    layout = ParamLayout(cfg)
    st = LocalParamStore(layout, "cpu", seed=3)
    sd = to_hf_state_dict(cfg, layout, st.params)
    m = TorchLlama(cfg).to(torch.bfloat16)
    m.load_state_dict(sd)
    flat2 = torch.zeros_like(st.params)
    load_hf_state_dict(cfg, layout, m.state_dict(), flat2)
    assert torch.equal(flat2, st.params)


def test_adamw_step_matches_torch():
    cfg = PRESETS["tiny"]
    layout = ParamLayout(cfg)
    st = LocalParamStore(layout, "cpu", seed=2)
    st.grads = torch.randn(layout.total).to(torch.bfloat16)
    p0 = st.master.clone()
    p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(3):
        p.grad = st.grads.float()
        opt.step()
        st.optimizer_step(1e-3)
    assert torch.allclose(st.master, p.detach(), atol=1e-6)
