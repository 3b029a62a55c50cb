"""Grouped-GEMM mixture-of-experts path against a per-expert fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(x, wts, idx, gw, uw, dw):
    T, D = x.shape
    out = torch.zeros(T, D, dtype=torch.float32, device=x.device)
    for t_k in range(idx.shape[1]):
        for e in range(gw.shape[0]):
            sel = idx[:, t_k] == e
            if sel.any():
                xs = x[sel].float()
                h = torch.nn.functional.silu(xs @ gw[e].float().t()) * (xs @ uw[e].float().t())
                out[sel] += wts[sel, t_k, None].float() * (h @ dw[e].float().t())
    return out


@pytest.mark.parametrize("T,E,k,D,Fd", [(300, 8, 2, 128, 192), (64, 16, 4, 256, 64), (1000, 4, 1, 192, 320)])
def test_experts_forward_backward(T, E, k, D, Fd):
    from tunix_b200 import _lib
    from tunix_b200.ops import moe
    torch.manual_seed(0)
    dev = "cuda"
    x = (torch.randn(T, D, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
    gw = (torch.randn(E, Fd, D, device=dev) * 0.08).to(torch.bfloat16).requires_grad_()
    uw = (torch.randn(E, Fd, D, device=dev) * 0.08).to(torch.bfloat16).requires_grad_()
    dw = (torch.randn(E, D, Fd, device=dev) * 0.08).to(torch.bfloat16).requires_grad_()
    logits = torch.randn(T, E, device=dev)
    if E == 16:
        logits[:, 5] = -1e9       # an expert nobody picks
    wts, idx = torch.topk(torch.softmax(logits, -1), k, -1)
    wts = wts.detach().requires_grad_()
    res = torch.randn(T, D, device=dev).to(torch.bfloat16)
    out = moe.experts(x, wts, idx, gw, uw, dw, residual=res)
    _lib.raise_if_kernel_error()
    dout = torch.randn(T, D, device=dev).to(torch.bfloat16)
    out.backward(dout)
    _lib.raise_if_kernel_error()
    xr, wr = x.detach().float().requires_grad_(), wts.detach().clone().requires_grad_()
    gr, ur, dr = (w.detach().float().requires_grad_() for w in (gw, uw, dw))
    ref = _ref(xr, wr, idx, gr, ur, dr) + res.float()
    ref.backward(dout.float())

    def rel(a, b):
        return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()
    assert rel(out, ref) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(wts.grad, wr.grad) < 2e-2
    assert rel(gw.grad, gr.grad) < 2e-2 and rel(uw.grad, ur.grad) < 2e-2 and rel(dw.grad, dr.grad) < 2e-2


def test_moe_model_trains_and_matches_fallback():
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    cfg = ModelConfig(family="qwen3", num_layers=2, vocab_size=512, embed_dim=128, hidden_dim=256, num_heads=4, head_dim=32,
                      num_kv_heads=2, qk_norm=True, dtype=torch.bfloat16, max_position=256, num_experts=8,
                      num_experts_per_tok=2, moe_hidden_dim=64)
    model = create_model(cfg, device=torch.device("cuda"), seed=0)
    toks = torch.randint(0, 512, (2, 64), device="cuda")
    logits = model(toks)[0] if isinstance(model(toks), tuple) else model(toks)
    layer = model.layers[0].mlp
    x = torch.randn(128, 128, device="cuda").to(torch.bfloat16)
    w, idx = torch.topk(torch.softmax(torch.randn(128, 8, device="cuda"), -1), 2, -1)
    from tunix_b200.parallel import moe_dispatch
    fast = moe_dispatch.expert_forward(layer, x, w, idx)
    slow = _ref(x, w, idx, layer.gate_proj, layer.up_proj, layer.down_proj)
    assert ((fast.float() - slow).norm() / slow.norm()).item() < 1e-2
    loss = logits.float().logsumexp(-1).mean()
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad.float()).all() for p in layer.parameters())
