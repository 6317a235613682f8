"""GPT model: the hand-scheduled forward/backward must match PyTorch autograd of an independent
plain implementation (CPU fp32), and the CUDA bf16 step must track the CPU one."""
import math

import pytest
import torch

from spiraltorch_b200.models.gpt import GPTConfig, GPTModel


def _plain_loss(model: GPTModel, tokens, targets):
    """Independent PyTorch statement of the same network, built on the model's parameters."""
    cfg, P = model.cfg, {k: v.detach().clone().float().requires_grad_(True) for k, v in model.p.items()}
    B, S = tokens.shape
    d, H, D = cfg.d_model, cfg.n_heads, cfg.head_dim

    def norm(x, name):
        if cfg.norm == "rms":
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * P[name + ".gamma"]
        return torch.nn.functional.layer_norm(x, (d,), P[name + ".gamma"], P[name + ".beta"], cfg.norm_eps)

    h = P["embed.weight"][tokens.reshape(-1)]
    if cfg.positional == "learned":
        h = h + P["pos.weight"][torch.arange(B * S) % S]
    inv = 1.0 / (cfg.rope_base ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = torch.arange(S, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos().float(), ang.sin().float()

    def rope(x):  # [B,S,H,D]
        a, b = x[..., : D // 2], x[..., D // 2:]
        c, s_ = cos[None, :, None], sin[None, :, None]
        return torch.cat([a * c - b * s_, b * c + a * s_], -1)

    for l in range(cfg.n_layers):
        y = norm(h, f"h{l}.norm1")
        qkv = (y @ P[f"h{l}.qkv.weight"].T).view(B, S, 3, H, D)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if cfg.positional == "rope":
            q, k = rope(q), rope(k)
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        o = o.transpose(1, 2).reshape(B * S, H * D)
        h = h + o @ P[f"h{l}.proj.weight"].T
        y = norm(h, f"h{l}.norm2")
        a = torch.nn.functional.gelu(y @ P[f"h{l}.fc1.weight"].T, approximate="tanh")
        h = h + a @ P[f"h{l}.fc2.weight"].T
    logits = norm(h, "norm_f") @ P["embed.weight"].T
    return torch.nn.functional.cross_entropy(logits, targets.reshape(-1)), P


@pytest.mark.parametrize("norm,positional", [("rms", "rope"), ("layer", "learned")])
def test_manual_backward_matches_autograd_cpu(norm, positional):
    torch.manual_seed(0)
    cfg = GPTConfig(vocab_size=96, d_model=128, n_layers=2, n_heads=2, ffn=256, seq_len=16,
                    norm=norm, positional=positional, init_std=0.05)
    model = GPTModel(cfg, device="cpu", dtype=torch.float32)
    tokens = torch.randint(0, 96, (3, 16))
    targets = torch.randint(0, 96, (3, 16))
    loss = model.forward_backward(tokens, targets)
    ref_loss, P = _plain_loss(model, tokens, targets)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 1e-4
    for name, p in model.p.items():
        g, r = p.main_grad, P[name].grad
        assert torch.allclose(g, r, atol=2e-4, rtol=2e-3), (name, (g - r).abs().max().item())


def test_autograd_facade_accumulates_main_grad():
    cfg = GPTConfig(vocab_size=64, d_model=128, n_layers=1, n_heads=2, ffn=128, seq_len=8)
    model = GPTModel(cfg, device="cpu", dtype=torch.float32)
    tokens = torch.randint(0, 64, (2, 8))
    targets = torch.randint(0, 64, (2, 8))
    loss = model(tokens, targets)
    loss.backward()
    g1 = model.flat_grad.clone()
    model.zero_grad_buffers()
    model.forward_backward(tokens, targets)
    assert torch.allclose(g1, model.flat_grad, atol=1e-6)
    logits = model(tokens)
    assert logits.shape == (16, 64)


@pytest.mark.gpu
def test_cuda_step_tracks_cpu_reference():
    torch.manual_seed(0)
    cfg = GPTConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=2, ffn=512, seq_len=256, init_std=0.05)
    gpu = GPTModel(cfg, device="cuda", dtype=torch.bfloat16)
    cpu = GPTModel(cfg, device="cpu", dtype=torch.float32)
    cpu.flat_w.copy_(gpu.flat_w.float().cpu())
    tokens = torch.randint(0, 512, (2, 256))
    targets = torch.randint(0, 512, (2, 256))
    lg = gpu.forward_backward(tokens.cuda(), targets.cuda())
    lc = cpu.forward_backward(tokens, targets)
    assert abs(lg.item() - lc.item()) < 3e-2
    gg, gc = gpu.flat_grad.cpu(), cpu.flat_grad
    cos = torch.nn.functional.cosine_similarity(gg, gc, dim=0).item()
    assert cos > 0.99, cos
    rel = (gg - gc).norm() / gc.norm()
    assert rel < 0.1, rel.item()
