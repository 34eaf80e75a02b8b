"""One Llama block through the block-level driver calls (the single-block microbenchmark
configuration): against a plain PyTorch fp32 restatement of the reference's block
(src/llama.cpp:9-60: pre-RMSNorm with eps 1e-5, q/k/v projections stored [in, out],
interleaved-pair rotary on every head, causal attention per sequence with grouped kv heads,
SwiGLU, residual adds), and checkpointed against plain -- the reference's own assertion for
checkpoint(fn, x), tests/test_checkpointing.cpp:45-90, here bitwise."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mt():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from paperkiln_b200 import model
    model.init(0, model.FP32)
    yield model
    model.init(0, model.FP32)


def torch_block(params, x, B, S, H, Hkv, dk, theta):
    import torch
    d = x.shape[1]

    def rms(t, w):
        return t * torch.rsqrt((t * t).mean(dim=1, keepdim=True) + 1e-5) * w

    def rope(t, heads):
        pos = torch.arange(S, dtype=torch.float32).repeat(B)
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), torch.arange(0, dk, 2, dtype=torch.float32) / dk)
        ang = pos[:, None] * inv[None, :]
        c, s = torch.cos(ang), torch.sin(ang)
        t = t.view(-1, heads, dk // 2, 2)
        x0, x1 = t[..., 0], t[..., 1]
        out = torch.stack((x0 * c[:, None, :] - x1 * s[:, None, :], x0 * s[:, None, :] + x1 * c[:, None, :]), dim=-1)
        return out.reshape(-1, heads * dk)

    h = rms(x, params["input_layernorm.weight"])
    q = rope(h @ params["self_attn.q_proj.weight"], H)
    k = rope(h @ params["self_attn.k_proj.weight"], Hkv)
    v = h @ params["self_attn.v_proj.weight"]
    qh = q.view(B, S, H, dk).transpose(1, 2)
    kh = k.view(B, S, Hkv, dk).transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    vh = v.view(B, S, Hkv, dk).transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    s = (qh @ kh.transpose(-1, -2)) / math.sqrt(dk)
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    a = (torch.softmax(s, dim=-1) @ vh).transpose(1, 2).reshape(B * S, H * dk)
    x = x + a @ params["self_attn.o_proj.weight"]
    h = rms(x, params["post_attention_layernorm.weight"])
    g = h @ params["mlp.gate_proj.weight"]
    u = h @ params["mlp.up_proj.weight"]
    return x + (torch.nn.functional.silu(g) * u) @ params["mlp.down_proj.weight"]


def test_block_matches_fp32_restatement(mt):
    import torch
    B, S, H, Hkv, d, dff, theta = 2, 24, 4, 2, 64, 160, 10000.0
    dk = d // H
    rng = np.random.RandomState(3)
    x = rng.randn(B * S, d).astype(np.float32)
    dy = (rng.randn(B * S, d) * 1e-2).astype(np.float32)
    for ckpt in (0, 1):
        m = mt.Model(family="block", d=d, heads=H, kv_heads=Hkv, dff=dff, theta=theta, rope_all=1, seed=5, ckpt=ckpt)
        params = {n: torch.tensor(m.get_param(n), requires_grad=True) for n in m.names}
        xt = torch.tensor(x, requires_grad=True)
        ref = torch_block(params, xt, B, S, H, Hkv, dk, theta)
        ref.backward(torch.tensor(dy))
        m.block_set_input(x, dy, S)
        m.block_forward()
        y = m.block_output()
        m.block_backward()
        assert np.abs(y - ref.detach().numpy()).max() <= 1e-4 * max(1.0, float(ref.abs().max()))
        dx = m.block_input_grad()
        assert np.abs(dx - xt.grad.numpy()).max() <= 1e-4 * max(1.0, float(xt.grad.abs().max()))
        for n in m.names:
            g, r = m.get_grad(n), params[n].grad.numpy()
            assert g is not None, n
            a_, b_ = g.astype(np.float64).ravel(), r.astype(np.float64).ravel()
            assert a_ @ b_ / (np.linalg.norm(a_) * np.linalg.norm(b_)) >= 0.9999, n
            assert np.abs(g - r).max() <= 1e-4 * max(1.0, float(np.abs(r).max())), n
        m.close()


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_block_checkpointed_equals_plain_bitwise(mt, dtype):
    """Shape of the single-block configuration at reduced width: head_dim 128, SwiGLU, batch 4."""
    mt.init(0, mt.BF16 if dtype == "bf16" else mt.FP32)
    try:
        B, S, H, d, dff = 4, 256, 2, 256, 704
        rng = np.random.RandomState(7)
        x = rng.randn(B * S, d).astype(np.float32)
        dy = (rng.randn(B * S, d) * 1e-3).astype(np.float32)
        res = {}
        for ckpt in (0, 1):
            m = mt.Model(family="block", d=d, heads=H, kv_heads=H, dff=dff, theta=10000.0, rope_all=1, seed=9, ckpt=ckpt)
            m.block_set_input(x, dy, S)
            m.block_forward()
            live = m.live_after_forward()
            y = m.block_output()
            m.block_backward()
            res[ckpt] = (y, m.block_input_grad(), m.grads(), live)
            m.close()
        assert np.array_equal(res[0][0], res[1][0])
        assert np.array_equal(res[0][1], res[1][1])
        for n, g in res[0][2].items():
            assert np.array_equal(g, res[1][2][n]), n
        assert res[1][3] * 2 < res[0][3], f"live variables {res[0][3]} -> {res[1][3]}"
    finally:
        mt.init(0, mt.FP32)
