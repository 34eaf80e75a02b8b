"""TEST INFRASTRUCTURE -- CPU oracle for the checkpointed transformer training step.

A numpy (float32) restatement of the reference's algorithm for this path, one function
per tape op plus the three model families, each citing the reference source it follows
(paths relative to the paperkiln repository). It exists to check the CUDA path; only
tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may import it, and only
as the checker -- never as something measured as the product or shipped.

Pinned: tests/test_oracle_cpu.py compares every function here with golden vectors that
the unmodified reference wrote (tests/golden/*.npz via oracle/ref_harness.cpp), so
parity of this oracle with the reference is pinned, not assumed.

Activation checkpointing does not change the mathematics (the reference recomputes the
same ops on the same values, src/autograd.cpp:68-102), so the oracle has no checkpoint
switch: its result is the one both modes must produce.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import numpy as np

F = np.float32


# ----------------------------------------------------------------------------- ops
def rmsnorm_fwd(x, w, eps=1e-5):
    """ops::rmsnorm forward, src/ops.cpp:426-447 (eps is the literal 1e-5)."""
    ms = (x * x).sum(axis=1, dtype=F) / F(x.shape[1])
    rinv = (F(1.0) / np.sqrt(ms + F(eps))).astype(F)
    return (x * rinv[:, None] * w).astype(F), rinv


def rmsnorm_bwd(dy, x, w, rinv):
    """src/ops.cpp:448-478: dw = colsum(dy*x*rinv); dx = rinv*(dy*w - x*rinv^2*sum(dy*w*x)/C)."""
    C = x.shape[1]
    dw = (dy * x * rinv[:, None]).sum(axis=0, dtype=F)[None, :]
    term = (dy * w * x).sum(axis=1, dtype=F)
    dx = rinv[:, None] * (dy * w - x * (rinv * rinv)[:, None] * term[:, None] / F(C))
    return dx.astype(F), dw.astype(F)


def layernorm_fwd(x, g, b, eps=1e-5):
    """ops::layernorm forward, src/ops.cpp:248-283 (biased variance)."""
    C = x.shape[1]
    mu = x.sum(axis=1, dtype=F) / F(C)
    d = x - mu[:, None]
    var = (d * d).sum(axis=1, dtype=F) / F(C)
    rstd = (F(1.0) / np.sqrt(var + F(eps))).astype(F)
    xhat = (d * rstd[:, None]).astype(F)
    return (g * xhat + b).astype(F), xhat, rstd


def layernorm_bwd(dy, xhat, rstd, g):
    """src/ops.cpp:284-326."""
    dg = (dy * xhat).sum(axis=0, dtype=F)[None, :]
    db = dy.sum(axis=0, dtype=F)[None, :]
    dxh = dy * g
    m1 = dxh.mean(axis=1, dtype=F)[:, None]
    m2 = (dxh * xhat).mean(axis=1, dtype=F)[:, None]
    dx = rstd[:, None] * (dxh - m1 - xhat * m2)
    return dx.astype(F), dg.astype(F), db.astype(F)


_K = F(0.7978845608028654)


def gelu_fwd(x):
    """Matrix::apply_gelu, third_party/transformer_cpp/src/components.cpp:192-200."""
    return (x * (F(0.5) * (F(1.0) + np.tanh(_K * (x + F(0.044715) * x * x * x))))).astype(F)


def gelu_bwd(dy, x):
    """src/ops.cpp:118-136 (the correct tanh-GELU derivative)."""
    u = _K * (x + F(0.044715) * x * x * x)
    t = np.tanh(u)
    cdf = F(0.5) * (F(1.0) + t)
    pdf = F(0.5) * (F(1.0) - t * t) * _K * (F(1.0) + F(0.134145) * x * x)
    return (dy * (cdf + x * pdf)).astype(F)


def silu_fwd(x):
    """src/ops.cpp:404-410."""
    return (x / (F(1.0) + np.exp(-x))).astype(F)


def silu_bwd(dy, x):
    """src/ops.cpp:411-423."""
    s = F(1.0) / (F(1.0) + np.exp(-x))
    return (dy * (s * (F(1.0) + x * (F(1.0) - s)))).astype(F)


def relu_fwd(x):
    return np.maximum(x, F(0)).astype(F)


def relu_bwd(dy, x):
    """src/ops.cpp:788-801."""
    return np.where(x > 0, dy, F(0)).astype(F)


def rope_table(n_pos: int, head_dim: int, theta_base: float):
    """cos/sin per (position, pair) with the float expressions of src/ops.cpp:499-503."""
    dims = np.arange(0, head_dim, 2, dtype=F)
    inv_freq = (F(1.0) / np.power(F(theta_base), dims / F(head_dim), dtype=F)).astype(F)
    ang = (np.arange(n_pos, dtype=F)[:, None] * inv_freq[None, :]).astype(F)
    return np.cos(ang).astype(F), np.sin(ang).astype(F)


def rope_apply(x, pos, theta_base, head_dim, col0, n_heads, inverse=False):
    """Interleaved-pair rotation of n_heads heads starting at column col0
    (src/ops.cpp:495-511; the backward, :519-534, is the rotation by -theta)."""
    out = x.copy()
    cos, sin = rope_table(int(pos.max()) + 1, head_dim, theta_base)
    c, s = cos[pos], sin[pos]
    if inverse:
        s = -s
    for h in range(n_heads):
        a = col0 + h * head_dim
        x0 = x[:, a:a + head_dim:2]
        x1 = x[:, a + 1:a + head_dim:2]
        out[:, a:a + head_dim:2] = x0 * c - x1 * s
        out[:, a + 1:a + head_dim:2] = x0 * s + x1 * c
    return out.astype(F)


def apply_rope_reference(qkv, pos, theta_base, head_dim):
    """ops::apply_rope on the fused [T,3d] layout: only the FIRST head of q and of k is
    rotated (src/ops.cpp:495-511 loops dim < head_dim from column 0 and column d)."""
    d = qkv.shape[1] // 3
    out = rope_apply(qkv, pos, theta_base, head_dim, 0, 1)
    return rope_apply(out, pos, theta_base, head_dim, d, 1)


def attention_fwd(q, k, v, scale, seq_len, causal=True):
    """One head of ops::fused_attention, src/ops.cpp:863-901. Returns y and the weights A."""
    T = q.shape[0]
    sl = T if seq_len == 0 else seq_len
    A = np.zeros((T, T), dtype=F)
    for b0 in range(0, T, sl):
        s = (q[b0:b0 + sl] @ k[b0:b0 + sl].T).astype(F) * F(scale)
        if causal:
            s = np.where(np.tril(np.ones((sl, sl), dtype=bool)), s, F(-np.inf))
        s = s - s.max(axis=1, keepdims=True)
        e = np.exp(s).astype(F)
        A[b0:b0 + sl, b0:b0 + sl] = e / e.sum(axis=1, keepdims=True, dtype=F)
    return (A @ v).astype(F), A


def attention_bwd(dy, q, k, v, A, scale):
    """src/ops.cpp:903-933."""
    dv = (A.T @ dy).astype(F)
    dA = (dy @ v.T).astype(F)
    dot = (dA * A).sum(axis=1, keepdims=True, dtype=F)
    ds = (F(scale) * A * (dA - dot)).astype(F)
    return (ds @ k).astype(F), (ds.T @ q).astype(F), dv


def cross_entropy_fwd(logits, targets):
    """ops::cross_entropy, src/ops.cpp:350-369: softmax, NLL summed in double, clamp 1e-12."""
    z = logits - logits.max(axis=1, keepdims=True)
    e = np.exp(z).astype(F)
    P = (e / e.sum(axis=1, keepdims=True, dtype=F)).astype(F)
    pt = np.maximum(P[np.arange(len(targets)), targets], F(1e-12))
    loss = F(-np.log(pt).astype(np.float64).sum() / len(targets))
    return loss, P


def cross_entropy_bwd(P, targets, g=1.0):
    """src/ops.cpp:370-375."""
    dl = P.copy()
    dl[np.arange(len(targets)), targets] -= F(1.0)
    return (dl * F(g / P.shape[0])).astype(F)


def embedding_bwd(dy, ids, vocab):
    """Scatter-add in ascending position order, src/ops.cpp:338-347."""
    out = np.zeros((vocab, dy.shape[1]), dtype=F)
    np.add.at(out, ids, dy)
    return out


def adamw_step(p, g, m, v, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01):
    """AdamW::step, src/nn.cpp:301-321 (float arithmetic throughout). Returns p, m, v."""
    b1, b2, lr, eps, wd = F(b1), F(b2), F(lr), F(eps), F(wd)
    c1 = F(1.0) - np.power(b1, F(t), dtype=F)
    c2 = F(1.0) - np.power(b2, F(t), dtype=F)
    m = (b1 * m + (F(1.0) - b1) * g).astype(F)
    v = (b2 * v + (F(1.0) - b2) * g * g).astype(F)
    upd = (m / c1) / (np.sqrt(v / c2) + eps)
    return (p - lr * (upd + wd * p)).astype(F), m, v


def clip_grad_norm(grads: List[np.ndarray], max_norm: float):
    """ops::clip_grad_norm, src/ops.cpp:1046-1064 (sum of squares in double)."""
    sq = sum(float((g.astype(np.float64) ** 2).sum()) for g in grads)
    total = F(math.sqrt(sq))
    if total > max_norm and total > 0:
        s = F(max_norm) / total
        grads = [(g * s).astype(F) for g in grads]
    return float(total), grads


def quantize_q8_0(W):
    """quantize_int8 (src/quant.cpp:11-37) at block 32 with the scale rounded to binary16
    (a zero-rounded scale becomes the smallest normal half) and q recomputed against the
    stored scale. Returns int8 q [rows, cols] and float32 scales [rows, cols/32]."""
    rows, cols = W.shape
    Wb = W.reshape(rows, cols // 32, 32)
    amax = np.abs(Wb).max(axis=2)
    s = np.where(amax > 0, amax / F(127.0), F(1.0)).astype(F)
    s16 = s.astype(np.float16).astype(F)
    s16 = np.where(s16 == 0, F(6.103515625e-05), s16)
    v = np.clip(Wb / s16[:, :, None], F(-127.0), F(127.0))
    q = np.where(v >= 0, np.floor(v + F(0.5)), np.ceil(v - F(0.5))).astype(np.int8)  # lround
    return q.reshape(rows, cols), s16


def dequantize_q8_0(q, scales):
    """dequantize, src/quant.cpp:39-48: float(q) * scale."""
    rows, cols = q.shape
    return (q.reshape(rows, cols // 32, 32).astype(F) * scales[:, :, None]).reshape(rows, cols).astype(F)


# ----------------------------------------------------------------------------- models
def _mha(q, k, v, H, Hkv, dk, seq_len, causal=True):
    """Per-head loop of the reference's blocks (src/llama.cpp:44-52, src/nn.cpp:144-150)
    with grouped-query head mapping h -> h // (H/Hkv). Returns out and a backward closure."""
    scale = F(1.0) / np.sqrt(F(dk))
    outs, caches = [], []
    grp = H // Hkv
    for h in range(H):
        g = h // grp
        qh, kh, vh = q[:, h * dk:(h + 1) * dk], k[:, g * dk:(g + 1) * dk], v[:, g * dk:(g + 1) * dk]
        y, A = attention_fwd(qh, kh, vh, scale, seq_len, causal)
        outs.append(y)
        caches.append((qh, kh, vh, A))

    def bwd(dy):
        dq, dk_, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
        for h in range(H):
            g = h // grp
            qh, kh, vh, A = caches[h]
            a, b, c = attention_bwd(dy[:, h * dk:(h + 1) * dk], qh, kh, vh, A, scale)
            dq[:, h * dk:(h + 1) * dk] = a
            dk_[:, g * dk:(g + 1) * dk] += b
            dv[:, g * dk:(g + 1) * dk] += c
        return dq, dk_, dv

    return np.concatenate(outs, axis=1).astype(F), bwd


class StepOracle:
    """Forward + backward of one family on a dict of float32 parameters named as the
    reference names them. `frozen` holds tensors that take no gradient (Q8_0-dequantized
    base weights, frozen embeddings / gains in the QLoRA harness)."""

    def __init__(self, family: str, params: Dict[str, np.ndarray], *, heads: int, kv_heads: int = 0,
                 layers: int, theta: float = 10000.0, tie: bool = True, rope_all: bool = False,
                 norm: str = "layernorm", act: str = "gelu", pos: str = "learned",
                 frozen: Optional[Dict[str, np.ndarray]] = None, lora_scaling: float = 0.0):
        self.family, self.p = family, {k: v.astype(F) for k, v in params.items()}
        self.H, self.Hkv, self.L = heads, kv_heads or heads, layers
        self.theta, self.tie, self.rope_all = theta, tie, rope_all
        self.norm, self.act, self.pos = norm, act, pos
        self.frozen = {k: v.astype(F) for k, v in (frozen or {}).items()}
        self.s = F(lora_scaling)
        self.g: Dict[str, np.ndarray] = {}

    # -- helpers
    def _w(self, name):
        return self.p[name] if name in self.p else self.frozen[name]

    def _acc(self, name, g):
        if name in self.p:
            self.g[name] = self.g.get(name, 0) + g.astype(F)

    def _proj(self, x, prefix):
        """Dense Linear, or frozen Q8_0 base + optional LoRA side path
        (QLoRALinear::forward, src/quant.cpp:114-119)."""
        if prefix + ".weight" in self.p or prefix + ".weight" in self.frozen:
            W = self._w(prefix + ".weight")
            y = (x @ W).astype(F)
            if prefix + ".lora_A" in self.p:
                A, B = self.p[prefix + ".lora_A"], self.p[prefix + ".lora_B"]
                xa = (x @ A).astype(F)
                y = (y + ((xa @ B).astype(F) * self.s)).astype(F)
            else:
                xa = None
            b = self.p.get(prefix + ".bias")
            if b is not None:
                y = (y + b).astype(F)

            def bwd(dy):
                dx = (dy @ W.T).astype(F)
                self._acc(prefix + ".weight", x.T @ dy)
                if b is not None:
                    self._acc(prefix + ".bias", dy.sum(axis=0, dtype=F)[None, :])
                if xa is not None:
                    dd = (dy * self.s).astype(F)
                    self._acc(prefix + ".lora_B", xa.T @ dd)
                    dxa = (dd @ B.T).astype(F)
                    self._acc(prefix + ".lora_A", x.T @ dxa)
                    dx = dx + (dxa @ A.T).astype(F)
                return dx.astype(F)

            return y, bwd
        raise KeyError(prefix)

    def _norm(self, x, wname, bname=None):
        if bname is None:
            w = self._w(wname)
            y, rinv = rmsnorm_fwd(x, w)

            def bwd(dy):
                dx, dw = rmsnorm_bwd(dy, x, w, rinv)
                self._acc(wname, dw)
                return dx
            return y, bwd
        g, b = self.p[wname], self.p[bname]
        y, xhat, rstd = layernorm_fwd(x, g, b)

        def bwd(dy):
            dx, dg, db = layernorm_bwd(dy, xhat, rstd, g)
            self._acc(wname, dg)
            self._acc(bname, db)
            return dx
        return y, bwd

    # -- blocks
    def _llama_block(self, x, i, pos, seq_len):
        pre = f"layers.{i}."
        d = x.shape[1]
        dk = d // self.H
        h, n1b = self._norm(x, pre + "input_layernorm.weight")
        q, qb = self._proj(h, pre + "self_attn.q_proj")
        k, kb = self._proj(h, pre + "self_attn.k_proj")
        v, vb = self._proj(h, pre + "self_attn.v_proj")
        nq, nk = (self.H, self.Hkv) if self.rope_all else (1, 1)
        qr = rope_apply(q, pos, self.theta, dk, 0, nq)
        kr = rope_apply(k, pos, self.theta, dk, 0, nk)
        a, ab = _mha(qr, kr, v, self.H, self.Hkv, dk, seq_len)
        o, ob = self._proj(a, pre + "self_attn.o_proj")
        x1 = (x + o).astype(F)
        h2, n2b = self._norm(x1, pre + "post_attention_layernorm.weight")
        gt, gb = self._proj(h2, pre + "mlp.gate_proj")
        up, ub = self._proj(h2, pre + "mlp.up_proj")
        sg = silu_fwd(gt)
        f, fb = self._proj((sg * up).astype(F), pre + "mlp.down_proj")
        out = (x1 + f).astype(F)

        def bwd(dout):
            dm = fb(dout)
            dh2 = gb(silu_bwd((dm * up).astype(F), gt)) + ub((dm * sg).astype(F))
            dx1 = dout + n2b(dh2.astype(F))
            da = ob(dx1)
            dq, dk_, dv = ab(da)
            dq = rope_apply(dq, pos, self.theta, dk, 0, nq, inverse=True)
            dk_ = rope_apply(dk_, pos, self.theta, dk, 0, nk, inverse=True)
            dh = qb(dq) + kb(dk_) + vb(dv)
            return (dx1 + n1b(dh.astype(F))).astype(F)
        return out, bwd

    def _gpt_block(self, x, pre, seq_len, flex):
        d = x.shape[1]
        dk = d // self.H
        if flex and self.norm == "rmsnorm":
            n1, n1b = self._norm(x, pre + "norm1.weight")
        else:
            n1, n1b = self._norm(x, pre + "ln_1.weight", pre + "ln_1.bias")
        qkv, cab = self._proj(n1, pre + "attn.c_attn")
        q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
        a, ab = _mha(q, k, v, self.H, self.H, dk, seq_len)
        o, cpb = self._proj(a, pre + "attn.c_proj")
        h = (x + o).astype(F)
        if flex and self.norm == "rmsnorm":
            n2, n2b = self._norm(h, pre + "norm2.weight")
        else:
            n2, n2b = self._norm(h, pre + "ln_2.weight", pre + "ln_2.bias")
        act = self.act if flex else "gelu"
        if act == "swiglu":
            gt, gb = self._proj(n2, pre + "mlp.gate_proj")
            up, ub = self._proj(n2, pre + "mlp.up_proj")
            sg = silu_fwd(gt)
            f, fb = self._proj((sg * up).astype(F), pre + "mlp.down_proj")

            def mlp_bwd(df):
                dm = fb(df)
                return gb(silu_bwd((dm * up).astype(F), gt)) + ub((dm * sg).astype(F))
        else:
            u, fcb = self._proj(n2, pre + "mlp.c_fc")
            z = gelu_fwd(u) if act == "gelu" else relu_fwd(u)
            f, pjb = self._proj(z, pre + "mlp.c_proj")

            def mlp_bwd(df):
                dz = pjb(df)
                return fcb(gelu_bwd(dz, u) if act == "gelu" else relu_bwd(dz, u))
        out = (h + f).astype(F)

        def bwd(dout):
            dh = dout + n2b(mlp_bwd(dout).astype(F))
            dq, dk_, dv = ab(cpb(dh))
            dn1 = cab(np.concatenate([dq, dk_, dv], axis=1).astype(F))
            return (dh + n1b(dn1)).astype(F)
        return out, bwd

    # -- the step: loss and gradients of every trainable parameter
    def step(self, ids, targets, seq_len=0) -> Tuple[float, Dict[str, np.ndarray]]:
        ids = np.asarray(ids)
        targets = np.asarray(targets)
        self.g = {}
        n = len(ids)
        sl = n if seq_len == 0 else seq_len
        pos = (np.arange(n) % sl).astype(np.int64)
        fam = self.family
        bwds = []
        if fam == "llama":
            E_name = "embed_tokens.weight"
            E = self._w(E_name)
            x = E[ids]
            for i in range(self.L):
                x, b = self._llama_block(x, i, pos, seq_len)
                bwds.append(b)
            hn, nb = self._norm(x, "norm.weight")
            if self.tie:
                logits = (hn @ E.T).astype(F)
            else:
                logits, hb = self._proj(hn, "lm_head")
        else:
            flex = fam == "flex"
            E_name = "wte.weight"
            E = self.p[E_name]
            if "wpe.weight" in self.p:
                x = (E[ids] + self.p["wpe.weight"][pos]).astype(F)
            else:
                x = (E[ids] + self.frozen["sin_table"][pos]).astype(F)
            for i in range(self.L):
                x, b = self._gpt_block(x, (f"layers.{i}." if flex else f"h.{i}."), seq_len, flex)
                bwds.append(b)
            if flex and self.norm == "rmsnorm":
                hn, nb = self._norm(x, "norm.weight")
            else:
                hn, nb = self._norm(x, "ln_f.weight", "ln_f.bias")
            if flex:
                logits, hb = self._proj(hn, "head")
            else:
                logits = (hn @ E.T).astype(F)
        loss, P = cross_entropy_fwd(logits, targets)
        dl = cross_entropy_bwd(P, targets)
        if (fam == "llama" and self.tie) or fam == "gpt2":
            dhn = (dl @ E).astype(F)
            self._acc(E_name, dl.T @ hn)
        else:
            dhn = hb(dl)
        dx = nb(dhn)
        for b in reversed(bwds):
            dx = b(dx)
        if E_name in self.p:
            self._acc(E_name, embedding_bwd(dx, ids, E.shape[0]))
        if "wpe.weight" in self.p:
            self._acc("wpe.weight", embedding_bwd(dx, pos, self.p["wpe.weight"].shape[0]))
        return float(loss), self.g


def sinusoidal_table(n_ctx: int, d: int):
    """tools/parity_model.hpp:253-259 (built in double, stored as float)."""
    t = np.zeros((n_ctx, d), dtype=F)
    for p in range(n_ctx):
        for i in range(d):
            ang = p / math.pow(10000.0, float(2 * (i // 2)) / float(d))
            t[p, i] = math.sin(ang) if i % 2 == 0 else math.cos(ang)
    return t
