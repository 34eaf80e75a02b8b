"""GGUF export on CPU: the host library's exporter against files written by the unmodified
reference exporter (tests/golden/ref_export_*.gguf; generator tests/golden/gguf_ref_writer.cpp,
reference src/gguf.cpp:27-166) from the same seeded tensors -- byte for byte -- and against the
GGUF v3 layout read back field by field."""
import ctypes
import struct
from pathlib import Path

import numpy as np
import pytest

from paperkiln_b200._capi import libmt
from tests.test_safetensors_cpu import write_file

GOLDEN = Path(__file__).resolve().parent / "golden"
TOKENS = ["<unk>", "<s>", "a", "b", "cc", "ddd", "e", "f", "g", "h", "ii"]
SPEC = "name=tiny;ctx=64;d=8;layers=2;dff=16;heads=2;kv_heads=1;vocab=11;eps=1e-5;theta=10000"


def make_state(in_out: bool):
    """Seeded tensors of a 2-block model; projections [in, out] or [out, in]."""
    rng = np.random.RandomState(11)
    d, dkv, ff, vocab = 8, 4, 16, 11

    def proj(i, o):
        w = rng.randn(i, o).astype("<f4")
        return w if in_out else np.ascontiguousarray(w.T)

    t = [("embed_tokens.weight", rng.randn(vocab, d).astype("<f4")), ("norm.weight", rng.randn(d).astype("<f4"))]
    for l in range(2):
        p = f"layers.{l}."
        t += [(p + "self_attn.q_proj.weight", proj(d, d)), (p + "self_attn.k_proj.weight", proj(d, dkv)),
              (p + "self_attn.v_proj.weight", proj(d, dkv)), (p + "self_attn.o_proj.weight", proj(d, d)),
              (p + "mlp.gate_proj.weight", proj(d, ff)), (p + "mlp.up_proj.weight", proj(d, ff)),
              (p + "mlp.down_proj.weight", proj(ff, d)), (p + "input_layernorm.weight", rng.randn(d).astype("<f4")),
              (p + "post_attention_layernorm.weight", rng.randn(d).astype("<f4"))]
    if not in_out:
        t += [("model.lm_head.weight", proj(d, vocab)), ("layers.0.self_attn.q_proj.bias", rng.randn(d).astype("<f4"))]
    return t


def export(tmp_path, in_out, tokens):
    src = tmp_path / "state.safetensors"
    write_file(src, [(n, "F32", a) for n, a in make_state(in_out)])
    tok = None
    if tokens:
        tok = tmp_path / "tokens.txt"
        tok.write_text("\n".join(TOKENS) + "\n")
    dst = tmp_path / "out.gguf"
    n = ctypes.c_int64(-1)
    rc = libmt().mt_gguf_export_llama(str(src).encode(), str(dst).encode(), (SPEC + f";in_out={int(in_out)}").encode(),
                                      str(tok).encode() if tok else None, ctypes.byref(n))
    assert rc == 0, libmt().mt_last_error()
    return dst, n.value, src


class Reader:
    def __init__(self, raw):
        self.raw, self.at = raw, 0

    def take(self, fmt):
        v = struct.unpack_from("<" + fmt, self.raw, self.at)
        self.at += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def text(self):
        n = self.take("Q")
        s = self.raw[self.at:self.at + n].decode()
        self.at += n
        return s

    def value(self, t):
        if t == 4:
            return self.take("I")
        if t == 6:
            return self.take("f")
        if t == 8:
            return self.text()
        assert t == 9
        et, n = self.take("I"), self.take("Q")
        return [self.value(et) for _ in range(n)]


def parse(path):
    r = Reader(open(path, "rb").read())
    assert r.raw[:4] == b"GGUF" and r.take("I") == 0x46554747 and r.take("I") == 3
    n_t, n_kv = r.take("Q"), r.take("Q")
    kv = {}
    for _ in range(n_kv):
        k = r.text()
        kv[k] = r.value(r.take("I"))
    infos = []
    for _ in range(n_t):
        name = r.text()
        dims = [r.take("Q") for _ in range(r.take("I"))]
        typ, off = r.take("I"), r.take("Q")
        infos.append((name, dims, typ, off))
    data0 = (r.at + 31) // 32 * 32
    assert not any(r.raw[r.at:data0])
    tensors = {}
    for name, dims, typ, off in infos:
        assert typ == 0 and off % 32 == 0
        n = int(np.prod(dims))
        tensors[name] = np.frombuffer(r.raw[data0 + off:data0 + off + 4 * n], dtype="<f4").reshape(dims)
    return kv, tensors, [i[0] for i in infos]


@pytest.mark.parametrize("in_out,tokens,gold,unmapped", [(True, True, "ref_export_in_out.gguf", 0),
                                                         (False, False, "ref_export_out_in.gguf", 1)])
def test_export_matches_reference_bytes(tmp_path, in_out, tokens, gold, unmapped):
    dst, n, _ = export(tmp_path, in_out, tokens)
    assert n == unmapped
    assert open(dst, "rb").read() == open(GOLDEN / gold, "rb").read()


def test_layout_field_by_field(tmp_path):
    dst, _, _ = export(tmp_path, True, True)
    kv, tensors, order = parse(dst)
    assert list(kv)[:4] == ["general.architecture", "general.name", "general.alignment", "llama.context_length"]
    assert kv["general.architecture"] == "llama" and kv["general.name"] == "tiny" and kv["general.alignment"] == 32
    assert kv["llama.embedding_length"] == 8 and kv["llama.block_count"] == 2 and kv["llama.feed_forward_length"] == 16
    assert kv["llama.attention.head_count"] == 2 and kv["llama.attention.head_count_kv"] == 1
    assert kv["llama.vocab_size"] == 11 and kv["llama.rope.dimension_count"] == 4
    assert abs(kv["llama.attention.layer_norm_rms_epsilon"] - 1e-5) < 1e-12 and kv["llama.rope.freq_base"] == 10000.0
    assert kv["tokenizer.ggml.tokens"] == TOKENS and kv["tokenizer.ggml.scores"] == [0.0] * 11
    assert kv["tokenizer.ggml.model"] == "word" and kv["tokenizer.ggml.bos_token_id"] == 1
    state = dict(make_state(True))
    assert order[0] == "token_embd.weight" and order[-1] == "output_norm.weight" and len(order) == 2 + 9 * 2
    assert order[1:10] == ["blk.0.attn_q.weight", "blk.0.attn_k.weight", "blk.0.attn_v.weight",
                           "blk.0.attn_output.weight", "blk.0.attn_norm.weight", "blk.0.ffn_gate.weight",
                           "blk.0.ffn_up.weight", "blk.0.ffn_down.weight", "blk.0.ffn_norm.weight"]
    assert np.array_equal(tensors["token_embd.weight"], state["embed_tokens.weight"])
    # [in, out] weights leave as [out][in] values
    assert np.array_equal(tensors["blk.1.attn_k.weight"], state["layers.1.self_attn.k_proj.weight"].T)
    assert np.array_equal(tensors["blk.0.ffn_down.weight"], state["layers.0.mlp.down_proj.weight"].T)
    assert np.array_equal(tensors["output_norm.weight"], state["norm.weight"])


def test_export_errors(tmp_path):
    src = tmp_path / "state.safetensors"
    write_file(src, [(n, "F32", a) for n, a in make_state(True) if n != "layers.1.mlp.up_proj.weight"])
    n = ctypes.c_int64(0)
    rc = libmt().mt_gguf_export_llama(str(src).encode(), str(tmp_path / "o.gguf").encode(), (SPEC + ";in_out=1").encode(),
                                      None, ctypes.byref(n))
    assert rc != 0 and b"missing tensor layers.1.mlp.up_proj.weight" in libmt().mt_last_error()
    rc = libmt().mt_gguf_export_llama(str(src).encode(), str(tmp_path / "o.gguf").encode(), b"d=8;layers=2", None,
                                      ctypes.byref(n))
    assert rc != 0 and b"must all be set" in libmt().mt_last_error()
