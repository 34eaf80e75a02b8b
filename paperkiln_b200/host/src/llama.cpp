// Llama-family model. Behavioural reference: src/llama.cpp of paperkiln
// (LlamaBlock 9-60, Llama 62-89).
#include "microtorch/llama.hpp"
#include "microtorch/ops_detail.hpp"
#include "pk.h"

#include <cmath>
#include <stdexcept>

namespace microtorch {
namespace nn {

Projection::Projection(size_t in, size_t out, unsigned seed, bool quantized, bool lora, size_t rank, float alpha) {
    // Same generator and seed as nn::Linear, so dense mode owns the reference's weights.
    Matrix W0 = randn(in, out, seed * 7919u + 1u, 0.02f);
    if (!quantized) {
        W = reg("weight", std::move(W0));
        return;
    }
    Wq = std::make_shared<Q8Weight>(Q8Weight::from_matrix(W0));
    if (lora) {
        A = reg("lora_A", randn(in, rank, seed * 31u + 5u, 0.02f));
        B = reg("lora_B", randn(rank, out, seed * 31u + 6u, 0.01f));
        scaling = alpha / static_cast<float>(rank);
    }
}

Var Projection::forward(const Var& x) const { return forward_residual(x, nullptr); }

Var Projection::forward_residual(const Var& x, const Var& residual) const {
    if (W) return ops::linear(x, W, nullptr, residual);
    if (!A) return ops::q8_linear(x, Wq, nullptr, residual);
    return ops::q8_lora_linear(x, Wq, A, B, scaling, nullptr, residual);
}

Var Projection::forward_rope(const Var& x, const std::vector<int>& pos, float theta_base, size_t head_dim, size_t n_rot) const {
    if (W) return ops::linear_rope(x, W, pos, theta_base, head_dim, n_rot);
    const ops::Rotary rot{pos, theta_base, head_dim, n_rot};
    if (!A) return ops::q8_linear(x, Wq, nullptr, nullptr, &rot);
    return ops::q8_lora_linear(x, Wq, A, B, scaling, nullptr, nullptr, &rot);
}

LlamaBlock::LlamaBlock(const LlamaConfig& cfg, unsigned seed)
    : H(cfg.n_heads), Hkv(cfg.n_kv_heads ? cfg.n_kv_heads : cfg.n_heads), dk(cfg.d / cfg.n_heads),
      rope_theta_(cfg.rope_theta), rms_eps_(cfg.rms_eps), rope_all_(cfg.rope_all_heads) {
    if (cfg.d % cfg.n_heads != 0) throw std::runtime_error("llama: d must divide by n_heads");
    if (H % Hkv != 0) throw std::runtime_error("llama: n_heads must be a multiple of n_kv_heads");
    const bool q = cfg.qlora;
    if (q) {  // frozen gains: plain leaves, not registered
        ln1_w = make_var(Matrix(1, cfg.d, 1.0f), false);
        ln2_w = make_var(Matrix(1, cfg.d, 1.0f), false);
    } else {
        ln1_w = reg("input_layernorm.weight", Matrix(1, cfg.d, 1.0f));
        ln2_w = reg("post_attention_layernorm.weight", Matrix(1, cfg.d, 1.0f));
    }
    const size_t r = cfg.lora_rank;
    const float a = cfg.lora_alpha;
    q_proj = mod<Projection>("self_attn.q_proj", cfg.d, H * dk, seed + 1, q, q, r, a);
    k_proj = mod<Projection>("self_attn.k_proj", cfg.d, Hkv * dk, seed + 2, q, false, r, a);
    v_proj = mod<Projection>("self_attn.v_proj", cfg.d, Hkv * dk, seed + 3, q, q, r, a);
    o_proj = mod<Projection>("self_attn.o_proj", H * dk, cfg.d, seed + 4, q, false, r, a);
    gate_proj = mod<Projection>("mlp.gate_proj", cfg.d, cfg.d_ff, seed + 5, q, false, r, a);
    up_proj = mod<Projection>("mlp.up_proj", cfg.d, cfg.d_ff, seed + 6, q, false, r, a);
    down_proj = mod<Projection>("mlp.down_proj", cfg.d_ff, cfg.d, seed + 7, q, false, r, a);
}

Var LlamaBlock::forward(const Var& x, const std::vector<int>& pos, size_t seq_len) const {
    // ---- attention sublayer (pre-RMSNorm)
    Var h = ops::rmsnorm(x, ln1_w);
    // q and k are rotated on their way out of the projection's GEMM
    Var q = q_proj->forward_rope(h, pos, rope_theta_, dk, rope_all_ ? H : 1);
    Var k = k_proj->forward_rope(h, pos, rope_theta_, dk, rope_all_ ? Hkv : 1);
    Var v = v_proj->forward(h);
    Var a = ops::attention(q, k, v, H, Hkv, seq_len, /*causal=*/true);
    Var x1 = o_proj->forward_residual(a, x);  // x + attn
    // ---- SwiGLU FFN sublayer
    Var h2 = ops::rmsnorm(x1, ln2_w);
    Var f = (gate_proj->W && up_proj->W) ? ops::linear_swiglu(h2, gate_proj->W, up_proj->W)
                                         : ops::swiglu(gate_proj->forward(h2), up_proj->forward(h2));
    return down_proj->forward_residual(f, x1);  // x1 + ffn
}

Llama::Llama(const LlamaConfig& cfg_, unsigned seed) : cfg(cfg_) {
    if (cfg.qlora) {
        embed_frozen = make_var(randn(cfg.vocab, cfg.d, (seed + 11) * 104729u + 3u, 0.02f), false);
    } else {
        embed_tokens = mod<Embedding>("embed_tokens", cfg.vocab, cfg.d, seed + 11);
    }
    for (size_t i = 0; i < cfg.n_layers; ++i)
        blocks.push_back(mod<LlamaBlock>("layers." + std::to_string(i), cfg, seed + 100 * static_cast<unsigned>(i + 1)));
    if (cfg.qlora) norm_w = make_var(Matrix(1, cfg.d, 1.0f), false);
    else norm_w = reg("norm.weight", Matrix(1, cfg.d, 1.0f));
    if (!cfg.tie_embeddings && !cfg.qlora) lm_head = mod<Linear>("lm_head", cfg.d, cfg.vocab, false, seed + 12);
}

void Llama::load_frozen_base(const std::map<std::string, Matrix>& dense) {
    if (!cfg.qlora) throw std::runtime_error("load_frozen_base: the model was not built in QLoRA mode");
    auto fetch = [&](const std::string& name, size_t rows, size_t cols) -> const Matrix& {
        auto it = dense.find(name);
        if (it == dense.end()) throw std::runtime_error("checkpoint has no tensor " + name);
        if (it->second.rows() != rows || it->second.cols() != cols)
            throw std::runtime_error("checkpoint tensor " + name + " is [" + std::to_string(it->second.rows()) + ", " +
                                     std::to_string(it->second.cols()) + "], the model wants [" +
                                     std::to_string(rows) + ", " + std::to_string(cols) + "]");
        return it->second;
    };
    struct Proj {
        const char* name;
        std::shared_ptr<Projection> LlamaBlock::*member;
    };
    static const Proj projs[] = {
        {"self_attn.q_proj", &LlamaBlock::q_proj}, {"self_attn.k_proj", &LlamaBlock::k_proj},
        {"self_attn.v_proj", &LlamaBlock::v_proj}, {"self_attn.o_proj", &LlamaBlock::o_proj},
        {"mlp.gate_proj", &LlamaBlock::gate_proj}, {"mlp.up_proj", &LlamaBlock::up_proj},
        {"mlp.down_proj", &LlamaBlock::down_proj}};
    for (int pass = 0; pass < 2; ++pass) {  // pass 0 checks, pass 1 replaces
        const Matrix& e = fetch("embed_tokens.weight", cfg.vocab, cfg.d);
        const Matrix& n = fetch("norm.weight", 1, cfg.d);
        if (pass) {
            embed_frozen = make_var(e, false);
            norm_w = make_var(n, false);
        }
        for (size_t i = 0; i < blocks.size(); ++i) {
            const std::string pre = "layers." + std::to_string(i) + ".";
            LlamaBlock& b = *blocks[i];
            const Matrix& g1 = fetch(pre + "input_layernorm.weight", 1, cfg.d);
            const Matrix& g2 = fetch(pre + "post_attention_layernorm.weight", 1, cfg.d);
            if (pass) {
                b.ln1_w = make_var(g1, false);
                b.ln2_w = make_var(g2, false);
            }
            for (const Proj& pr : projs) {
                Projection& p = *(b.*(pr.member));
                const Matrix& w = fetch(pre + pr.name + ".weight", p.Wq->rows, p.Wq->cols);
                if (pass) p.Wq = std::make_shared<Q8Weight>(Q8Weight::from_matrix(w));
            }
        }
    }
}

std::map<std::string, Matrix> Llama::merged_state() const {
    std::map<std::string, Matrix> out;
    if (!cfg.qlora) {
        for (const auto& [name, p] : named_parameters()) out[name] = p->data.host();
        return out;
    }
    out["embed_tokens.weight"] = embed_frozen->data.host();
    out["norm.weight"] = norm_w->data.host();
    for (size_t i = 0; i < blocks.size(); ++i) {
        const std::string pre = "layers." + std::to_string(i) + ".";
        const LlamaBlock& b = *blocks[i];
        out[pre + "input_layernorm.weight"] = b.ln1_w->data.host();
        out[pre + "post_attention_layernorm.weight"] = b.ln2_w->data.host();
        const std::pair<const char*, const Projection*> projs[] = {
            {"self_attn.q_proj", b.q_proj.get()}, {"self_attn.k_proj", b.k_proj.get()},
            {"self_attn.v_proj", b.v_proj.get()}, {"self_attn.o_proj", b.o_proj.get()},
            {"mlp.gate_proj", b.gate_proj.get()}, {"mlp.up_proj", b.up_proj.get()},
            {"mlp.down_proj", b.down_proj.get()}};
        for (const auto& [pname, p] : projs) {
            Tensor w = p->Wq->dequantize(DType::F32);
            if (p->A) {
                Tensor a = p->A->data.device().cast(DType::F32), bb = p->B->data.device().cast(DType::F32);
                Tensor ab = Tensor::empty(a.rows(), bb.cols(), DType::F32);
                ops::detail::gemm_raw(a, false, bb, false, ab, false);
                device::check(pk_axpy(device::stream(), PK_F32, w.ptr(), PK_F32, ab.ptr(), p->scaling,
                                      static_cast<int64_t>(ab.numel())),
                              "pk_axpy");
            }
            out[pre + pname + ".weight"] = w.to_host();
        }
    }
    return out;
}

Var Llama::hidden(const std::vector<int>& ids, size_t seq_len) const {
    const size_t sl = seq_len == 0 ? ids.size() : seq_len;
    if (sl == 0 || ids.size() % sl != 0) throw std::runtime_error("ids not a multiple of seq_len");
    std::vector<int> pos(ids.size());
    for (size_t i = 0; i < pos.size(); ++i) pos[i] = static_cast<int>(i % sl);
    const Var& table = cfg.qlora ? embed_frozen : embed_tokens->weight;
    Var h = ops::embedding(table, ids);
    for (const auto& b : blocks) {
        h = checkpoint_blocks && grad_enabled()
                ? checkpoint([b, pos, seq_len](const Var& in) { return b->forward(in, pos, seq_len); }, h)
                : b->forward(h, pos, seq_len);
    }
    return ops::rmsnorm(h, norm_w);
}

Var Llama::forward(const std::vector<int>& ids, size_t seq_len) const {
    Var h = hidden(ids, seq_len);
    if (lm_head) return lm_head->forward(h);
    // Tied head: logits = h E^T; the embedding receives gradient from the gather and
    // from this GEMM (src/llama.cpp:85-88). No transposed copy of E is made.
    const Var& table = cfg.qlora ? embed_frozen : embed_tokens->weight;
    return ops::linear(h, table, nullptr, nullptr, /*transposed_w=*/true);
}

Var Llama::loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len, size_t chunk_rows) const {
    if (lm_head && lm_head->b) return ops::cross_entropy(forward(ids, seq_len), targets);
    Var h = hidden(ids, seq_len);
    if (lm_head) return ops::linear_cross_entropy(h, lm_head->W, false, targets, chunk_rows);
    const Var& table = cfg.qlora ? embed_frozen : embed_tokens->weight;
    return ops::linear_cross_entropy(h, table, true, targets, chunk_rows);
}

}  // namespace nn
}  // namespace microtorch
