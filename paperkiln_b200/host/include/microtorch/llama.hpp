#pragma once
// Llama-family model: RMSNorm, rotary embedding, SwiGLU, no biases; parameter names
// follow HF LlamaForCausalLM ("layers.N.self_attn.q_proj.weight", ...).
//
// Reference: include/microtorch/llama.hpp:14-51 and src/llama.cpp:9-89. LlamaConfig
// keeps the reference's fields and adds, with defaults that reproduce the reference:
//   n_kv_heads      grouped-query attention (0 = n_heads, the reference's layout)
//   rope_all_heads  false = the reference's behaviour, which rotates only the first
//                   head of q and of k (src/ops.cpp:495-511 applied to the fused
//                   [T,3d] layout); true = every head is rotated
//   qlora           frozen Q8_0 base weights (embedding and norm gains frozen too)
//                   with trainable LoRA adapters on q_proj and v_proj
// The block is written against the fused ops: one attention node for all heads,
// in-place rotary on the projection outputs, residual adds in the GEMM epilogues.
#include "microtorch/nn.hpp"
#include "microtorch/quant.hpp"

namespace microtorch {
namespace nn {

struct LlamaConfig {
    size_t vocab = 4096, d = 128, n_layers = 2, n_heads = 4;
    size_t d_ff = 512;
    size_t n_ctx = 256;
    float rms_eps = 1e-6f;  // unused, as in the reference: ops::rmsnorm fixes eps = 1e-5
    float rope_theta = 10000.0f;
    bool tie_embeddings = true;
    size_t n_kv_heads = 0;
    bool rope_all_heads = false;
    bool qlora = false;
    size_t lora_rank = 16;
    float lora_alpha = 32.0f;
};

// A projection that is either a trainable dense Linear or a frozen Q8_0 weight with an
// optional LoRA side path (QLoRA mode).
class Projection : public Module {
public:
    Projection(size_t in, size_t out, unsigned seed, bool quantized, bool lora, size_t rank, float alpha);
    Var forward(const Var& x) const;
    Var forward_residual(const Var& x, const Var& residual) const;
    // forward(x) with the rotary embedding applied to the first n_rot heads of the result
    Var forward_rope(const Var& x, const std::vector<int>& pos, float theta_base, size_t head_dim, size_t n_rot) const;
    Var W;     // dense mode
    Var A, B;  // LoRA (QLoRA mode, q/v projections)
    std::shared_ptr<Q8Weight> Wq;
    float scaling = 0.0f;
};

class LlamaBlock : public Module {
public:
    LlamaBlock(const LlamaConfig& cfg, unsigned seed);
    Var forward(const Var& x, const std::vector<int>& positions, size_t seq_len = 0) const;

    Var ln1_w, ln2_w;
    std::shared_ptr<Projection> q_proj, k_proj, v_proj, o_proj;
    std::shared_ptr<Projection> gate_proj, up_proj, down_proj;
    size_t H, Hkv, dk;
    float rope_theta_, rms_eps_;
    bool rope_all_;
};

class Llama : public Module {
public:
    explicit Llama(const LlamaConfig& cfg, unsigned seed = 0);
    Var forward(const std::vector<int>& ids, size_t seq_len = 0) const;
    // Final-norm output, before the vocabulary projection.
    Var hidden(const std::vector<int>& ids, size_t seq_len = 0) const;
    // cross_entropy(forward(ids), targets) with the head and the loss fused over row chunks.
    Var loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len = 0,
             size_t chunk_rows = 16384) const;

    // QLoRA mode: takes the frozen base (projections, embedding, norm gains) from the tensors of
    // a DENSE model of the same shape, named as that model registers them ("layers.0.self_attn.
    // q_proj.weight", "embed_tokens.weight", "norm.weight", ...); the projections are quantised
    // to Q8_0 on the device. Every tensor is checked before the first one is replaced. The LoRA
    // matrices are parameters and are not touched. The reference builds its QLoRA layers from
    // fp32 weights the same way (QLoRALinear's constructor, src/quant.cpp:102-110).
    void load_frozen_base(const std::map<std::string, Matrix>& dense);
    // The inverse direction: the tensors of the equivalent DENSE model, under that model's names,
    // with every projection merged as deq(Wq) + (alpha / r) A B in fp32 on the device (the
    // reference's merged_weight, src/quant.cpp:82-89). Dense models return their parameters.
    std::map<std::string, Matrix> merged_state() const;

    LlamaConfig cfg;
    bool checkpoint_blocks = false;
    std::shared_ptr<Embedding> embed_tokens;  // dense mode
    Var embed_frozen;                          // QLoRA mode: not a registered parameter
    std::vector<std::shared_ptr<LlamaBlock>> blocks;
    Var norm_w;
    std::shared_ptr<Linear> lm_head;  // null when tied
};

}  // namespace nn
}  // namespace microtorch
