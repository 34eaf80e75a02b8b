#pragma once
// Flexible-depth LM family: norm (layernorm | rmsnorm) x MLP activation (gelu | relu |
// swiglu) x position encoding (learned | sinusoidal), pre-norm wiring, untied head.
//
// Reference: tools/parity_model.hpp:192-294 of paperkiln (FlexConfig, FlexBlock, FlexLM;
// same parameter names and seed layout). The reference's FlexLM has no per-block
// checkpoint switch; `checkpoint_blocks` here wraps each block exactly as nn::GPT2 does
// (src/nn.cpp:249-253).
#include <string>

#include "microtorch/nn.hpp"

namespace microtorch {
namespace parity {

struct FlexConfig {
    size_t vocab = 0, d = 128, n_layers = 2, n_heads = 4, d_ff = 512, n_ctx = 128;
    std::string norm = "layernorm";
    std::string act = "gelu";
    std::string pos = "learned";
};

class FlexBlock : public nn::Module {
public:
    FlexBlock(const FlexConfig& c, unsigned s);
    Var forward(const Var& x, size_t seq_len = 0) const;

    std::string norm_, act_;
    std::shared_ptr<nn::LayerNorm> ln1, ln2;
    Var n1_w, n2_w;
    std::shared_ptr<nn::CausalSelfAttention> attn;
    std::shared_ptr<nn::MLP> mlp;
    std::shared_ptr<nn::Linear> gate, up, down, fc, proj;
};

class FlexLM : public nn::Module {
public:
    FlexLM(const FlexConfig& c, unsigned seed);
    Var forward(const std::vector<int>& ids, size_t seq_len = 0) const;
    Var hidden(const std::vector<int>& ids, size_t seq_len = 0) const;  // final-norm output
    // cross_entropy(forward(ids), targets) with the head and the loss fused over row chunks.
    Var loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len = 0,
             size_t chunk_rows = 16384) const;

    FlexConfig cfg;
    bool checkpoint_blocks = false;
    std::shared_ptr<nn::Embedding> wte, wpe;
    Matrix sin_table;
    std::vector<std::shared_ptr<FlexBlock>> blocks;
    std::shared_ptr<nn::LayerNorm> ln_f_ln;
    Var ln_f_w;
    std::shared_ptr<nn::Linear> head;
};

}  // namespace parity
}  // namespace microtorch
