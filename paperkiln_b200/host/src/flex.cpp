// Flex LM family. Behavioural reference: tools/parity_model.hpp:199-294 of paperkiln.
#include "microtorch/flex.hpp"

#include <cmath>
#include <stdexcept>

namespace microtorch {
namespace parity {

FlexBlock::FlexBlock(const FlexConfig& c, unsigned s) : norm_(c.norm), act_(c.act) {
    if (norm_ == "layernorm") {
        ln1 = mod<nn::LayerNorm>("ln_1", c.d);
        ln2 = mod<nn::LayerNorm>("ln_2", c.d);
    } else if (norm_ == "rmsnorm") {
        n1_w = reg("norm1.weight", Matrix(1, c.d, 1.0f));
        n2_w = reg("norm2.weight", Matrix(1, c.d, 1.0f));
    } else {
        throw std::runtime_error("flex: norm must be layernorm or rmsnorm");
    }
    attn = mod<nn::CausalSelfAttention>("attn", c.d, c.n_heads, s);
    if (act_ == "swiglu") {
        gate = mod<nn::Linear>("mlp.gate_proj", c.d, c.d_ff, false, s + 3 + 17);
        up = mod<nn::Linear>("mlp.up_proj", c.d, c.d_ff, false, s + 3 + 18);
        down = mod<nn::Linear>("mlp.down_proj", c.d_ff, c.d, false, s + 3 + 19);
    } else if (act_ == "gelu") {
        mlp = mod<nn::MLP>("mlp", c.d, c.d_ff, s + 3);
    } else if (act_ == "relu") {
        fc = mod<nn::Linear>("mlp.c_fc", c.d, c.d_ff, true, s + 3 + 17);
        proj = mod<nn::Linear>("mlp.c_proj", c.d_ff, c.d, true, s + 3 + 19);
    } else {
        throw std::runtime_error("flex: act must be gelu, relu or swiglu");
    }
}

Var FlexBlock::forward(const Var& x, size_t seq_len) const {
    Var n1 = ln1 ? ln1->forward(x) : ops::rmsnorm(x, n1_w);
    Var h = attn->forward_residual(n1, x, seq_len);
    Var n = ln2 ? ln2->forward(h) : ops::rmsnorm(h, n2_w);
    if (mlp) return mlp->forward_residual(n, h);
    if (gate) return down->forward_residual(ops::swiglu(gate->forward(n), up->forward(n)), h);
    return proj->forward_residual(ops::relu(fc->forward(n)), h);
}

FlexLM::FlexLM(const FlexConfig& c, unsigned seed) : cfg(c) {
    wte = mod<nn::Embedding>("wte", c.vocab, c.d, seed + 1);
    if (c.pos == "learned") {
        wpe = mod<nn::Embedding>("wpe", c.n_ctx, c.d, seed + 2);
    } else if (c.pos == "sinusoidal") {  // fixed table, built in double then cast
        sin_table = Matrix(c.n_ctx, c.d);
        for (size_t p = 0; p < c.n_ctx; ++p)
            for (size_t i = 0; i < c.d; ++i) {
                const double angle = p / std::pow(10000.0, double(2 * (i / 2)) / double(c.d));
                sin_table(p, i) = static_cast<float>(i % 2 == 0 ? std::sin(angle) : std::cos(angle));
            }
    } else {
        throw std::runtime_error("flex: pos must be learned or sinusoidal");
    }
    for (size_t b = 0; b < c.n_layers; ++b)
        blocks.push_back(mod<FlexBlock>("layers." + std::to_string(b), c, seed + 10 * static_cast<unsigned>(b + 1)));
    ln_f_ln = c.norm == "layernorm" ? mod<nn::LayerNorm>("ln_f", c.d) : nullptr;
    if (!ln_f_ln) ln_f_w = reg("norm.weight", Matrix(1, c.d, 1.0f));
    head = mod<nn::Linear>("head", c.d, c.vocab, false, seed + 99);
}

Var FlexLM::hidden(const std::vector<int>& ids, size_t seq_len) const {
    const size_t sl = seq_len == 0 ? ids.size() : seq_len;
    if (sl == 0 || ids.size() % sl != 0) throw std::runtime_error("ids not a multiple of seq_len");
    if (sl > cfg.n_ctx) throw std::runtime_error("sequence too long");
    std::vector<int> pos(ids.size());
    for (size_t i = 0; i < pos.size(); ++i) pos[i] = static_cast<int>(i % sl);
    Var h;
    if (wpe) {
        h = ops::add(wte->forward(ids), wpe->forward(pos));
    } else {
        // rows of the fixed table gathered on the GPU (a frozen embedding)
        Var table = make_var(sin_table, false);
        h = ops::add(wte->forward(ids), ops::embedding(table, pos));
    }
    for (auto& b : blocks) {
        h = checkpoint_blocks && grad_enabled()
                ? checkpoint([b, seq_len](const Var& in) { return b->forward(in, seq_len); }, h)
                : b->forward(h, seq_len);
    }
    return ln_f_ln ? ln_f_ln->forward(h) : ops::rmsnorm(h, ln_f_w);
}

Var FlexLM::forward(const std::vector<int>& ids, size_t seq_len) const { return head->forward(hidden(ids, seq_len)); }

Var FlexLM::loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len, size_t chunk_rows) const {
    if (head->b) return ops::cross_entropy(forward(ids, seq_len), targets);
    return ops::linear_cross_entropy(hidden(ids, seq_len), head->W, false, targets, chunk_rows);
}

}  // namespace parity
}  // namespace microtorch
