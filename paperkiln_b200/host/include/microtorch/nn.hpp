#pragma once
// Module / parameter registry, the GPT-2 layer set and the optimizers.
//
// Same public surface as the reference's include/microtorch/nn.hpp:22-190 for the
// classes on the training-step path (Module, Linear, LayerNorm, Embedding,
// CausalSelfAttention, MLP, Block, GPT2, SGD, AdamW), with the same parameter names,
// storage order (Linear weight is [in, out]) and initialisation seeds, so a
// state_dict written by one loads into the other. Layers are compositions of ops::*;
// blocks call the fused forms (one attention node for all heads, bias / residual in
// the GEMM epilogue).
#include <cmath>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "microtorch/ops.hpp"

namespace microtorch {
namespace nn {

class Module {
public:
    virtual ~Module() = default;
    std::vector<std::pair<std::string, Var>> named_parameters() const;
    std::vector<Var> parameters() const;
    size_t parameter_count() const;
    std::map<std::string, Matrix> state_dict() const;
    void load_state_dict(const std::map<std::string, Matrix>& sd, bool strict = true,
                         const std::vector<std::string>& missing_ok = {});
    void train() { set_training(true); }
    void eval() { set_training(false); }
    bool training() const { return training_; }

protected:
    Var reg(const std::string& name, Matrix init);
    template <typename M, typename... A>
    std::shared_ptr<M> mod(const std::string& name, A&&... a) {
        auto m = std::make_shared<M>(std::forward<A>(a)...);
        children_.emplace_back(name, m);
        return m;
    }
    void adopt(const std::string& name, std::shared_ptr<Module> child) {
        children_.emplace_back(name, std::move(child));
    }

private:
    void collect(const std::string& prefix, std::vector<std::pair<std::string, Var>>& out) const;
    void set_training(bool t);
    std::vector<std::pair<std::string, Var>> params_;
    std::vector<std::pair<std::string, std::shared_ptr<Module>>> children_;
    bool training_ = true;
};

// Moves the parameters into one flat fp32 buffer (data), one flat fp32 gradient buffer
// and, in bf16 mode, one flat bf16 shadow buffer, in the order given, each parameter
// padded to 128 bytes. After packing, zero_grad is one memset, the optimizer step one
// kernel launch, and the gradients of consecutive parameters form one contiguous range
// (the unit a data-parallel all-reduce works on).
struct ParamPack {
    Tensor data, grad, shadow;           // flat buffers ([1, total] elements)
    std::vector<size_t> offset, count;   // per parameter, in elements
    size_t total = 0;
};
ParamPack pack_parameters(const std::vector<Var>& params);

// N(0, std) fill with std::mt19937(seed) + std::normal_distribution<float>, row-major --
// the generator every layer constructor of the reference uses (src/nn.cpp:14-21).
Matrix randn(size_t rows, size_t cols, unsigned seed, float std);

class Linear : public Module {
public:
    Linear(size_t in, size_t out, bool bias = true, unsigned seed = 0);
    Var forward(const Var& x) const;
    // y = x W + b + residual in one GEMM
    Var forward_residual(const Var& x, const Var& residual) const;
    Var W, b;
};

class LayerNorm : public Module {
public:
    explicit LayerNorm(size_t d, float eps = 1e-5f);
    Var forward(const Var& x) const;
    Var weight, bias;
    float eps;
};

class Embedding : public Module {
public:
    Embedding(size_t vocab, size_t d, unsigned seed = 0);
    Var forward(const std::vector<int>& ids) const;
    Var weight;
};

class CausalSelfAttention : public Module {
public:
    CausalSelfAttention(size_t d, size_t n_heads, unsigned seed = 0, bool causal = true);
    Var forward(const Var& x, size_t seq_len = 0) const;
    // c_proj output added to `residual` in the projection's epilogue
    Var forward_residual(const Var& x, const Var& residual, size_t seq_len) const;
    std::shared_ptr<Linear> c_attn, c_proj;
    size_t H, dk;
    bool causal;

private:
    Var heads(const Var& x, size_t seq_len) const;
};

class MLP : public Module {
public:
    MLP(size_t d, size_t hidden, unsigned seed = 0);
    Var forward(const Var& x) const;
    Var forward_residual(const Var& x, const Var& residual) const;
    std::shared_ptr<Linear> c_fc, c_proj;
};

class Block : public Module {
public:
    Block(size_t d, size_t n_heads, unsigned seed = 0);
    Var forward(const Var& x, size_t seq_len = 0) const;
    std::shared_ptr<LayerNorm> ln_1, ln_2;
    std::shared_ptr<CausalSelfAttention> attn;
    std::shared_ptr<MLP> mlp;
};

struct GPT2Config {
    size_t vocab = 50257, n_ctx = 1024, d = 768, n_layers = 12, n_heads = 12;
};

class GPT2 : public Module {
public:
    explicit GPT2(const GPT2Config& cfg, unsigned seed = 0);
    Var forward(const std::vector<int>& ids, size_t seq_len = 0) const;
    Var hidden(const std::vector<int>& ids, size_t seq_len = 0) const;  // ln_f output
    // cross_entropy(forward(ids), targets) with the head and the loss fused over row chunks.
    Var loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len = 0,
             size_t chunk_rows = 16384) const;
    GPT2Config cfg;
    bool checkpoint_blocks = false;
    std::shared_ptr<Embedding> wte, wpe;
    std::vector<std::shared_ptr<Block>> h;
    std::shared_ptr<LayerNorm> ln_f;
};

class SGD {
public:
    SGD(std::vector<Var> params, float lr, float momentum = 0.0f);
    void step();
    void zero_grad();
    float lr;

private:
    std::vector<Var> params_;
    std::vector<Tensor> vel_;
    float mu_;
};

class AdamW {
public:
    AdamW(std::vector<Var> params, float lr = 1e-3f, float beta1 = 0.9f, float beta2 = 0.999f,
          float eps = 1e-8f, float weight_decay = 0.01f);
    void step();
    void zero_grad();
    float lr;
    long steps_taken() const { return t_; }
    // Checkpointing of the optimizer: the step counter and the two moment estimates of
    // parameter `index` (position in the constructor's list), `numel` floats each, on the host.
    // The reference's trainer saves weights only (tools/mtstudio.cpp:437-441), so a resumed
    // run restarts its moments; these entries let a resumed run continue bit-identically.
    // Before the first step the moments read as zero, and imported moments are held on the
    // host until the step that creates the device state.
    void set_steps_taken(long t) { t_ = t; }
    void export_state(size_t index, float* m_h, float* v_h);
    void import_state(size_t index, const float* m_h, const float* v_h);

private:
    struct Run {  // parameters whose data, grad (and shadow) are adjacent in memory
        size_t first = 0, last = 0;  // parameter index range [first, last]
        float* p = nullptr;
        float* g = nullptr;
        void* shadow = nullptr;
        size_t n = 0;
        Tensor m, v;
    };
    void build_runs();
    bool locate(size_t index, size_t* run, size_t* offset) const;
    struct Pending { std::vector<float> m, v; };
    std::map<size_t, Pending> pending_;
    std::vector<Var> params_;
    std::vector<Run> runs_;
    bool runs_built_ = false;
    float b1_, b2_, eps_, wd_;
    long t_ = 0;
};

// Inverted dropout layer (reference: include/microtorch/nn.hpp:281-289, src/nn.cpp:479-482):
// identity in eval mode or when p == 0; in training mode each call draws a fresh mask from the
// next seed. Must not be used inside a checkpointed segment (the recomputation would draw a
// different mask), as the reference's checkpoint contract says.
class Dropout : public Module {
public:
    explicit Dropout(float p, unsigned long long seed = 0) : p_(p), next_seed_(seed) {}
    Var forward(const Var& x) const;

private:
    float p_;
    mutable unsigned long long next_seed_;
};

// ---- learning-rate schedules over an optimizer's public `lr` field ----------------------
// (reference: include/microtorch/nn.hpp:291-340; templated because SGD and AdamW share the
// field, not a base class)
// Linear warm-up over `warmup` steps, then half a cosine from the base rate down to min_lr at
// step `total`; constant min_lr afterwards.
template <typename Opt>
class CosineWarmupLR {
public:
    CosineWarmupLR(Opt& opt, size_t warmup, size_t total, float min_lr = 0.0f)
        : opt_(opt), base_(opt.lr), warmup_(warmup), total_(total), floor_(min_lr) {}
    void step() {
        ++count_;
        if (warmup_ > 0 && count_ <= warmup_) {
            opt_.lr = base_ * static_cast<float>(count_) / warmup_;
            return;
        }
        float frac = 1.0f;
        if (total_ > warmup_) frac = static_cast<float>(count_ - warmup_) / (total_ - warmup_);
        if (frac > 1.0f) frac = 1.0f;
        opt_.lr = floor_ + 0.5f * (base_ - floor_) * (1.0f + std::cos(3.14159265358979f * frac));
    }
    size_t current_step() const { return count_; }

private:
    Opt& opt_;
    float base_;
    size_t warmup_, total_, count_ = 0;
    float floor_;
};

// lr = base * gamma^(steps / step_size), the product formed by repeated multiplication.
template <typename Opt>
class StepLR {
public:
    StepLR(Opt& opt, size_t step_size, float gamma = 0.1f) : opt_(opt), base_(opt.lr), every_(step_size), gamma_(gamma) {}
    void step() {
        ++count_;
        float lr = base_;
        for (size_t k = 0; k < count_ / every_; ++k) lr *= gamma_;
        opt_.lr = lr;
    }

private:
    Opt& opt_;
    float base_;
    size_t every_, count_ = 0;
    float gamma_;
};

// ---- declared for source compatibility, not provided -------------------------------------
// Attention variants and the depth-attention stack of the reference's research models. They
// are outside the checkpointed transformer-block training path; the classes exist so that code
// written against the reference's headers (its Python bindings, tools/parity_model.hpp)
// compiles unchanged. Constructors that own ordinary Linear layers build them; every forward
// throws std::runtime_error.
class SlidingWindowAttention : public Module {
public:
    SlidingWindowAttention(size_t d, size_t n_heads, size_t window, size_t sinks = 1, unsigned seed = 0);
    Var forward(const Var& x, size_t seq_len = 0) const;
    std::shared_ptr<Linear> c_attn, c_proj;
    size_t H, dk, window, sinks;
};

class KimiLinearAttention : public Module {
public:
    KimiLinearAttention(size_t d, size_t n_heads, unsigned seed = 0, bool causal = true);
    Var forward(const Var& x, size_t seq_len = 0) const;
    std::shared_ptr<Linear> c_attn, c_proj;
    size_t H, dk;
    bool causal;
};

class AttnResStack : public Module {
public:
    AttnResStack(std::vector<std::shared_ptr<Module>> owned, std::vector<std::function<Var(const Var&)>> fns, size_t d,
                 size_t block_size = 0);
    Var forward(const Var& h1) const;
    std::vector<Var> w;
    size_t block_size;
};

}  // namespace nn
}  // namespace microtorch
