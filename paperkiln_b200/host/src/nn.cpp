// Module registry, GPT-2 layers, optimizers and parameter packing.
// Behavioural reference: src/nn.cpp of paperkiln (Module 27-96, layers 100-257,
// SGD 261-291, AdamW 293-325).
#include "microtorch/nn.hpp"

#include <random>
#include <stdexcept>

#include "pk.h"

namespace microtorch {
namespace nn {

using device::check;

Matrix randn(size_t r, size_t c, unsigned seed, float std) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.0f, std);
    Matrix m(r, c);
    float* p = m.data();
    for (size_t i = 0; i < r * c; ++i) p[i] = dist(gen);
    return m;
}

// ---------------------------------------------------------------- Module
Var Module::reg(const std::string& name, Matrix init) {
    Var v = make_var(std::move(init), true);
    v->is_param = true;
    params_.emplace_back(name, v);
    return v;
}

void Module::collect(const std::string& prefix, std::vector<std::pair<std::string, Var>>& out) const {
    for (const auto& np : params_) out.emplace_back(prefix + np.first, np.second);
    for (const auto& nc : children_) nc.second->collect(prefix + nc.first + ".", out);
}

std::vector<std::pair<std::string, Var>> Module::named_parameters() const {
    std::vector<std::pair<std::string, Var>> out;
    collect("", out);
    return out;
}

std::vector<Var> Module::parameters() const {
    std::vector<Var> out;
    for (auto& np : named_parameters()) out.push_back(np.second);
    return out;
}

size_t Module::parameter_count() const {
    size_t n = 0;
    for (const auto& p : parameters()) n += p->data.rows() * p->data.cols();
    return n;
}

std::map<std::string, Matrix> Module::state_dict() const {
    std::map<std::string, Matrix> sd;
    for (auto& np : named_parameters()) sd.emplace(np.first, np.second->data.host());
    return sd;
}

void Module::load_state_dict(const std::map<std::string, Matrix>& sd, bool strict,
                             const std::vector<std::string>& missing_ok) {
    auto named = named_parameters();
    std::map<std::string, Var> byname(named.begin(), named.end());
    for (const auto& kv : sd) {
        auto it = byname.find(kv.first);
        if (it == byname.end()) {
            if (strict) throw std::runtime_error("load_state_dict: unexpected key " + kv.first);
            continue;
        }
        if (kv.second.rows() != it->second->data.rows() || kv.second.cols() != it->second->data.cols())
            throw std::runtime_error("load_state_dict: shape mismatch at " + kv.first);
        it->second->data = kv.second;
    }
    if (strict) {
        for (auto& np : named) {
            bool ok = sd.count(np.first) > 0;
            for (const auto& allow : missing_ok) ok = ok || np.first == allow;
            if (!ok) throw std::runtime_error("load_state_dict: missing key " + np.first);
        }
    }
}

void Module::set_training(bool t) {
    training_ = t;
    for (auto& nc : children_) nc.second->set_training(t);
}

// ---------------------------------------------------------------- packing
ParamPack pack_parameters(const std::vector<Var>& params) {
    ParamPack pk;
    const size_t align = 32;  // elements: 128 bytes of fp32, 64 bytes of bf16
    for (const auto& p : params) {
        pk.offset.push_back(pk.total);
        const size_t n = p->data.rows() * p->data.cols();
        pk.count.push_back(n);
        pk.total += (n + align - 1) / align * align;
    }
    if (pk.total == 0) return pk;
    const bool lowp = device::compute_dtype() == DType::BF16;
    pk.data = Tensor::zeros(1, pk.total, DType::F32, device::Pool::Persistent);
    pk.grad = Tensor::zeros(1, pk.total, DType::F32, device::Pool::Persistent);
    if (lowp) pk.shadow = Tensor::zeros(1, pk.total, DType::BF16, device::Pool::Persistent);
    void* s = device::stream();
    for (size_t i = 0; i < params.size(); ++i) {
        const Var& p = params[i];
        const size_t r = p->data.rows(), c = p->data.cols();
        Tensor win = pk.data.view(pk.offset[i], r, c);
        const Tensor& cur = p->data.device();
        check(pk_memcpy_d2d(win.ptr(), cur.ptr(), win.nbytes(), s), "pk_memcpy_d2d");
        p->data.set_device(win);
        p->grad.reset();
        p->grad_home = pk.grad.view(pk.offset[i], r, c);
        if (lowp) {
            p->shadow = pk.shadow.view(pk.offset[i], r, c);
            check(pk_cast(s, PK_F32, win.ptr(), PK_BF16, p->shadow.ptr(), static_cast<int64_t>(r * c)), "pk_cast");
            p->shadow_version = p->data.version();
        }
    }
    return pk;
}

// ---------------------------------------------------------------- layers
Linear::Linear(size_t in, size_t out, bool bias, unsigned seed) {
    W = reg("weight", randn(in, out, seed * 7919u + 1u, 0.02f));
    if (bias) b = reg("bias", Matrix(1, out));
}
Var Linear::forward(const Var& x) const { return ops::linear(x, W, b); }
Var Linear::forward_residual(const Var& x, const Var& residual) const { return ops::linear(x, W, b, residual); }

LayerNorm::LayerNorm(size_t d, float e) : eps(e) {
    weight = reg("weight", Matrix(1, d, 1.0f));
    bias = reg("bias", Matrix(1, d));
}
Var LayerNorm::forward(const Var& x) const { return ops::layernorm(x, weight, bias, eps); }

Embedding::Embedding(size_t vocab, size_t d, unsigned seed) {
    weight = reg("weight", randn(vocab, d, seed * 104729u + 3u, 0.02f));
}
Var Embedding::forward(const std::vector<int>& ids) const { return ops::embedding(weight, ids); }

// reference: src/nn.cpp:479-482
Var Dropout::forward(const Var& x) const {
    if (!training() || p_ == 0.0f) return x;
    return ops::dropout(x, p_, next_seed_++);
}

CausalSelfAttention::CausalSelfAttention(size_t d, size_t n_heads, unsigned seed, bool causal_)
    : H(n_heads), dk(d / n_heads), causal(causal_) {
    if (d % n_heads != 0) throw std::runtime_error("attention: d must divide by n_heads");
    c_attn = mod<Linear>("c_attn", d, 3 * d, true, seed + 11);
    c_proj = mod<Linear>("c_proj", d, d, true, seed + 13);
}

Var CausalSelfAttention::heads(const Var& x, size_t seq_len) const {
    Var qkv = c_attn->forward(x);  // [T, 3d]: q | k | v, heads contiguous inside each, read in place
    return ops::attention_packed(qkv, H, seq_len, causal);
}
Var CausalSelfAttention::forward(const Var& x, size_t seq_len) const { return c_proj->forward(heads(x, seq_len)); }
Var CausalSelfAttention::forward_residual(const Var& x, const Var& residual, size_t seq_len) const {
    return c_proj->forward_residual(heads(x, seq_len), residual);
}

MLP::MLP(size_t d, size_t hidden, unsigned seed) {
    c_fc = mod<Linear>("c_fc", d, hidden, true, seed + 17);
    c_proj = mod<Linear>("c_proj", hidden, d, true, seed + 19);
}
Var MLP::forward(const Var& x) const { return c_proj->forward(ops::gelu(c_fc->forward(x))); }
Var MLP::forward_residual(const Var& x, const Var& residual) const {
    return c_proj->forward_residual(ops::gelu(c_fc->forward(x)), residual);
}

Block::Block(size_t d, size_t n_heads, unsigned seed) {
    ln_1 = mod<LayerNorm>("ln_1", d);
    attn = mod<CausalSelfAttention>("attn", d, n_heads, seed + 23);
    ln_2 = mod<LayerNorm>("ln_2", d);
    mlp = mod<MLP>("mlp", d, 4 * d, seed + 29);
}
Var Block::forward(const Var& x, size_t seq_len) const {
    Var y = attn->forward_residual(ln_1->forward(x), x, seq_len);
    return mlp->forward_residual(ln_2->forward(y), y);
}

GPT2::GPT2(const GPT2Config& c, unsigned seed) : cfg(c) {
    wte = mod<Embedding>("wte", cfg.vocab, cfg.d, seed + 31);
    wpe = mod<Embedding>("wpe", cfg.n_ctx, cfg.d, seed + 37);
    for (size_t l = 0; l < cfg.n_layers; ++l)
        h.push_back(mod<Block>("h." + std::to_string(l), cfg.d, cfg.n_heads, seed + 41 + static_cast<unsigned>(l)));
    ln_f = mod<LayerNorm>("ln_f", cfg.d);
}

Var GPT2::hidden(const std::vector<int>& ids, size_t seq_len) const {
    const size_t sl = seq_len == 0 ? ids.size() : seq_len;
    if (sl > cfg.n_ctx) throw std::runtime_error("sequence too long");
    if (sl == 0 || ids.size() % sl != 0) throw std::runtime_error("ids not a multiple of seq_len");
    std::vector<int> pos(ids.size());
    for (size_t i = 0; i < pos.size(); ++i) pos[i] = static_cast<int>(i % sl);
    Var x = ops::add(wte->forward(ids), wpe->forward(pos));
    for (const auto& blk : h) {
        x = checkpoint_blocks && grad_enabled()
                ? checkpoint([blk, seq_len](const Var& in) { return blk->forward(in, seq_len); }, x)
                : blk->forward(x, seq_len);
    }
    return ln_f->forward(x);
}

Var GPT2::forward(const std::vector<int>& ids, size_t seq_len) const {
    return ops::linear(hidden(ids, seq_len), wte->weight, nullptr, nullptr, /*transposed_w=*/true);  // tied head: x wte^T
}

Var GPT2::loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len, size_t chunk_rows) const {
    return ops::linear_cross_entropy(hidden(ids, seq_len), wte->weight, true, targets, chunk_rows);
}

// ---------------------------------------------------------------- optimizers
SGD::SGD(std::vector<Var> params, float lr_, float momentum) : lr(lr_), params_(std::move(params)), mu_(momentum) {}

void SGD::step() {
    void* s = device::stream();
    if (mu_ != 0.0f && vel_.empty())
        for (const auto& p : params_) vel_.push_back(Tensor::zeros(p->data.rows(), p->data.cols(), DType::F32, device::Pool::Persistent));
    for (size_t k = 0; k < params_.size(); ++k) {
        Var& p = params_[k];
        if (p->grad.empty()) continue;
        Tensor g = p->grad.device().cast(DType::F32);
        const Tensor& d = p->data.device();
        const int64_t n = static_cast<int64_t>(d.numel());
        if (mu_ != 0.0f) {
            Tensor& v = vel_[k];
            check(pk_scale(s, PK_F32, v.ptr(), mu_, v.ptr(), n), "pk_scale");      // v = mu v
            check(pk_axpy(s, PK_F32, v.ptr(), PK_F32, g.ptr(), 1.0f, n), "pk_axpy");  // v += g
            check(pk_axpy(s, PK_F32, d.ptr(), PK_F32, v.ptr(), -lr, n), "pk_axpy");
        } else {
            check(pk_axpy(s, PK_F32, d.ptr(), PK_F32, g.ptr(), -lr, n), "pk_axpy");
        }
        p->data.mark_device_modified();
    }
}
void SGD::zero_grad() { microtorch::zero_grad(params_); }

AdamW::AdamW(std::vector<Var> params, float lr_, float b1, float b2, float eps, float wd)
    : lr(lr_), params_(std::move(params)), b1_(b1), b2_(b2), eps_(eps), wd_(wd) {}

// Groups parameters whose fp32 data, gradient and bf16 shadow are laid out back to back
// (packed models: all of them) so that one kernel launch updates the whole group.
void AdamW::build_runs() {
    std::vector<bool> covered(params_.size(), false);
    for (const auto& r : runs_)
        for (size_t i = r.first; i <= r.last; ++i) covered[i] = true;
    size_t i = 0;
    while (i < params_.size()) {
        if (covered[i] || params_[i]->grad.empty() || params_[i]->data.device().dtype() != DType::F32 ||
            params_[i]->grad.device().dtype() != DType::F32) {
            ++i;
            continue;
        }
        Run r;
        r.first = r.last = i;
        r.p = params_[i]->data.device().f32();
        r.g = params_[i]->grad.device().f32();
        r.shadow = params_[i]->shadow.defined() && params_[i]->shadow.dtype() == DType::BF16 ? params_[i]->shadow.ptr() : nullptr;
        r.n = params_[i]->data.device().numel();
        size_t j = i + 1;
        while (j < params_.size() && !covered[j] && !params_[j]->grad.empty() && params_[j]->grad_home.defined() &&
               params_[i]->grad_home.defined()) {
            float* pj = params_[j]->data.device().f32();
            float* gj = params_[j]->grad.device().f32();
            const ptrdiff_t dp = pj - r.p, dg = gj - r.g;
            if (dp != dg || dp < static_cast<ptrdiff_t>(r.n) || dp - static_cast<ptrdiff_t>(r.n) >= 32) break;
            const bool sh = params_[j]->shadow.defined() && params_[j]->shadow.dtype() == DType::BF16;
            if (sh != (r.shadow != nullptr)) break;
            if (sh && (static_cast<char*>(params_[j]->shadow.ptr()) - static_cast<char*>(r.shadow)) != dp * 2) break;
            r.n = static_cast<size_t>(dp) + params_[j]->data.device().numel();
            r.last = j;
            ++j;
        }
        r.m = Tensor::zeros(1, r.n, DType::F32, device::Pool::Persistent);
        r.v = Tensor::zeros(1, r.n, DType::F32, device::Pool::Persistent);
        runs_.push_back(std::move(r));
        // moments imported before this state existed
        const Run& made = runs_.back();
        for (size_t k = made.first; k <= made.last; ++k) {
            auto it = pending_.find(k);
            if (it == pending_.end()) continue;
            const size_t off = static_cast<size_t>(params_[k]->data.device().f32() - made.p);
            const size_t bytes = it->second.m.size() * sizeof(float);
            check(pk_memcpy_h2d(made.m.f32() + off, it->second.m.data(), bytes, device::stream()), "pk_memcpy_h2d");
            check(pk_memcpy_h2d(made.v.f32() + off, it->second.v.data(), bytes, device::stream()), "pk_memcpy_h2d");
            device::synchronize();  // the host vectors go away below
            pending_.erase(it);
        }
        i = j;
    }
}

bool AdamW::locate(size_t index, size_t* run, size_t* offset) const {
    for (size_t r = 0; r < runs_.size(); ++r) {
        if (index < runs_[r].first || index > runs_[r].last) continue;
        *run = r;
        *offset = static_cast<size_t>(params_[index]->data.device().f32() - runs_[r].p);
        return true;
    }
    return false;
}

void AdamW::export_state(size_t index, float* m_h, float* v_h) {
    if (index >= params_.size()) throw std::runtime_error("AdamW: parameter index out of range");
    const size_t n = params_[index]->data.rows() * params_[index]->data.cols();
    size_t run = 0, off = 0;
    if (locate(index, &run, &off)) {
        check(pk_memcpy_d2h(m_h, runs_[run].m.f32() + off, n * sizeof(float), device::stream()), "pk_memcpy_d2h");
        check(pk_memcpy_d2h(v_h, runs_[run].v.f32() + off, n * sizeof(float), device::stream()), "pk_memcpy_d2h");
        device::synchronize();
        return;
    }
    auto it = pending_.find(index);
    for (size_t k = 0; k < n; ++k) {
        m_h[k] = it == pending_.end() ? 0.0f : it->second.m[k];
        v_h[k] = it == pending_.end() ? 0.0f : it->second.v[k];
    }
}

void AdamW::import_state(size_t index, const float* m_h, const float* v_h) {
    if (index >= params_.size()) throw std::runtime_error("AdamW: parameter index out of range");
    const size_t n = params_[index]->data.rows() * params_[index]->data.cols();
    size_t run = 0, off = 0;
    if (locate(index, &run, &off)) {
        check(pk_memcpy_h2d(runs_[run].m.f32() + off, m_h, n * sizeof(float), device::stream()), "pk_memcpy_h2d");
        check(pk_memcpy_h2d(runs_[run].v.f32() + off, v_h, n * sizeof(float), device::stream()), "pk_memcpy_h2d");
        device::synchronize();
        return;
    }
    Pending& pd = pending_[index];
    pd.m.assign(m_h, m_h + n);
    pd.v.assign(v_h, v_h + n);
}

void AdamW::step() {
    ++t_;
    const float c1 = 1.0f - std::pow(b1_, static_cast<float>(t_));
    const float c2 = 1.0f - std::pow(b2_, static_cast<float>(t_));
    build_runs();
    void* s = device::stream();
    for (auto& r : runs_) {
        check(pk_adamw(s, r.p, r.g, r.m.f32(), r.v.f32(), static_cast<int64_t>(r.n), lr, b1_, b2_, eps_, wd_, c1, c2,
                       r.shadow),
              "pk_adamw");
        for (size_t i = r.first; i <= r.last; ++i) {
            params_[i]->data.mark_device_modified();
            if (r.shadow) params_[i]->shadow_version = params_[i]->data.version();
        }
    }
}
void AdamW::zero_grad() { microtorch::zero_grad(params_); }

}  // namespace nn
}  // namespace microtorch
