// Tape ops. Every forward and backward runs on the GPU through the libpk C ABI; the
// host only shapes the calls. Formulas and error behaviour follow the reference's
// src/ops.cpp (line references beside each op).
#include "microtorch/ops.hpp"
#include "microtorch/ops_detail.hpp"

#include <cstdlib>
#include <algorithm>
#include <cmath>
#include <cstring>
#include <list>
#include <random>
#include <stdexcept>

#include "pk.h"

namespace microtorch {
namespace ops {

namespace {

using device::check;

void* S() { return device::stream(); }
DType cdt() { return device::compute_dtype(); }
int64_t i64(size_t v) { return static_cast<int64_t>(v); }

Tensor new_act(size_t r, size_t c) { return Tensor::empty(r, c, cdt()); }

// Tape node unless grad is off or no input requires it (reference: src/ops.cpp:17-29).
Var record_value(Value result, std::vector<Var> parents, std::function<void(Variable*)> bw) {
    bool needs = false;
    if (grad_enabled())
        for (const auto& p : parents) needs = needs || (p && p->requires_grad);
    Var out = std::make_shared<Variable>(std::move(result), needs);
    if (needs) {
        parents.erase(std::remove(parents.begin(), parents.end(), nullptr), parents.end());
        out->parents = std::move(parents);
        Variable* self = out.get();
        out->backward_fn = [self, bw]() { bw(self); };
    }
    return out;
}

Var record(Tensor result, std::vector<Var> parents, std::function<void(Variable*)> bw) {
    return record_value(Value(std::move(result)), std::move(parents), std::move(bw));
}

// Upstream gradient of a node in the compute dtype.
Tensor grad_of(Variable* self) { return self->grad.device().cast(cdt()); }

// fp32 view of a small parameter-like tensor (norm gains, biases).
Tensor f32_of(const Var& v) { return v->data.device().cast(DType::F32); }

// Runs fn(dst) where dst is an fp32 [rows, cols] buffer whose contents are ADDED to the
// gradient of `v`: the gradient itself when it is fp32, else a zeroed temporary.
template <typename F>
void into_f32_grad(const Var& v, F fn) {
    if (v->grad_dtype() == DType::F32) {
        Tensor& g = v->grad_for_accumulate();
        fn(g.f32());
    } else {
        Tensor tmp = Tensor::zeros(v->data.rows(), v->data.cols(), DType::F32);
        fn(tmp.f32());
        v->accumulate(tmp);
    }
}

void gemm(const Tensor& A, bool ta, const Tensor& B, bool tb, Tensor& C, bool accumulate,
          const float* bias = nullptr, const Tensor* residual = nullptr) {
    const int64_t M = i64(ta ? A.cols() : A.rows()), K = i64(ta ? A.rows() : A.cols());
    const int64_t N = i64(tb ? B.rows() : B.cols());
    check(pk_gemm(S(), A.dt(), C.dt(), ta, tb, M, N, K, A.ptr(), i64(A.ld()), B.ptr(), i64(B.ld()), C.ptr(),
                  i64(C.ld()), accumulate ? 1 : 0, bias, residual ? residual->ptr() : nullptr,
                  residual ? i64(residual->ld()) : 0),
          "pk_gemm");
}

// target.grad += op(A) . op(B). reuse_data: when this is the first contribution and target's own
// output is dead after the calling closure (autograd::disposable_input), the product is written
// over that output instead of into a fresh buffer; the caller must be done reading it.
void gemm_to_grad(const Var& target, const Tensor& A, bool ta, const Tensor& B, bool tb, bool reuse_data = false) {
    const bool first = target->grad.empty() && !target->grad_home.defined();
    if (!first && (target->grad_home.defined() || target->grad.device().use_count() == 1) &&
        (target->grad_dtype() == DType::F32 || cdt() == DType::BF16)) {
        // accumulate in the GEMM epilogue: grad += op(A).op(B), no temporary
        Tensor& g = target->grad_for_accumulate();
        gemm(A, ta, B, tb, g, true);
        return;
    }
    Tensor c;
    if (reuse_data && first && autograd::disposable_input(target) && target->data.device().dtype() == target->grad_dtype())
        c = target->data.device();
    else
        c = Tensor::empty(target->data.rows(), target->data.cols(), target->grad_dtype());
    gemm(A, ta, B, tb, c, false);
    target->accumulate(c);
}

// ---- small caches for index arrays and rotary tables -------------------------------
uint64_t hash_ints(const std::vector<int>& v) {
    uint64_t h = 1469598103934665603ull;
    for (int x : v) {
        h ^= static_cast<uint32_t>(x);
        h *= 1099511628211ull;
    }
    return h ^ (static_cast<uint64_t>(v.size()) << 1);
}
struct IndexEntry {
    uint64_t key;
    size_t n;
    Tensor dev;
};
// Device copy (int32) of a host index vector; the last few are kept so that the
// positions / ids of a step are uploaded once, not once per block.
Tensor device_ints(const std::vector<int>& v) {
    static std::list<IndexEntry> cache;
    const uint64_t key = hash_ints(v);
    for (auto it = cache.begin(); it != cache.end(); ++it)
        if (it->key == key && it->n == v.size()) {
            cache.splice(cache.begin(), cache, it);
            return cache.front().dev;
        }
    static_assert(sizeof(int) == 4, "int32 index arrays");
    Tensor t = Tensor::bytes(v.size() * 4 + 4, device::Pool::Persistent);
    if (!v.empty()) {
        check(pk_memcpy_h2d(t.ptr(), v.data(), v.size() * 4, S()), "pk_memcpy_h2d");
        check(pk_stream_sync(S()), "pk_stream_sync");
    }
    cache.push_front({key, v.size(), t});
    if (cache.size() > 12) cache.pop_back();
    return t;
}
Tensor upload_ints_once(const std::vector<int32_t>& v) {
    Tensor t = Tensor::bytes(v.size() * 4 + 4);
    if (!v.empty()) {
        check(pk_memcpy_h2d(t.ptr(), v.data(), v.size() * 4, S()), "pk_memcpy_h2d");
        check(pk_stream_sync(S()), "pk_stream_sync");
    }
    return t;
}

struct RopeEntry {
    float theta;
    size_t head_dim, n_pos;
    Tensor table;
};
// cos/sin table [n_pos, head_dim/2, 2] with the reference's float expressions
// (src/ops.cpp:499-503): inv_freq = 1 / pow(theta_base, float(dim) / head_dim),
// angle = float(pos) * inv_freq.
Tensor rope_table(float theta_base, size_t head_dim, size_t n_pos) {
    static std::list<RopeEntry> cache;
    for (auto& e : cache)
        if (e.theta == theta_base && e.head_dim == head_dim && e.n_pos >= n_pos) return e.table;
    const size_t half = head_dim / 2;
    Matrix m(n_pos, half * 2);
    for (size_t p = 0; p < n_pos; ++p) {
        const float pos = static_cast<float>(static_cast<int>(p));
        for (size_t dim = 0; dim < head_dim; dim += 2) {
            const float inv_freq = 1.0f / std::pow(theta_base, static_cast<float>(dim) / head_dim);
            const float theta = pos * inv_freq;
            m(p, dim) = std::cos(theta);
            m(p, dim + 1) = std::sin(theta);
        }
    }
    Tensor t = Tensor::from_host(m, DType::F32, device::Pool::Persistent);
    cache.push_front({theta_base, head_dim, n_pos, t});
    if (cache.size() > 8) cache.pop_back();
    return t;
}
size_t max_pos(const std::vector<int>& pos) {
    int m = 0;
    for (int p : pos) {
        if (p < 0) throw std::runtime_error("rope: negative position");
        m = std::max(m, p);
    }
    return static_cast<size_t>(m) + 1;
}

void rope_apply(Tensor& t, size_t col0, size_t n_heads, size_t head_dim, const std::vector<int>& pos,
                float theta_base, bool inverse) {
    const size_t n_pos = max_pos(pos);
    Tensor table = rope_table(theta_base, head_dim, n_pos);
    Tensor dpos = device_ints(pos);
    check(pk_rope(S(), t.dt(), t.ptr(), i64(t.cols()), i64(col0), static_cast<int>(n_heads),
                  static_cast<int>(head_dim), static_cast<const int32_t*>(dpos.ptr()), table.f32(),
                  i64(table.rows()), i64(t.rows()), inverse ? 1 : 0),
          "pk_rope");
}

template <typename Fwd, typename Bwd>
Var unary_op(const Var& x, Fwd fwd, Bwd bwd, const char* name) {
    const Tensor& xt = x->compute();
    Tensor y = new_act(xt.rows(), xt.cols());
    check(fwd(S(), xt.dt(), xt.ptr(), y.ptr(), i64(xt.numel())), name);
    return record(std::move(y), {x}, [bwd, name](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        const Tensor& xt = x->compute();
        Tensor g = grad_of(self);
        Tensor dx = new_act(xt.rows(), xt.cols());
        check(bwd(S(), xt.dt(), g.ptr(), xt.ptr(), dx.ptr(), i64(xt.numel())), name);
        x->accumulate(dx);
    });
}

void same_shape(const Var& a, const Var& b, const char* what) {
    if (a->data.rows() != b->data.rows() || a->data.cols() != b->data.cols())
        throw std::runtime_error(std::string(what) + ": shape mismatch");
}

Var binary_op(const Var& a, const Var& b, int op, const char* what) {
    same_shape(a, b, what);
    const Tensor& at = a->compute();
    const Tensor& bt = b->compute();
    Tensor y = new_act(at.rows(), at.cols());
    check(pk_binary(S(), at.dt(), op, at.ptr(), bt.ptr(), y.ptr(), i64(at.numel())), "pk_binary");
    return record(std::move(y), {a, b}, [op](Variable* self) {
        const Var& a = self->parents[0];
        const Var& b = self->parents[1];
        Tensor g = grad_of(self);
        if (op == 2) {  // hadamard: da = g .* b, db = g .* a
            if (a->requires_grad) {
                Tensor d = new_act(g.rows(), g.cols());
                check(pk_binary(S(), g.dt(), 2, g.ptr(), b->compute().ptr(), d.ptr(), i64(g.numel())), "pk_binary");
                a->accumulate(d);
            }
            if (b->requires_grad) {
                Tensor d = new_act(g.rows(), g.cols());
                check(pk_binary(S(), g.dt(), 2, g.ptr(), a->compute().ptr(), d.ptr(), i64(g.numel())), "pk_binary");
                b->accumulate(d);
            }
            return;
        }
        if (a->requires_grad) a->accumulate(g);
        if (b->requires_grad) {
            if (op == 0) {
                b->accumulate(g);
            } else {
                Tensor d = new_act(g.rows(), g.cols());
                check(pk_scale(S(), g.dt(), g.ptr(), -1.0f, d.ptr(), i64(g.numel())), "pk_scale");
                b->accumulate(d);
            }
        }
    });
}

struct EmbedIndex {
    std::vector<int32_t> order, seg, uniq;
};
// Positions grouped by id, ascending position inside a group (counting sort).
EmbedIndex build_embed_index(const std::vector<int>& ids, size_t vocab) {
    EmbedIndex ix;
    std::vector<int32_t> count(vocab + 1, 0);
    for (int id : ids) ++count[static_cast<size_t>(id) + 1];
    for (size_t v = 0; v < vocab; ++v) count[v + 1] += count[v];
    ix.order.resize(ids.size());
    std::vector<int32_t> cursor(count.begin(), count.end() - 1);
    for (size_t i = 0; i < ids.size(); ++i) ix.order[cursor[ids[i]]++] = static_cast<int32_t>(i);
    for (size_t v = 0; v < vocab; ++v)
        if (count[v + 1] > count[v]) {
            ix.uniq.push_back(static_cast<int32_t>(v));
            ix.seg.push_back(count[v]);
        }
    ix.seg.push_back(static_cast<int32_t>(ids.size()));
    return ix;
}

Var attention_impl(const Var& q, const Var& k, const Var& v, size_t Hq, size_t Hkv, float scale, size_t seq_len,
                   bool causal, bool scale_given) {
    const size_t T = q->data.rows();
    if (k->data.rows() != T || v->data.rows() != T || Hq == 0 || Hkv == 0 || q->data.cols() % Hq != 0)
        throw std::runtime_error("fused_attention: shape mismatch");
    const size_t dk = q->data.cols() / Hq;
    if (k->data.cols() != Hkv * dk || v->data.cols() != Hkv * dk || Hq % Hkv != 0)
        throw std::runtime_error("fused_attention: shape mismatch");
    const size_t sl = seq_len == 0 ? T : seq_len;
    if (sl == 0 || T % sl != 0) throw std::runtime_error("fused_attention: rows not a multiple of seq_len");
    const size_t B = T / sl;
    if (!scale_given) scale = 1.0f / std::sqrt(static_cast<float>(dk));
    const Tensor& qt = q->compute();
    const Tensor& kt = k->compute();
    const Tensor& vt = v->compute();
    Tensor out = new_act(T, Hq * dk);
    Tensor lse = Tensor::empty(T, Hq, DType::F32);
    check(pk_attn_fwd(S(), qt.dt(), qt.ptr(), i64(qt.cols()), kt.ptr(), i64(kt.cols()), vt.ptr(), i64(vt.cols()),
                      out.ptr(), i64(out.cols()), lse.f32(), i64(B), i64(sl), static_cast<int>(Hq),
                      static_cast<int>(Hkv), static_cast<int>(dk), scale, causal ? 1 : 0),
          "pk_attn_fwd");
    Tensor out_saved = out;
    return record(std::move(out), {q, k, v}, [out_saved, lse, B, sl, Hq, Hkv, dk, scale, causal](Variable* self) {
        const Var& q = self->parents[0];
        const Var& k = self->parents[1];
        const Var& v = self->parents[2];
        if (!q->requires_grad && !k->requires_grad && !v->requires_grad) return;
        const Tensor& qt = q->compute();
        const Tensor& kt = k->compute();
        const Tensor& vt = v->compute();
        Tensor g = grad_of(self);
        Tensor dq = new_act(qt.rows(), qt.cols()), dk_ = new_act(kt.rows(), kt.cols()), dv = new_act(vt.rows(), vt.cols());
        Tensor scratch = Tensor::bytes(pk_attn_bwd_scratch_bytes(i64(B), i64(sl), static_cast<int>(Hq)));
        check(pk_attn_bwd(S(), qt.dt(), qt.ptr(), i64(qt.cols()), kt.ptr(), i64(kt.cols()), vt.ptr(), i64(vt.cols()),
                          out_saved.ptr(), i64(out_saved.cols()), lse.f32(), g.ptr(), i64(g.cols()), dq.ptr(),
                          i64(dq.cols()), dk_.ptr(), i64(dk_.cols()), dv.ptr(), i64(dv.cols()), scratch.ptr(),
                          i64(B), i64(sl), static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<int>(dk), scale,
                          causal ? 1 : 0),
              "pk_attn_bwd");
        if (q->requires_grad) q->accumulate(dq);
        if (k->requires_grad) k->accumulate(dk_);
        if (v->requires_grad) v->accumulate(dv);
    });
}

// Attention over a packed [T, 3 d] projection (q | k | v, heads contiguous inside each, as GPT-2's
// c_attn produces it): the kernels read the three column ranges in place through the row stride
// and write dq | dk | dv into one [T, 3 d] gradient, so nothing is sliced or concatenated.
Var attention_packed_impl(const Var& qkv, size_t H, size_t seq_len, bool causal) {
    const size_t T = qkv->data.rows();
    if (H == 0 || qkv->data.cols() % (3 * H) != 0) throw std::runtime_error("fused_attention: shape mismatch");
    const size_t d = qkv->data.cols() / 3, dk = d / H;
    const size_t sl = seq_len == 0 ? T : seq_len;
    if (sl == 0 || T % sl != 0) throw std::runtime_error("fused_attention: rows not a multiple of seq_len");
    const size_t B = T / sl;
    const float scale = 1.0f / std::sqrt(static_cast<float>(dk));
    const Tensor& pt = qkv->compute();
    const size_t es = dtype_bytes(pt.dtype());
    auto col = [es](const Tensor& t, size_t c) { return static_cast<void*>(static_cast<char*>(t.ptr()) + c * es); };
    Tensor out = new_act(T, d);
    Tensor lse = Tensor::empty(T, H, DType::F32);
    check(pk_attn_fwd(S(), pt.dt(), col(pt, 0), i64(pt.ld()), col(pt, d), i64(pt.ld()), col(pt, 2 * d), i64(pt.ld()), out.ptr(),
                      i64(out.cols()), lse.f32(), i64(B), i64(sl), static_cast<int>(H), static_cast<int>(H),
                      static_cast<int>(dk), scale, causal ? 1 : 0),
          "pk_attn_fwd");
    Tensor out_saved = out;
    return record(std::move(out), {qkv}, [out_saved, lse, B, sl, H, d, dk, scale, causal, es](Variable* self) {
        const Var& qkv = self->parents[0];
        if (!qkv->requires_grad) return;
        const Tensor& pt = qkv->compute();
        auto col = [es](const Tensor& t, size_t c) { return static_cast<void*>(static_cast<char*>(t.ptr()) + c * es); };
        Tensor g = grad_of(self);
        Tensor dp = new_act(pt.rows(), pt.cols());
        Tensor scratch = Tensor::bytes(pk_attn_bwd_scratch_bytes(i64(B), i64(sl), static_cast<int>(H)));
        check(pk_attn_bwd(S(), pt.dt(), col(pt, 0), i64(pt.ld()), col(pt, d), i64(pt.ld()), col(pt, 2 * d), i64(pt.ld()),
                          out_saved.ptr(), i64(out_saved.cols()), lse.f32(), g.ptr(), i64(g.cols()), col(dp, 0), i64(dp.ld()),
                          col(dp, d), i64(dp.ld()), col(dp, 2 * d), i64(dp.ld()), scratch.ptr(), i64(B), i64(sl),
                          static_cast<int>(H), static_cast<int>(H), static_cast<int>(dk), scale, causal ? 1 : 0),
              "pk_attn_bwd");
        qkv->accumulate(dp);
    });
}

}  // namespace

namespace detail {
Var record_node(Tensor result, std::vector<Var> parents, std::function<void(Variable*)> bw) {
    return record(std::move(result), std::move(parents), std::move(bw));
}
Var record_projection(size_t rows, size_t cols, std::function<Tensor()> produce, std::vector<Var> parents,
                      std::function<void(Variable*)> bw) {
    // While a checkpointed segment is re-run for its backward pass, a projection's value is
    // produced when its first consumer asks for it. The segment's last projection has none
    // (its closure reads x, W and the upstream gradient), so its GEMM is not run a second time.
    if (grad_enabled() && recomputing())
        return record_value(Value::deferred(rows, cols, std::move(produce)), std::move(parents), std::move(bw));
    return record(produce(), std::move(parents), std::move(bw));
}
Tensor upstream(Variable* self) { return grad_of(self); }
void gemm_raw(const Tensor& A, bool ta, const Tensor& B, bool tb, Tensor& C, bool accumulate, const float* bias,
              const Tensor* residual) {
    gemm(A, ta, B, tb, C, accumulate, bias, residual);
}
void gemm_into_grad(const Var& target, const Tensor& A, bool ta, const Tensor& B, bool tb) {
    gemm_to_grad(target, A, ta, B, tb);
}
void rope_operands(const std::vector<int>& pos, float theta_base, size_t head_dim, Tensor& table, Tensor& dpos) {
    table = rope_table(theta_base, head_dim, max_pos(pos));
    dpos = device_ints(pos);
}
bool rope_in_gemm() {
    static const bool on = [] {
        const char* e = std::getenv("MICROTORCH_ROPE_IN_GEMM");
        return !(e && e[0] == '0');
    }();
    return on;
}
void rope_inplace(Tensor& t, size_t n_rot, size_t head_dim, const std::vector<int>& pos, float theta_base, bool inverse) {
    rope_apply(t, 0, n_rot, head_dim, pos, theta_base, inverse);
}
void colsum_into_grad(const Var& b, const Tensor& g) {
    Tensor scratch = Tensor::bytes(pk_colsum_scratch_bytes(i64(g.rows()), i64(g.cols())));
    into_f32_grad(b, [&](float* dst) {
        check(pk_colsum(S(), g.dt(), g.ptr(), dst, scratch.ptr(), i64(g.rows()), i64(g.cols())), "pk_colsum");
    });
}
}  // namespace detail

// ---------------------------------------------------------------- matmul family
// reference: src/ops.cpp:33-58
Var matmul(const Var& a, const Var& b) {
    if (a->data.cols() != b->data.rows()) throw std::runtime_error("matmul: inner dimensions disagree");
    const Tensor& at = a->compute();
    const Tensor& bt = b->compute();
    Tensor c = new_act(at.rows(), bt.cols());
    gemm(at, false, bt, false, c, false);
    return record(std::move(c), {a, b}, [](Variable* self) {
        const Var& a = self->parents[0];
        const Var& b = self->parents[1];
        Tensor g = grad_of(self);
        if (a->requires_grad) gemm_to_grad(a, g, false, b->compute(), true);   // dA = dC B^T
        if (b->requires_grad) gemm_to_grad(b, a->compute(), true, g, false);   // dB = A^T dC
    });
}

// Backward of y = x W (+ bias) (+ residual) given the upstream gradient g (reference: src/ops.cpp:50-55, 96-103).
static void linear_backward(Variable* self, const Tensor& g, bool transposed_w, bool has_bias, bool has_res) {
        const Var& x = self->parents[0];
        const Var& W = self->parents[1];
        if (W->requires_grad) {
            if (!transposed_w) gemm_to_grad(W, x->compute(), true, g, false);  // [in,out] = X^T G
            else gemm_to_grad(W, g, true, x->compute(), false);               // [out,in] = G^T X
        }
        // last use of x by this node is behind us: dX may take x's place when x is dead otherwise
        if (x->requires_grad) gemm_to_grad(x, g, false, W->compute(), !transposed_w, /*reuse_data=*/true);
        size_t idx = 2;
        if (has_bias) {
            const Var& b = self->parents[idx++];
            if (b->requires_grad) {
                const Tensor gd = g.dense();
                Tensor scratch = Tensor::bytes(pk_colsum_scratch_bytes(i64(gd.rows()), i64(gd.cols())));
                into_f32_grad(b, [&](float* dst) {
                    check(pk_colsum(S(), gd.dt(), gd.ptr(), dst, scratch.ptr(), i64(gd.rows()), i64(gd.cols())), "pk_colsum");
                });
            }
        }
        if (has_res) {
            const Var& r = self->parents[idx++];
            if (r->requires_grad) r->accumulate(g.dense());
        }
    }

Var linear(const Var& x, const Var& W, const Var& bias, const Var& residual, bool transposed_w) {
    const size_t in = transposed_w ? W->data.cols() : W->data.rows();
    const size_t out = transposed_w ? W->data.rows() : W->data.cols();
    if (x->data.cols() != in) throw std::runtime_error("matmul: inner dimensions disagree");
    if (bias && (bias->data.rows() != 1 || bias->data.cols() != out))
        throw std::runtime_error("add_bias: bias must be [1, cols(x)]");
    if (residual && (residual->data.rows() != x->data.rows() || residual->data.cols() != out))
        throw std::runtime_error("linear: residual shape mismatch");
    auto produce = [x, W, bias, residual, transposed_w, out]() {
        const Tensor& xt = x->compute();
        const Tensor& wt = W->compute();
        // A row stride that is a multiple of 16 bytes keeps ragged widths (a 50257-wide
        // vocabulary) on the tensor-core kernel.
        Tensor y = (cdt() == DType::BF16 && out % 8 != 0) ? Tensor::empty_strided(xt.rows(), out, (out + 7) / 8 * 8, cdt())
                                                          : new_act(xt.rows(), out);
        Tensor bt;
        if (bias) bt = f32_of(bias);
        Tensor rt;
        if (residual) rt = residual->compute();
        gemm(xt, false, wt, transposed_w, y, false, bias ? bt.f32() : nullptr, residual ? &rt : nullptr);
        return y;
    };
    const bool has_bias = bias != nullptr, has_res = residual != nullptr;
    return detail::record_projection(x->data.rows(), out, produce, {x, W, bias, residual}, [transposed_w, has_bias, has_res](Variable* self) {
        linear_backward(self, grad_of(self), transposed_w, has_bias, has_res);
    });
}

// y = rope(x W): the q / k projection with the rotary embedding applied in the GEMM's epilogue
// (pk_gemm_rope), bit-identical to rope_(linear(x, W), ...) and falling back to exactly that when
// the kernel does not take the shape. Backward: the gradient is rotated back in place, then the
// projection's backward runs on it.
Var linear_rope(const Var& x, const Var& W, const std::vector<int>& pos, float theta_base, size_t head_dim, size_t n_rot) {
    const size_t in = W->data.rows(), out = W->data.cols();
    if (x->data.cols() != in) throw std::runtime_error("matmul: inner dimensions disagree");
    if (head_dim % 2 != 0 || n_rot * head_dim > out) throw std::runtime_error("apply_rope: head_dim must be even and <= d");
    if (pos.size() != x->data.rows()) throw std::runtime_error("apply_rope: one position per row");
    if (cdt() != DType::BF16 || (head_dim != 64 && head_dim != 128) || n_rot == 0 || !detail::rope_in_gemm())
        return rope_(linear(x, W), pos, theta_base, head_dim, n_rot);
    auto produce = [x, W, pos, theta_base, head_dim, n_rot, out]() {
        const Tensor& xt = x->compute();
        const Tensor& wt = W->compute();
        Tensor y = new_act(xt.rows(), out);
        Tensor table = rope_table(theta_base, head_dim, max_pos(pos));
        Tensor dpos = device_ints(pos);
        const int rc = pk_gemm_rope(S(), 0, i64(xt.rows()), i64(out), i64(xt.cols()), xt.ptr(), i64(xt.ld()), wt.ptr(), i64(wt.ld()),
                                    y.ptr(), i64(y.ld()), nullptr, static_cast<const int32_t*>(dpos.ptr()), table.f32(),
                                    i64(table.rows()), static_cast<int>(n_rot), static_cast<int>(head_dim), 0);
        if (rc == PK_ERR_UNSUPPORTED) {
            gemm(xt, false, wt, false, y, false);
            rope_apply(y, 0, n_rot, head_dim, pos, theta_base, false);
        } else {
            check(rc, "pk_gemm_rope");
        }
        return y;
    };
    return detail::record_projection(x->data.rows(), out, produce, {x, W}, [pos, theta_base, head_dim, n_rot](Variable* self) {
        Tensor g = grad_of(self);
        self->grad.reset();
        if (g.use_count() > 1) g = g.clone();  // someone else still reads the unrotated gradient
        rope_apply(g, 0, n_rot, head_dim, pos, theta_base, true);
        linear_backward(self, g, false, false, false);
    });
}

// reference: src/ops.cpp:60-83
Var add(const Var& a, const Var& b) { return binary_op(a, b, 0, "add"); }
Var sub(const Var& a, const Var& b) { return binary_op(a, b, 1, "sub"); }
Var mul(const Var& a, const Var& b) { return binary_op(a, b, 2, "mul"); }

// reference: src/ops.cpp:85-104
Var add_bias(const Var& x, const Var& b) {
    if (b->data.rows() != 1 || b->data.cols() != x->data.cols())
        throw std::runtime_error("add_bias: bias must be [1, cols(x)]");
    const Tensor& xt = x->compute();
    Tensor bt = f32_of(b);
    Tensor y = new_act(xt.rows(), xt.cols());
    check(pk_add_bias(S(), xt.dt(), xt.ptr(), bt.f32(), y.ptr(), i64(xt.rows()), i64(xt.cols())), "pk_add_bias");
    return record(std::move(y), {x, b}, [](Variable* self) {
        const Var& x = self->parents[0];
        const Var& b = self->parents[1];
        Tensor g = grad_of(self);
        if (x->requires_grad) x->accumulate(g);
        if (b->requires_grad) {
            Tensor scratch = Tensor::bytes(pk_colsum_scratch_bytes(i64(g.rows()), i64(g.cols())));
            into_f32_grad(b, [&](float* dst) {
                check(pk_colsum(S(), g.dt(), g.ptr(), dst, scratch.ptr(), i64(g.rows()), i64(g.cols())), "pk_colsum");
            });
        }
    });
}

// reference: src/ops.cpp:106-138, 788-801, 404-424
Var gelu(const Var& x) { return unary_op(x, pk_gelu_fwd, pk_gelu_bwd, "pk_gelu"); }
Var relu(const Var& x) { return unary_op(x, pk_relu_fwd, pk_relu_bwd, "pk_relu"); }
Var silu(const Var& x) { return unary_op(x, pk_silu_fwd, pk_silu_bwd, "pk_silu"); }

Var swiglu(const Var& gate, const Var& up) {
    same_shape(gate, up, "swiglu");
    // Produced on first read inside a recomputed segment: when the consumer is a frozen projection
    // at the end of the segment (QLoRA down_proj: its backward reads neither its input nor its
    // value), the recompute needs this product no more than the projection's.
    auto produce = [gate, up]() {
        const Tensor& gt = gate->compute();
        const Tensor& ut = up->compute();
        Tensor y = new_act(gt.rows(), gt.cols());
        check(pk_swiglu_fwd(S(), gt.dt(), gt.ptr(), ut.ptr(), y.ptr(), i64(gt.numel())), "pk_swiglu_fwd");
        return y;
    };
    return detail::record_projection(gate->data.rows(), gate->data.cols(), produce, {gate, up}, [](Variable* self) {
        const Var& gate = self->parents[0];
        const Var& up = self->parents[1];
        const Tensor& gt = gate->compute();
        const Tensor& ut = up->compute();
        Tensor g = grad_of(self);
        // gate and up have no other use once this closure has read them: inside a checkpointed
        // segment their gradients take their place (the kernel reads an element before it writes it)
        const bool in_place = gate.get() != up.get() && autograd::disposable_input(gate) && autograd::disposable_input(up) &&
                              gt.dtype() == gate->grad_dtype();
        Tensor dg = in_place ? gt : new_act(gt.rows(), gt.cols()), du = in_place ? ut : new_act(gt.rows(), gt.cols());
        check(pk_swiglu_bwd(S(), gt.dt(), g.ptr(), gt.ptr(), ut.ptr(), dg.ptr(), du.ptr(), i64(gt.numel())), "pk_swiglu_bwd");
        if (gate->requires_grad) gate->accumulate(dg);
        if (up->requires_grad) up->accumulate(du);
    });
}

Var linear_swiglu(const Var& x, const Var& Wg, const Var& Wu) {
    if (x->data.cols() != Wg->data.rows() || x->data.cols() != Wu->data.rows())
        throw std::runtime_error("matmul: inner dimensions disagree");
    same_shape(Wg, Wu, "swiglu");
    const size_t R = x->data.rows(), F = Wg->data.cols();
    const bool want = grad_enabled() && (x->requires_grad || Wg->requires_grad || Wu->requires_grad);
    if (cdt() != DType::BF16) return swiglu(linear(x, Wg), linear(x, Wu));
    const Tensor& xt = x->compute();
    const Tensor& gw = Wg->compute();
    const Tensor& uw = Wu->compute();
    Tensor y = new_act(R, F), G, U;
    if (want) {
        G = new_act(R, F);
        U = new_act(R, F);
    }
    const int rc = pk_gemm_swiglu(S(), i64(R), i64(F), i64(xt.cols()), xt.ptr(), i64(xt.ld()), gw.ptr(), i64(gw.ld()), uw.ptr(),
                                  i64(uw.ld()), want ? G.ptr() : nullptr, want ? U.ptr() : nullptr, i64(F), y.ptr(), i64(F));
    if (rc == PK_ERR_UNSUPPORTED) return swiglu(linear(x, Wg), linear(x, Wu));
    check(rc, "pk_gemm_swiglu");
    return record(std::move(y), {x, Wg, Wu}, [G, U](Variable* self) {
        const Var& x = self->parents[0];
        const Var& Wg = self->parents[1];
        const Var& Wu = self->parents[2];
        Tensor g = grad_of(self);
        // G and U belong to this node alone: their gradients take their place
        check(pk_swiglu_bwd(S(), G.dt(), g.ptr(), G.ptr(), U.ptr(), G.ptr(), U.ptr(), i64(G.numel())), "pk_swiglu_bwd");
        if (Wg->requires_grad) gemm_to_grad(Wg, x->compute(), true, G, false);   // dWg = x^T dG
        if (Wu->requires_grad) gemm_to_grad(Wu, x->compute(), true, U, false);   // dWu = x^T dU
        if (x->requires_grad) {
            gemm_to_grad(x, G, false, Wg->compute(), true, /*reuse_data=*/false);   // dx  = dG Wg^T
            gemm_to_grad(x, U, false, Wu->compute(), true);                          //     + dU Wu^T
        }
    });
}

Var mean(const Var& x) {
    Tensor xf = x->data.device().cast(DType::F32);
    const size_t n = xf.numel();
    if (n == 0) throw std::runtime_error("mean: empty input");
    Tensor sum = Tensor::bytes(8), scratch = Tensor::bytes(pk_reduce_scratch_bytes());
    check(pk_reduce_sum_f64(S(), xf.f32(), i64(n), 0, 0, static_cast<double*>(sum.ptr()), scratch.ptr()), "pk_reduce_sum_f64");
    Tensor out = Tensor::empty(1, 1, DType::F32);
    check(pk_sum_to_mean(S(), static_cast<const double*>(sum.ptr()), static_cast<double>(n), out.f32()), "pk_sum_to_mean");
    return record(std::move(out), {x}, [n](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        const float g = self->grad.host()(0, 0) / static_cast<float>(n);
        Tensor dx = Tensor::empty(x->data.rows(), x->data.cols(), x->grad_dtype());
        check(pk_fill(S(), dx.dt(), dx.ptr(), g, i64(dx.numel())), "pk_fill");
        x->accumulate(dx);
    });
}

// reference: src/ops.cpp:184-198
Var scale(const Var& x, float s) {
    const Tensor& xt = x->compute();
    Tensor y = new_act(xt.rows(), xt.cols());
    check(pk_scale(S(), xt.dt(), xt.ptr(), s, y.ptr(), i64(xt.numel())), "pk_scale");
    return record(std::move(y), {x}, [s](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        Tensor g = self->grad.device();
        Tensor d = Tensor::empty(g.rows(), g.cols(), g.dtype());
        check(pk_scale(S(), g.dt(), g.ptr(), s, d.ptr(), i64(g.numel())), "pk_scale");
        x->accumulate(d);
    });
}

Var transpose(const Var& x) {
    const Tensor& xt = x->compute();
    Tensor y = new_act(xt.cols(), xt.rows());
    check(pk_transpose(S(), xt.dt(), xt.ptr(), y.ptr(), i64(xt.rows()), i64(xt.cols())), "pk_transpose");
    return record(std::move(y), {x}, [](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        Tensor g = self->grad.device();
        Tensor d = Tensor::empty(g.cols(), g.rows(), g.dtype());
        check(pk_transpose(S(), g.dt(), g.ptr(), d.ptr(), i64(g.rows()), i64(g.cols())), "pk_transpose");
        x->accumulate(d);
    });
}

// reference: src/ops.cpp:200-246
Var slice_cols(const Var& x, size_t j0, size_t j1) {
    if (j1 <= j0 || j1 > x->data.cols()) throw std::runtime_error("slice_cols: bad range");
    const Tensor& xt = x->compute();
    Tensor y = new_act(xt.rows(), j1 - j0);
    check(pk_copy_cols(S(), xt.dt(), xt.ptr(), i64(xt.cols()), i64(j0), y.ptr(), i64(y.cols()), 0, i64(xt.rows()),
                       i64(j1 - j0), 0),
          "pk_copy_cols");
    return record(std::move(y), {x}, [j0](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        Tensor g = self->grad.device();
        Tensor dx = Tensor::zeros(x->data.rows(), x->data.cols(), g.dtype());
        check(pk_copy_cols(S(), g.dt(), g.ptr(), i64(g.cols()), 0, dx.ptr(), i64(dx.cols()), i64(j0), i64(g.rows()),
                           i64(g.cols()), 0),
              "pk_copy_cols");
        x->accumulate(dx);
    });
}

Var concat_cols(const std::vector<Var>& xs) {
    if (xs.empty()) throw std::runtime_error("concat_cols: empty input");
    const size_t rows = xs[0]->data.rows();
    size_t cols = 0;
    for (const auto& x : xs) {
        if (x->data.rows() != rows) throw std::runtime_error("concat_cols: row mismatch");
        cols += x->data.cols();
    }
    Tensor y = new_act(rows, cols);
    size_t off = 0;
    for (const auto& x : xs) {
        const Tensor& xt = x->compute();
        check(pk_copy_cols(S(), xt.dt(), xt.ptr(), i64(xt.cols()), 0, y.ptr(), i64(cols), i64(off), i64(rows),
                           i64(xt.cols()), 0),
              "pk_copy_cols");
        off += xt.cols();
    }
    return record(std::move(y), xs, [](Variable* self) {
        Tensor g = self->grad.device();
        size_t off = 0;
        for (const auto& p : self->parents) {
            const size_t w = p->data.cols();
            if (p->requires_grad) {
                Tensor d = Tensor::empty(g.rows(), w, g.dtype());
                check(pk_copy_cols(S(), g.dt(), g.ptr(), i64(g.cols()), i64(off), d.ptr(), i64(w), 0, i64(g.rows()),
                                   i64(w), 0),
                      "pk_copy_cols");
                p->accumulate(d);
            }
            off += w;
        }
    });
}

// reference: src/ops.cpp:248-327. Saves mean and rstd per row instead of xhat [R,C].
Var layernorm(const Var& x, const Var& gamma, const Var& beta, float eps) {
    const size_t R = x->data.rows(), C = x->data.cols();
    if (gamma->data.rows() != 1 || gamma->data.cols() != C || beta->data.rows() != 1 || beta->data.cols() != C)
        throw std::runtime_error("layernorm: gamma/beta must be [1, cols(x)]");
    const Tensor& xt = x->compute();
    Tensor gt = f32_of(gamma), bt = f32_of(beta);
    Tensor y = new_act(R, C);
    Tensor mean = Tensor::empty(1, R, DType::F32), rstd = Tensor::empty(1, R, DType::F32);
    check(pk_layernorm_fwd(S(), xt.dt(), xt.ptr(), gt.f32(), bt.f32(), y.ptr(), mean.f32(), rstd.f32(), i64(R), i64(C), eps),
          "pk_layernorm_fwd");
    return record(std::move(y), {x, gamma, beta}, [mean, rstd](Variable* self) {
        const Var& x = self->parents[0];
        const Var& g = self->parents[1];
        const Var& b = self->parents[2];
        const Tensor& xt = x->compute();
        const size_t R = xt.rows(), C = xt.cols();
        Tensor dy = grad_of(self);
        Tensor gt = f32_of(g);
        Tensor dx;
        if (x->requires_grad) dx = new_act(R, C);
        const bool want = g->requires_grad || b->requires_grad;
        Tensor scratch;
        if (want) scratch = Tensor::bytes(pk_layernorm_bwd_scratch_bytes(i64(R), i64(C)));
        // dgamma / dbeta are accumulated in place when their gradients are fp32
        Tensor tg, tb;
        float* pg = nullptr;
        float* pb = nullptr;
        if (g->requires_grad) {
            if (g->grad_dtype() == DType::F32) pg = g->grad_for_accumulate().f32();
            else { tg = Tensor::zeros(1, C, DType::F32); pg = tg.f32(); }
        }
        if (b->requires_grad) {
            if (b->grad_dtype() == DType::F32) pb = b->grad_for_accumulate().f32();
            else { tb = Tensor::zeros(1, C, DType::F32); pb = tb.f32(); }
        }
        check(pk_layernorm_bwd(S(), xt.dt(), dy.ptr(), xt.ptr(), gt.f32(), mean.f32(), rstd.f32(),
                               dx.defined() ? dx.ptr() : nullptr, pg, pb, want ? scratch.ptr() : nullptr, i64(R), i64(C)),
              "pk_layernorm_bwd");
        if (tg.defined()) g->accumulate(tg);
        if (tb.defined()) b->accumulate(tb);
        if (x->requires_grad) x->accumulate(dx);
    });
}

// reference: src/ops.cpp:426-479 (eps is the constant 1e-5 there as well)
Var rmsnorm(const Var& x, const Var& w) {
    const size_t R = x->data.rows(), C = x->data.cols();
    if (w->data.rows() != 1 || w->data.cols() != C) throw std::runtime_error("rmsnorm: w must be [1, cols(x)]");
    const Tensor& xt = x->compute();
    Tensor wt = f32_of(w);
    Tensor y = new_act(R, C);
    Tensor rinv = Tensor::empty(1, R, DType::F32);
    check(pk_rmsnorm_fwd(S(), xt.dt(), xt.ptr(), wt.f32(), y.ptr(), rinv.f32(), i64(R), i64(C), 1e-5f), "pk_rmsnorm_fwd");
    return record(std::move(y), {x, w}, [rinv](Variable* self) {
        const Var& x = self->parents[0];
        const Var& w = self->parents[1];
        const Tensor& xt = x->compute();
        const size_t R = xt.rows(), C = xt.cols();
        Tensor dy = grad_of(self);
        Tensor wt = f32_of(w);
        Tensor dx;
        if (x->requires_grad) dx = new_act(R, C);
        Tensor scratch, tw;
        float* pw = nullptr;
        if (w->requires_grad) {
            scratch = Tensor::bytes(pk_rmsnorm_bwd_scratch_bytes(i64(R), i64(C)));
            if (w->grad_dtype() == DType::F32) pw = w->grad_for_accumulate().f32();
            else { tw = Tensor::zeros(1, C, DType::F32); pw = tw.f32(); }
        }
        check(pk_rmsnorm_bwd(S(), xt.dt(), dy.ptr(), xt.ptr(), wt.f32(), rinv.f32(), dx.defined() ? dx.ptr() : nullptr,
                             pw, pw ? scratch.ptr() : nullptr, i64(R), i64(C)),
              "pk_rmsnorm_bwd");
        if (tw.defined()) w->accumulate(tw);
        if (x->requires_grad) x->accumulate(dx);
    });
}

// reference: src/ops.cpp:329-348
Var embedding(const Var& table, const std::vector<int>& ids) {
    const size_t V = table->data.rows(), d = table->data.cols();
    for (int id : ids)
        if (id < 0 || static_cast<size_t>(id) >= V) throw std::runtime_error("embedding: id out of range");
    const Tensor& tt = table->compute();
    Tensor dids = device_ints(ids);
    Tensor out = new_act(ids.size(), d);
    check(pk_embedding_fwd(S(), tt.dt(), tt.ptr(), static_cast<const int32_t*>(dids.ptr()), out.ptr(), i64(ids.size()),
                           i64(d), i64(V), nullptr),
          "pk_embedding_fwd");
    return record(std::move(out), {table}, [ids](Variable* self) {
        const Var& t = self->parents[0];
        if (!t->requires_grad) return;
        const size_t V = t->data.rows(), d = t->data.cols();
        EmbedIndex ix = build_embed_index(ids, V);
        Tensor order = upload_ints_once(ix.order), seg = upload_ints_once(ix.seg), uniq = upload_ints_once(ix.uniq);
        Tensor g = self->grad.device();
        into_f32_grad(t, [&](float* dst) {
            check(pk_embedding_bwd(S(), g.dt(), g.ptr(), static_cast<const int32_t*>(order.ptr()),
                                   static_cast<const int32_t*>(seg.ptr()), static_cast<const int32_t*>(uniq.ptr()),
                                   i64(ix.uniq.size()), dst, i64(d)),
                  "pk_embedding_bwd");
        });
    });
}

// reference: src/ops.cpp:350-376
Var cross_entropy(const Var& logits, const std::vector<int>& targets) {
    const size_t R = logits->data.rows(), C = logits->data.cols();
    if (targets.size() != R) throw std::runtime_error("cross_entropy: one target per row");
    for (int t : targets)
        if (t < 0 || static_cast<size_t>(t) >= C) throw std::runtime_error("cross_entropy: target out of range");
    const Tensor& lt = logits->compute_strided();
    Tensor dt = device_ints(targets);
    const bool want = grad_enabled() && logits->requires_grad;
    // The kernel writes (softmax - onehot)/R over its input, so a training step works on a copy.
    Tensor work = want ? lt.clone() : lt;
    Tensor rows = Tensor::empty(1, R, DType::F32);
    check(pk_cross_entropy(S(), work.dt(), work.ptr(), i64(work.ld()), static_cast<const int32_t*>(dt.ptr()), rows.f32(), i64(R),
                           i64(C), 1.0f / static_cast<float>(R), want ? 1 : 0, nullptr),
          "pk_cross_entropy");
    Tensor sum = Tensor::bytes(8), scratch = Tensor::bytes(pk_reduce_scratch_bytes());
    check(pk_reduce_sum_f64(S(), rows.f32(), i64(R), 0, 0, static_cast<double*>(sum.ptr()), scratch.ptr()), "pk_reduce_sum_f64");
    Tensor out = Tensor::empty(1, 1, DType::F32);
    check(pk_sum_to_mean(S(), static_cast<const double*>(sum.ptr()), static_cast<double>(R), out.f32()), "pk_sum_to_mean");
    return record(std::move(out), {logits}, [work](Variable* self) {
        const Var& l = self->parents[0];
        if (!l->requires_grad) return;
        const float g = self->grad.host()(0, 0);  // the seed is host-known: no readback in the common case
        Tensor dl = work;
        if (g != 1.0f)  // padding columns of a strided buffer hold zeros and stay zero
            check(pk_scale(S(), dl.dt(), dl.ptr(), g, dl.ptr(), i64(dl.rows() * dl.ld())), "pk_scale");
        l->accumulate(dl);
    });
}

// cross_entropy(linear(h, W), targets) without ever holding the [rows, vocab] logits: the rows
// are processed in chunks; each chunk's logits are produced, turned into (softmax - onehot)/R
// in place, and immediately contracted into dh and dW. Same arithmetic per row as the two
// separate ops (reference: src/ops.cpp:33-58 and 350-376); only the order in which rows are
// visited differs, and dW sums chunk contributions in ascending chunk order.
Var linear_cross_entropy(const Var& h, const Var& W, bool transposed_w, const std::vector<int>& targets,
                         size_t chunk_rows) {
    const size_t R = h->data.rows(), d = h->data.cols();
    const size_t in = transposed_w ? W->data.cols() : W->data.rows();
    const size_t V = transposed_w ? W->data.rows() : W->data.cols();
    if (d != in) throw std::runtime_error("matmul: inner dimensions disagree");
    if (targets.size() != R) throw std::runtime_error("cross_entropy: one target per row");
    for (int t : targets)
        if (t < 0 || static_cast<size_t>(t) >= V) throw std::runtime_error("cross_entropy: target out of range");
    if (chunk_rows == 0) chunk_rows = 16384;
    const Tensor& ht = h->compute();
    const Tensor& wt = W->compute();
    Tensor dtg = device_ints(targets);
    const bool want_h = grad_enabled() && h->requires_grad, want_w = grad_enabled() && W->requires_grad;
    const bool want = want_h || want_w;
    Tensor rows = Tensor::empty(1, R, DType::F32);
    Tensor dh, dw;
    if (want_h) dh = new_act(R, d);
    if (want_w) dw = Tensor::zeros(W->data.rows(), W->data.cols(), DType::F32);
    const size_t ldl = cdt() == DType::BF16 ? (V + 7) / 8 * 8 : V;
    for (size_t r0 = 0; r0 < R; r0 += chunk_rows) {
        const size_t rc = std::min(chunk_rows, R - r0);
        Tensor hc = ht.view(r0 * d, rc, d);
        Tensor logits = Tensor::empty_strided(rc, V, ldl, cdt());
        gemm(hc, false, wt, transposed_w, logits, false);
        check(pk_cross_entropy(S(), logits.dt(), logits.ptr(), i64(ldl), static_cast<const int32_t*>(dtg.ptr()) + r0,
                               rows.f32() + r0, i64(rc), i64(V), 1.0f / static_cast<float>(R), want ? 1 : 0, nullptr),
              "pk_cross_entropy");
        if (want_h) {  // dh = dlogits W^T   ([in,out] storage)  or  dlogits W   ([out,in] storage)
            Tensor dhc = dh.view(r0 * d, rc, d);
            gemm(logits, false, wt, !transposed_w, dhc, false);
        }
        if (want_w) {
            if (!transposed_w) gemm(hc, true, logits, false, dw, true);   // [in,out] += h^T dlogits
            else gemm(logits, true, hc, false, dw, true);                  // [out,in] += dlogits^T h
        }
    }
    Tensor sum = Tensor::bytes(8), scratch = Tensor::bytes(pk_reduce_scratch_bytes());
    check(pk_reduce_sum_f64(S(), rows.f32(), i64(R), 0, 0, static_cast<double*>(sum.ptr()), scratch.ptr()), "pk_reduce_sum_f64");
    Tensor out = Tensor::empty(1, 1, DType::F32);
    check(pk_sum_to_mean(S(), static_cast<const double*>(sum.ptr()), static_cast<double>(R), out.f32()), "pk_sum_to_mean");
    return record(std::move(out), {h, W}, [dh, dw](Variable* self) {
        const Var& h = self->parents[0];
        const Var& W = self->parents[1];
        const float g = self->grad.host()(0, 0);
        if (h->requires_grad && dh.defined()) {
            Tensor t = dh;
            if (g != 1.0f) check(pk_scale(S(), t.dt(), t.ptr(), g, t.ptr(), i64(t.numel())), "pk_scale");
            h->accumulate(t);
        }
        if (W->requires_grad && dw.defined()) {
            if (W->grad_dtype() == DType::F32) {
                Tensor& gw = W->grad_for_accumulate();
                check(pk_axpy(S(), gw.dt(), gw.ptr(), dw.dt(), dw.ptr(), g, i64(dw.numel())), "pk_axpy");
            } else {
                Tensor t = dw;
                if (g != 1.0f) check(pk_scale(S(), t.dt(), t.ptr(), g, t.ptr(), i64(t.numel())), "pk_scale");
                W->accumulate(t);
            }
        }
    });
}

// reference: src/ops.cpp:481-537 (first head of q and of k only)
Var apply_rope(const Var& qk, const std::vector<int>& pos, float theta_base, size_t head_dim) {
    const size_t T = qk->data.rows(), d3 = qk->data.cols();
    if (d3 % 3 != 0) throw std::runtime_error("apply_rope: cols must be divisible by 3");
    const size_t d = d3 / 3;
    if (head_dim % 2 != 0 || head_dim > d) throw std::runtime_error("apply_rope: head_dim must be even and <= d");
    if (pos.size() != T) throw std::runtime_error("apply_rope: one position per row");
    Tensor out = qk->compute().clone();
    rope_apply(out, 0, 1, head_dim, pos, theta_base, false);
    rope_apply(out, d, 1, head_dim, pos, theta_base, false);
    return record(std::move(out), {qk}, [pos, theta_base, head_dim, d](Variable* self) {
        const Var& qk = self->parents[0];
        if (!qk->requires_grad) return;
        Tensor g = self->grad.device().clone();
        rope_apply(g, 0, 1, head_dim, pos, theta_base, true);
        rope_apply(g, d, 1, head_dim, pos, theta_base, true);
        qk->accumulate(g);
    });
}

Var rope_(const Var& x, const std::vector<int>& pos, float theta_base, size_t head_dim, size_t n_rot) {
    if (head_dim % 2 != 0 || n_rot * head_dim > x->data.cols())
        throw std::runtime_error("apply_rope: head_dim must be even and <= d");
    if (pos.size() != x->data.rows()) throw std::runtime_error("apply_rope: one position per row");
    Tensor t = x->compute();
    rope_apply(t, 0, n_rot, head_dim, pos, theta_base, false);
    x->data.mark_device_modified();
    return record(std::move(t), {x}, [pos, theta_base, head_dim, n_rot](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        Tensor g = self->grad.device();
        self->grad.reset();
        if (g.use_count() > 1) g = g.clone();  // someone else still reads the unrotated gradient
        rope_apply(g, 0, n_rot, head_dim, pos, theta_base, true);
        x->accumulate(g);
    });
}

// reference: src/ops.cpp:863-934
Var fused_attention(const Var& q, const Var& k, const Var& v, float scale, size_t seq_len, bool causal) {
    if (q->data.cols() != k->data.cols()) throw std::runtime_error("fused_attention: shape mismatch");
    return attention_impl(q, k, v, 1, 1, scale, seq_len, causal, true);
}

Var attention_packed(const Var& qkv, size_t n_heads, size_t seq_len, bool causal) {
    return attention_packed_impl(qkv, n_heads, seq_len, causal);
}

Var attention(const Var& q, const Var& k, const Var& v, size_t n_heads, size_t n_kv_heads, size_t seq_len,
              bool causal) {
    return attention_impl(q, k, v, n_heads, n_kv_heads, 0.0f, seq_len, causal, false);
}

// reference: src/ops.cpp:1046-1064 (sum of squares in double)
float clip_grad_norm(const std::vector<Var>& params, float max_norm) {
    Tensor sum = Tensor::bytes(8), scratch = Tensor::bytes(pk_reduce_scratch_bytes());
    check(pk_memset(sum.ptr(), 0, 8, S()), "pk_memset");
    std::vector<Tensor> grads;
    for (const auto& p : params) {
        if (p->grad.empty()) continue;
        Tensor g = p->grad.device().cast(DType::F32);
        check(pk_reduce_sum_f64(S(), g.f32(), i64(g.numel()), 1, 1, static_cast<double*>(sum.ptr()), scratch.ptr()),
              "pk_reduce_sum_f64");
    }
    double sq = 0.0;
    check(pk_memcpy_d2h(&sq, sum.ptr(), 8, S()), "pk_memcpy_d2h");
    check(pk_stream_sync(S()), "pk_stream_sync");
    const float total = static_cast<float>(std::sqrt(sq));
    if (total > max_norm && total > 0.0f) {
        const float s = max_norm / total;
        for (const auto& p : params) {
            if (p->grad.empty()) continue;
            const Tensor& g = p->grad.device();
            check(pk_scale(S(), g.dt(), g.ptr(), s, g.ptr(), i64(g.numel())), "pk_scale");
            p->grad.mark_device_modified();
        }
    }
    return total;
}

// reference: src/ops.cpp:140-167
Var softmax_row(const Var& x) {
    const Tensor& xt = x->compute();
    Tensor y = new_act(xt.rows(), xt.cols());
    check(pk_softmax_fwd(S(), xt.dt(), xt.ptr(), y.ptr(), i64(xt.rows()), i64(xt.cols())), "pk_softmax_fwd");
    Tensor saved = y;
    return record(std::move(y), {x}, [saved](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        Tensor g = grad_of(self);
        Tensor dx = new_act(g.rows(), g.cols());
        check(pk_softmax_bwd(S(), g.dt(), saved.ptr(), g.ptr(), dx.ptr(), i64(g.rows()), i64(g.cols())), "pk_softmax_bwd");
        x->accumulate(dx);
    });
}

namespace {
// The reference's mask: one uniform draw per element in row-major order from mt19937_64(seed);
// an element is kept (and scaled by 1 / keep) when the draw is below keep (src/ops.cpp:766-773).
Tensor dropout_mask(size_t rows, size_t cols, float p, unsigned long long seed) {
    const float keep = 1.0f - p, inv_keep = 1.0f / keep;
    std::mt19937_64 rng(seed);
    std::uniform_real_distribution<float> u(0.0f, 1.0f);
    Matrix m(rows, cols);
    float* d = m.data();
    for (size_t i = 0; i < rows * cols; ++i) d[i] = (u(rng) < keep) ? inv_keep : 0.0f;
    return Tensor::from_host(m, cdt());
}
}  // namespace

// reference: src/ops.cpp:760-786
Var dropout(const Var& x, float p, unsigned long long seed) {
    if (p < 0.0f || p >= 1.0f) throw std::runtime_error("dropout: p must be in [0, 1)");
    if (p == 0.0f) return x;
    const Tensor& xt = x->compute();
    Tensor mask = dropout_mask(xt.rows(), xt.cols(), p, seed);
    Tensor y = new_act(xt.rows(), xt.cols());
    check(pk_binary(S(), xt.dt(), 2, xt.ptr(), mask.ptr(), y.ptr(), i64(xt.numel())), "pk_binary");
    return record(std::move(y), {x}, [p, seed](Variable* self) {
        const Var& x = self->parents[0];
        if (!x->requires_grad) return;
        Tensor g = grad_of(self);
        Tensor mask = dropout_mask(g.rows(), g.cols(), p, seed);  // replayed, not stored
        Tensor dx = new_act(g.rows(), g.cols());
        check(pk_binary(S(), g.dt(), 2, g.ptr(), mask.ptr(), dx.ptr(), i64(g.numel())), "pk_binary");
        x->accumulate(dx);
    });
}

Matrix attention_mask(size_t rows, size_t seq_len, bool causal) {
    const size_t sl = seq_len == 0 ? rows : seq_len;
    Matrix m(rows, rows, -1e9f);
    for (size_t i = 0; i < rows; ++i) {
        const size_t b0 = (i / sl) * sl;
        const size_t hi = causal ? i + 1 : std::min(rows, b0 + sl);
        for (size_t j = b0; j < hi; ++j) m(i, j) = 0.0f;
    }
    return m;
}

}  // namespace ops
}  // namespace microtorch
