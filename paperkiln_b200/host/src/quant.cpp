// Q8_0 weights and LoRA / QLoRA layers. Behavioural reference: src/quant.cpp of
// paperkiln (quantize_int8 11-37, dequantize 39-48, LoRALinear 63-89, QLinear 91-100,
// QLoRALinear 102-119).
#include "microtorch/quant.hpp"

#include <cstring>
#include <random>
#include <stdexcept>

#include "microtorch/ops_detail.hpp"
#include "pk.h"

namespace microtorch {

using device::check;

namespace {
float half_to_float(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal
            exp = 127 - 15 + 1;
            while (!(man & 0x400u)) {
                man <<= 1;
                --exp;
            }
            man &= 0x3ffu;
            bits = sign | (exp << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
}  // namespace

Q8Weight Q8Weight::from_matrix(const Matrix& W, size_t block) {
    if (block == 0) throw std::runtime_error("quantize_int8: block must be > 0");
    Q8Weight w;
    w.rows = W.rows();
    w.cols = W.cols();
    w.block = block;
    Tensor src = Tensor::from_host(W, DType::F32);
    w.q = Tensor::bytes(w.rows * w.cols, device::Pool::Persistent);
    if (w.is_q8_0()) {
        w.scales = Tensor::bytes(w.rows * (w.cols / 32) * 2, device::Pool::Persistent);
        check(pk_q8_quantize(device::stream(), src.f32(), static_cast<int8_t*>(w.q.ptr()),
                             static_cast<uint16_t*>(w.scales.ptr()), static_cast<int64_t>(w.rows),
                             static_cast<int64_t>(w.cols)),
              "pk_q8_quantize");
    } else {
        w.scales = Tensor::bytes(w.rows * w.blocks_per_row() * 4, device::Pool::Persistent);
        check(pk_q8_quantize_block(device::stream(), src.f32(), static_cast<int8_t*>(w.q.ptr()),
                                   static_cast<float*>(w.scales.ptr()), static_cast<int64_t>(w.rows),
                                   static_cast<int64_t>(w.cols), static_cast<int64_t>(block)),
              "pk_q8_quantize_block");
    }
    return w;
}

Tensor Q8Weight::dequantize(DType dt) const {
    Tensor out = Tensor::empty(rows, cols, dt);
    if (is_q8_0())
        check(pk_q8_dequantize(device::stream(), static_cast<const int8_t*>(q.ptr()),
                               static_cast<const uint16_t*>(scales.ptr()), static_cast<int>(dt), out.ptr(),
                               static_cast<int64_t>(rows), static_cast<int64_t>(cols)),
              "pk_q8_dequantize");
    else
        check(pk_q8_dequantize_block(device::stream(), static_cast<const int8_t*>(q.ptr()),
                                     static_cast<const float*>(scales.ptr()), static_cast<int64_t>(block),
                                     static_cast<int>(dt), out.ptr(), static_cast<int64_t>(rows),
                                     static_cast<int64_t>(cols)),
              "pk_q8_dequantize_block");
    return out;
}

static QuantizedTensor to_host(const Q8Weight& w) {
    QuantizedTensor t;
    t.rows = w.rows;
    t.cols = w.cols;
    t.block = w.block;
    t.q.resize(w.rows * w.cols);
    const size_t ns = w.rows * w.blocks_per_row();
    t.scales.resize(ns);
    void* s = device::stream();
    check(pk_memcpy_d2h(t.q.data(), w.q.ptr(), t.q.size(), s), "pk_memcpy_d2h");
    if (w.is_q8_0()) {
        std::vector<uint16_t> sc(ns);
        check(pk_memcpy_d2h(sc.data(), w.scales.ptr(), ns * 2, s), "pk_memcpy_d2h");
        check(pk_stream_sync(s), "pk_stream_sync");
        for (size_t i = 0; i < ns; ++i) t.scales[i] = half_to_float(sc[i]);
    } else {
        check(pk_memcpy_d2h(t.scales.data(), w.scales.ptr(), ns * 4, s), "pk_memcpy_d2h");
        check(pk_stream_sync(s), "pk_stream_sync");
    }
    return t;
}

// reference: src/quant.cpp:11-37
QuantizedTensor quantize_int8(const Matrix& m, size_t block) {
    if (block == 0) throw std::runtime_error("quantize_int8: block must be > 0");
    return to_host(Q8Weight::from_matrix(m, block));
}

// reference: src/quant.cpp:39-48
Matrix dequantize(const QuantizedTensor& t) {
    if (t.block == 0) throw std::runtime_error("dequantize: block must be > 0");
    // float(q) * float(scale): one exact int->float conversion and one fp32 multiply.
    Matrix m(t.rows, t.cols);
    const size_t bpr = (t.cols + t.block - 1) / t.block;
    for (size_t i = 0; i < t.rows; ++i)
        for (size_t j = 0; j < t.cols; ++j)
            m(i, j) = static_cast<float>(t.q[i * t.cols + j]) * t.scales[i * bpr + j / t.block];
    return m;
}

namespace ops {

namespace {
int64_t i64(size_t v) { return static_cast<int64_t>(v); }

// C (+)= A deq(W)^(T) + XA L^(T) through the fused kernel. Returns false when the kernel does not
// take the request (fp32 mode, a weight that is not Q8_0, an unaligned shape): the caller
// expands the weight and uses the dense GEMM instead.
bool q8_gemm_fused(const Tensor& A, const Q8Weight& W, bool trans_w, const Tensor* XA, const Tensor* L, Tensor& C,
                   bool accumulate, const float* bias, const Tensor* residual) {
    if (device::compute_dtype() != DType::BF16 || !W.is_q8_0() || A.dtype() != DType::BF16) return false;
    if (XA && (XA->dtype() != DType::BF16 || L->dtype() != DType::BF16)) return false;
    if (residual && residual->dtype() != C.dtype()) return false;
    const int64_t M = i64(A.rows()), K = i64(A.cols());
    const int64_t N = i64(trans_w ? W.rows : W.cols);
    const int r = XA ? static_cast<int>(XA->cols()) : 0;
    const int rc = pk_gemm_q8_lora(device::stream(), C.dt(), trans_w ? 1 : 0, M, N, K, A.ptr(), i64(A.ld()),
                                   static_cast<const int8_t*>(W.q.ptr()), static_cast<const uint16_t*>(W.scales.ptr()),
                                   XA ? XA->ptr() : nullptr, XA ? i64(XA->ld()) : 0, L ? L->ptr() : nullptr,
                                   L ? i64(L->ld()) : 0, r, C.ptr(), i64(C.ld()), accumulate ? 1 : 0, bias,
                                   residual ? residual->ptr() : nullptr, residual ? i64(residual->ld()) : 0);
    if (rc == PK_ERR_UNSUPPORTED) return false;
    check(rc, "pk_gemm_q8_lora");
    return true;
}

// target.grad += g deq(W)^T (+ DXA A^T): in the kernel's epilogue when the gradient buffer
// exists and has the compute dtype, else through a temporary.
void q8_dx_into_grad(const Var& x, const Tensor& g, const Q8Weight& W, const Tensor* DXA, const Tensor* Alora) {
    const DType cd = device::compute_dtype();
    const bool first = x->grad.empty() && !x->grad_home.defined();
    if (!first && (x->grad_home.defined() || x->grad.device().use_count() == 1) && x->grad_dtype() == cd) {
        Tensor& dst = x->grad_for_accumulate();
        if (q8_gemm_fused(g, W, true, DXA, Alora, dst, true, nullptr, nullptr)) return;
    }
    Tensor dx = Tensor::empty(x->data.rows(), x->data.cols(), cd);
    if (!q8_gemm_fused(g, W, true, DXA, Alora, dx, false, nullptr, nullptr)) {
        Tensor w = W.dequantize(cd);
        detail::gemm_raw(g, false, w, true, dx, false);                       // dX = dY deq(W)^T
        if (DXA) detail::gemm_raw(*DXA, false, *Alora, true, dx, true);       //      + DXA A^T
    }
    x->accumulate(dx);
}

void bias_residual_grads(Variable* self, size_t first_idx, bool has_bias, bool has_res, const Tensor& g) {
    size_t idx = first_idx;
    if (has_bias) {
        const Var& b = self->parents[idx++];
        if (b->requires_grad) detail::colsum_into_grad(b, g);
    }
    if (has_res) {
        const Var& r = self->parents[idx++];
        if (r->requires_grad) r->accumulate(g);
    }
}

void check_linear_shapes(const Var& x, const Q8Weight& W, const Var& bias, const Var& residual) {
    if (x->data.cols() != W.rows) throw std::runtime_error("matmul: inner dimensions disagree");
    if (bias && (bias->data.rows() != 1 || bias->data.cols() != W.cols))
        throw std::runtime_error("add_bias: bias must be [1, cols(x)]");
    if (residual && (residual->data.rows() != x->data.rows() || residual->data.cols() != W.cols))
        throw std::runtime_error("linear: residual shape mismatch");
}
void check_rotary(const Rotary* rot, const Var& x, const Q8Weight& W, const Var& residual) {
    if (!rot) return;
    if (residual) throw std::runtime_error("apply_rope: a rotated projection takes no residual");
    if (rot->head_dim % 2 != 0 || rot->n_rot * rot->head_dim > W.cols)
        throw std::runtime_error("apply_rope: head_dim must be even and <= d");
    if (rot->pos.size() != x->data.rows()) throw std::runtime_error("apply_rope: one position per row");
}

// Upstream gradient of a (possibly rotated) projection: rotated back in place first.
Tensor upstream_unrotated(Variable* self, const std::shared_ptr<Rotary>& rot) {
    Tensor g = detail::upstream(self);
    if (rot) {
        self->grad.reset();
        if (g.use_count() > 1) g = g.clone();  // someone else still reads the rotated gradient
        detail::rope_inplace(g, rot->n_rot, rot->head_dim, rot->pos, rot->theta_base, true);
    }
    return g;
}
}  // namespace

Var q8_linear(const Var& x, const std::shared_ptr<Q8Weight>& Wq, const Var& bias, const Var& residual, const Rotary* rot_in) {
    check_linear_shapes(x, *Wq, bias, residual);
    check_rotary(rot_in, x, *Wq, residual);
    const std::shared_ptr<Rotary> rot = rot_in ? std::make_shared<Rotary>(*rot_in) : nullptr;
    auto produce = [x, Wq, bias, residual, rot]() {
        const DType cd = device::compute_dtype();
        const Tensor& xt = x->compute();
        Tensor y = Tensor::empty(xt.rows(), Wq->cols, cd);
        Tensor bt, rt;
        if (bias) bt = bias->data.device().cast(DType::F32);
        if (residual) rt = residual->compute();
        if (!q8_gemm_fused(xt, *Wq, false, nullptr, nullptr, y, false, bias ? bt.f32() : nullptr, residual ? &rt : nullptr)) {
            Tensor w = Wq->dequantize(cd);  // expanded for this GEMM only
            detail::gemm_raw(xt, false, w, false, y, false, bias ? bt.f32() : nullptr, residual ? &rt : nullptr);
        }
        if (rot) detail::rope_inplace(y, rot->n_rot, rot->head_dim, rot->pos, rot->theta_base, false);
        return y;
    };
    const bool has_bias = bias != nullptr, has_res = residual != nullptr;
    return detail::record_projection(x->data.rows(), Wq->cols, produce, {x, bias, residual}, [Wq, has_bias, has_res, rot](Variable* self) {
        const Var& x = self->parents[0];
        Tensor g = upstream_unrotated(self, rot);
        if (x->requires_grad) q8_dx_into_grad(x, g, *Wq, nullptr, nullptr);
        bias_residual_grads(self, 1, has_bias, has_res, g);
    });
}

Var q8_lora_linear(const Var& x, const std::shared_ptr<Q8Weight>& Wq, const Var& A, const Var& B, float scaling,
                   const Var& bias, const Var& residual, const Rotary* rot_in) {
    check_linear_shapes(x, *Wq, bias, residual);
    check_rotary(rot_in, x, *Wq, residual);
    const std::shared_ptr<Rotary> rot = rot_in ? std::make_shared<Rotary>(*rot_in) : nullptr;
    const size_t r = A->data.cols();
    if (A->data.rows() != Wq->rows || B->data.rows() != r || B->data.cols() != Wq->cols)
        throw std::runtime_error("matmul: inner dimensions disagree");
    const DType cd = device::compute_dtype();
    const Tensor& xt = x->compute();
    const Tensor& at = A->compute();
    // the rank-r intermediate, scaled: XA = scaling (x A)
    Tensor xa = Tensor::empty(xt.rows(), r, cd);
    detail::gemm_raw(xt, false, at, false, xa, false);
    check(pk_scale(device::stream(), xa.dt(), xa.ptr(), scaling, xa.ptr(), i64(xa.numel())), "pk_scale");
    auto produce = [x, Wq, B, xa, bias, residual, rot]() {
        const DType cd = device::compute_dtype();
        const Tensor& xt = x->compute();
        const Tensor& bt_l = B->compute();
        Tensor y = Tensor::empty(xt.rows(), Wq->cols, cd);
        Tensor bt, rt;
        if (bias) bt = bias->data.device().cast(DType::F32);
        if (residual) rt = residual->compute();
        if (!q8_gemm_fused(xt, *Wq, false, &xa, &bt_l, y, false, bias ? bt.f32() : nullptr, residual ? &rt : nullptr)) {
            Tensor w = Wq->dequantize(cd);
            detail::gemm_raw(xt, false, w, false, y, false, bias ? bt.f32() : nullptr, residual ? &rt : nullptr);
            detail::gemm_raw(xa, false, bt_l, false, y, true);
        }
        if (rot) detail::rope_inplace(y, rot->n_rot, rot->head_dim, rot->pos, rot->theta_base, false);
        return y;
    };
    const bool has_bias = bias != nullptr, has_res = residual != nullptr;
    return detail::record_projection(x->data.rows(), Wq->cols, produce, {x, A, B, bias, residual}, [Wq, xa, scaling, has_bias, has_res, rot](Variable* self) {
        const Var& x = self->parents[0];
        const Var& A = self->parents[1];
        const Var& B = self->parents[2];
        const DType cd = device::compute_dtype();
        Tensor g = upstream_unrotated(self, rot);
        const bool need_dxa = x->requires_grad || A->requires_grad;
        Tensor dxa;  // scaling (dY B^T): the gradient that reaches x A
        if (need_dxa) {
            dxa = Tensor::empty(g.rows(), xa.cols(), cd);
            detail::gemm_raw(g, false, B->compute(), true, dxa, false);
            check(pk_scale(device::stream(), dxa.dt(), dxa.ptr(), scaling, dxa.ptr(), i64(dxa.numel())), "pk_scale");
        }
        if (B->requires_grad) detail::gemm_into_grad(B, xa, true, g, false);               // dB = XA^T dY
        if (A->requires_grad) detail::gemm_into_grad(A, x->compute(), true, dxa, false);   // dA = x^T DXA
        if (x->requires_grad) {
            const Tensor& at = A->compute();
            q8_dx_into_grad(x, g, *Wq, &dxa, &at);                                         // dx = dY deq(W)^T + DXA A^T
        }
        bias_residual_grads(self, 3, has_bias, has_res, g);
    });
}

}  // namespace ops

namespace nn {

namespace {
// LoRA A init N(0, 1/r), B = 0 (reference: src/quant.cpp:53-62, 66-67).
Matrix lora_a_init(size_t in, size_t r, unsigned seed) {
    Matrix a(in, r);
    std::mt19937 rng(seed + 7331);
    std::normal_distribution<float> dist(0.0f, 1.0f / static_cast<float>(r));
    float* p = a.data();
    for (size_t i = 0; i < in * r; ++i) p[i] = dist(rng);
    return a;
}

// base + (alpha/r) (x A) B with the scale folded into the rank-r intermediate and the
// sum taken in the second GEMM's epilogue (dense frozen base).
Var lora_delta_onto(const Var& base, const Var& x, const Var& A, const Var& B, float scaling) {
    Var xa = ops::scale(ops::matmul(x, A), scaling);
    return ops::linear(xa, B, nullptr, base);
}
}  // namespace

LoRALinear::LoRALinear(Matrix W, Matrix b, size_t rank, float alpha, unsigned seed)
    : r_(rank), scaling_(alpha / static_cast<float>(rank)) {
    if (rank == 0) throw std::runtime_error("LoRALinear: rank must be > 0");
    const size_t in = W.rows(), out = W.cols();
    W_ = make_var(std::move(W), false);
    if (b.rows() != 0) b_ = make_var(std::move(b), false);
    A = reg("lora_A", lora_a_init(in, r_, seed));
    B = reg("lora_B", Matrix(r_, out));
}
LoRALinear::LoRALinear(Matrix W, size_t rank, float alpha, unsigned seed)
    : LoRALinear(std::move(W), Matrix(), rank, alpha, seed) {}

Var LoRALinear::forward(const Var& x) const {
    return lora_delta_onto(ops::linear(x, W_, b_), x, A, B, scaling_);
}

Matrix LoRALinear::merged_weight() const {
    // W + scaling * A B, computed on the GPU in fp32
    Tensor a = A->data.device().cast(DType::F32), b = B->data.device().cast(DType::F32);
    Tensor ab = Tensor::empty(a.rows(), b.cols(), DType::F32);
    ops::detail::gemm_raw(a, false, b, false, ab, false);
    Tensor merged = W_->data.device().cast(DType::F32).clone();
    check(pk_axpy(device::stream(), PK_F32, merged.ptr(), PK_F32, ab.ptr(), scaling_, static_cast<int64_t>(ab.numel())), "pk_axpy");
    return merged.to_host();
}

QLinear::QLinear(const Matrix& W, Matrix b, size_t block) {
    Wq_ = std::make_shared<Q8Weight>(Q8Weight::from_matrix(W, block));
    if (b.rows() != 0) b_ = make_var(std::move(b), false);
}
QLinear::QLinear(const Matrix& W, size_t block) : QLinear(W, Matrix(), block) {}
Var QLinear::forward(const Var& x) const { return ops::q8_linear(x, Wq_, b_); }
Var QLinear::forward_residual(const Var& x, const Var& residual) const { return ops::q8_linear(x, Wq_, b_, residual); }
QuantizedTensor QLinear::weight_q() const { return to_host(*Wq_); }

QLoRALinear::QLoRALinear(const Matrix& W, Matrix b, size_t rank, float alpha, size_t block, unsigned seed)
    : r_(rank), scaling_(alpha / static_cast<float>(rank)) {
    if (rank == 0) throw std::runtime_error("QLoRALinear: rank must be > 0");
    Wq_ = std::make_shared<Q8Weight>(Q8Weight::from_matrix(W, block));
    if (b.rows() != 0) b_ = make_var(std::move(b), false);
    A = reg("lora_A", lora_a_init(W.rows(), r_, seed));
    B = reg("lora_B", Matrix(r_, W.cols()));
}

Var QLoRALinear::forward(const Var& x) const { return ops::q8_lora_linear(x, Wq_, A, B, scaling_, b_); }

}  // namespace nn
}  // namespace microtorch
