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

Q8Weight Q8Weight::from_matrix(const Matrix& W) {
    if (W.cols() % 32 != 0) throw std::runtime_error("quantize_int8: cols must be a multiple of the block (32)");
    Q8Weight w;
    w.rows = W.rows();
    w.cols = W.cols();
    Tensor src = Tensor::from_host(W, DType::F32);
    w.q = Tensor::bytes(w.rows * w.cols, device::Pool::Persistent);
    w.scales = Tensor::bytes(w.rows * (w.cols / 32) * 2, device::Pool::Persistent);
    check(pk_q8_quantize(device::stream(), src.f32(), static_cast<int8_t*>(w.q.ptr()),
                         static_cast<uint16_t*>(w.scales.ptr()), static_cast<int64_t>(w.rows),
                         static_cast<int64_t>(w.cols)),
          "pk_q8_quantize");
    return w;
}

Tensor Q8Weight::dequantize(DType dt) const {
    Tensor out = Tensor::empty(rows, cols, dt);
    check(pk_q8_dequantize(device::stream(), static_cast<const int8_t*>(q.ptr()),
                           static_cast<const uint16_t*>(scales.ptr()), static_cast<int>(dt), out.ptr(),
                           static_cast<int64_t>(rows), static_cast<int64_t>(cols)),
          "pk_q8_dequantize");
    return out;
}

static QuantizedTensor to_host(const Q8Weight& w) {
    QuantizedTensor t;
    t.rows = w.rows;
    t.cols = w.cols;
    t.block = 32;
    t.q.resize(w.rows * w.cols);
    std::vector<uint16_t> sc(w.rows * (w.cols / 32));
    void* s = device::stream();
    check(pk_memcpy_d2h(t.q.data(), w.q.ptr(), t.q.size(), s), "pk_memcpy_d2h");
    check(pk_memcpy_d2h(sc.data(), w.scales.ptr(), sc.size() * 2, s), "pk_memcpy_d2h");
    check(pk_stream_sync(s), "pk_stream_sync");
    t.scales.resize(sc.size());
    for (size_t i = 0; i < sc.size(); ++i) t.scales[i] = half_to_float(sc[i]);
    return t;
}

QuantizedTensor quantize_int8(const Matrix& m, size_t block) {
    if (block == 0) throw std::runtime_error("quantize_int8: block must be > 0");
    if (block != 32) throw std::runtime_error("quantize_int8: only the Q8_0 block size 32 is provided");
    return to_host(Q8Weight::from_matrix(m));
}

Matrix dequantize(const QuantizedTensor& t) {
    if (t.block != 32) throw std::runtime_error("dequantize: only the Q8_0 block size 32 is provided");
    // float(q) * float(scale): one exact int->float conversion and one fp32 multiply.
    Matrix m(t.rows, t.cols);
    const size_t bpr = t.cols / 32;
    for (size_t i = 0; i < t.rows; ++i)
        for (size_t j = 0; j < t.cols; ++j)
            m(i, j) = static_cast<float>(t.q[i * t.cols + j]) * t.scales[i * bpr + j / 32];
    return m;
}

namespace ops {

Var q8_linear(const Var& x, const std::shared_ptr<Q8Weight>& Wq, const Var& bias, const Var& residual) {
    if (x->data.cols() != Wq->rows) throw std::runtime_error("matmul: inner dimensions disagree");
    const size_t out = Wq->cols;
    if (bias && (bias->data.rows() != 1 || bias->data.cols() != out))
        throw std::runtime_error("add_bias: bias must be [1, cols(x)]");
    const DType cd = device::compute_dtype();
    const Tensor& xt = x->compute();
    Tensor y = Tensor::empty(xt.rows(), out, cd);
    Tensor bt, rt;
    if (bias) bt = bias->data.device().cast(DType::F32);
    if (residual) rt = residual->compute();
    {
        Tensor w = Wq->dequantize(cd);  // expanded for this GEMM only
        detail::gemm_raw(xt, false, w, false, y, false, bias ? bt.f32() : nullptr, residual ? &rt : nullptr);
    }
    const bool has_bias = bias != nullptr, has_res = residual != nullptr;
    return detail::record_node(std::move(y), {x, bias, residual}, [Wq, has_bias, has_res](Variable* self) {
        const Var& x = self->parents[0];
        Tensor g = detail::upstream(self);
        if (x->requires_grad) {
            Tensor w = Wq->dequantize(device::compute_dtype());
            detail::gemm_into_grad(x, g, false, w, true);  // dX = dY deq(W)^T
        }
        size_t idx = 1;
        if (has_bias) {
            const Var& b = self->parents[idx++];
            if (b->requires_grad) detail::colsum_into_grad(b, g);
        }
        if (has_res) {
            const Var& r = self->parents[idx++];
            if (r->requires_grad) r->accumulate(g);
        }
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
// sum taken in the second GEMM's epilogue.
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
    if (block != 32) throw std::runtime_error("QLinear: only the Q8_0 block size 32 is provided");
    Wq_ = std::make_shared<Q8Weight>(Q8Weight::from_matrix(W));
    if (b.rows() != 0) b_ = make_var(std::move(b), false);
}
QLinear::QLinear(const Matrix& W, size_t block) : QLinear(W, Matrix(), block) {}
Var QLinear::forward(const Var& x) const { return ops::q8_linear(x, Wq_, b_); }
Var QLinear::forward_residual(const Var& x, const Var& residual) const { return ops::q8_linear(x, Wq_, b_, residual); }
QuantizedTensor QLinear::weight_q() const { return to_host(*Wq_); }

QLoRALinear::QLoRALinear(const Matrix& W, Matrix b, size_t rank, float alpha, size_t block, unsigned seed)
    : r_(rank), scaling_(alpha / static_cast<float>(rank)) {
    if (rank == 0) throw std::runtime_error("QLoRALinear: rank must be > 0");
    if (block != 32) throw std::runtime_error("QLoRALinear: only the Q8_0 block size 32 is provided");
    Wq_ = std::make_shared<Q8Weight>(Q8Weight::from_matrix(W));
    if (b.rows() != 0) b_ = make_var(std::move(b), false);
    A = reg("lora_A", lora_a_init(W.rows(), r_, seed));
    B = reg("lora_B", Matrix(r_, W.cols()));
}

Var QLoRALinear::forward(const Var& x) const {
    return lora_delta_onto(ops::q8_linear(x, Wq_, b_), x, A, B, scaling_);
}

}  // namespace nn
}  // namespace microtorch
