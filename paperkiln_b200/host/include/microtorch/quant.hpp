#pragma once
// Q8_0 block quantization of frozen base weights and LoRA / QLoRA linear layers.
//
// Surface of the reference's include/microtorch/quant.hpp:31-100 (QuantizedTensor,
// quantize_int8, dequantize, LoRALinear, QLinear, QLoRALinear). Differences, all on the
// storage side:
//   * the quantized weight lives on the GPU as int8 values plus one scale per block along a
//     row of W[in, out]. Block 32 with a column count that is a multiple of 32 is stored as
//     Q8_0: the scale is rounded to IEEE binary16 (the reference keeps fp32 scales). Every
//     other block length -- the reference's default of 64, a ragged last block -- keeps the
//     reference's fp32 scale, bit for bit;
//   * no dequantized fp32 copy of the weight is cached (the reference keeps Wdq_). In bf16
//     mode a Q8_0 weight is expanded inside the GEMM kernel, tile by tile in shared memory
//     (pk_gemm_q8_lora), with the LoRA product added in the same accumulator; other modes
//     expand the weight for the duration of one GEMM;
//   * dequantisation is exactly float(q) * float(scale), so it is bit-identical to the
//     reference's dequantize() applied to the same q and scales.
#include <cstdint>
#include <vector>

#include "microtorch/nn.hpp"

namespace microtorch {

struct QuantizedTensor {
    std::vector<int8_t> q;      // rows*cols values, row-major (host copy)
    std::vector<float> scales;  // one per block (rounded to binary16 when the weight is Q8_0)
    size_t rows = 0, cols = 0;
    size_t block = 64;  // block length along a row (reference default)
    // binary16 scales for Q8_0 (block 32, cols % 32 == 0), fp32 scales otherwise
    size_t nbytes() const { return q.size() + scales.size() * ((block == 32 && cols % 32 == 0) ? 2 : sizeof(float)); }
};

// Device-resident block-quantized weight.
struct Q8Weight {
    Tensor q;       // int8 [rows, cols] (byte buffer)
    Tensor scales;  // Q8_0: binary16 [rows, cols/32]; otherwise fp32 [rows, ceil(cols/block)] (byte buffer)
    size_t rows = 0, cols = 0;
    size_t block = 32;
    bool is_q8_0() const { return block == 32 && cols % 32 == 0; }
    size_t blocks_per_row() const { return (cols + block - 1) / block; }
    static Q8Weight from_matrix(const Matrix& W, size_t block = 32);
    Tensor dequantize(DType dt) const;  // transient expansion
    size_t nbytes() const { return rows * cols + rows * blocks_per_row() * (is_q8_0() ? 2 : 4); }
};

QuantizedTensor quantize_int8(const Matrix& m, size_t block = 64);
Matrix dequantize(const QuantizedTensor& t);

namespace ops {
// Rotary embedding to apply to the first n_rot heads of a quantised projection's output, as one
// tape node with the projection (what rope_(y, pos, theta_base, head_dim, n_rot) would do; a second
// pass over y: the Q8_0 kernel's epilogue has no registers to spare for it).
struct Rotary {
    std::vector<int> pos;
    float theta_base;
    size_t head_dim;
    size_t n_rot;
};
// y = x deq(Wq) (+ bias) (+ residual); no gradient flows to the quantized weight.
Var q8_linear(const Var& x, const std::shared_ptr<Q8Weight>& Wq, const Var& bias = nullptr,
              const Var& residual = nullptr, const Rotary* rot = nullptr);
// y = x deq(Wq) + scaling (x A) B (+ bias) (+ residual): the QLoRA projection as one tape node.
// Gradients reach x, A and B (and bias / residual). In bf16 mode with a Q8_0 weight the base
// product and the rank-r product share one accumulator in one kernel, forward and backward.
Var q8_lora_linear(const Var& x, const std::shared_ptr<Q8Weight>& Wq, const Var& A, const Var& B, float scaling,
                   const Var& bias = nullptr, const Var& residual = nullptr, const Rotary* rot = nullptr);
}  // namespace ops

namespace nn {

class LoRALinear : public Module {
public:
    LoRALinear(Matrix W, Matrix b, size_t rank, float alpha, unsigned seed = 0);
    LoRALinear(Matrix W, size_t rank, float alpha, unsigned seed = 0);
    Var forward(const Var& x) const;
    Matrix merged_weight() const;
    size_t rank() const { return r_; }
    Var A, B;

protected:
    Var W_, b_;  // frozen (requires_grad = false)
    size_t r_;
    float scaling_;
};

class QLinear : public Module {
public:
    QLinear(const Matrix& W, Matrix b, size_t block = 64);
    explicit QLinear(const Matrix& W, size_t block = 64);
    Var forward(const Var& x) const;
    Var forward_residual(const Var& x, const Var& residual) const;
    QuantizedTensor weight_q() const;
    size_t nbytes() const { return Wq_->nbytes(); }

private:
    std::shared_ptr<Q8Weight> Wq_;
    Var b_;
};

class QLoRALinear : public Module {
public:
    QLoRALinear(const Matrix& W, Matrix b, size_t rank, float alpha, size_t block = 64, unsigned seed = 0);
    Var forward(const Var& x) const;
    size_t base_nbytes() const { return Wq_->nbytes(); }
    Var A, B;

private:
    std::shared_ptr<Q8Weight> Wq_;
    Var b_;
    size_t r_;
    float scaling_;
};

}  // namespace nn
}  // namespace microtorch
