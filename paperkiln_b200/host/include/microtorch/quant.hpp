#pragma once
// Q8_0 block quantization of frozen base weights and LoRA / QLoRA linear layers.
//
// Surface of the reference's include/microtorch/quant.hpp:31-100 (QuantizedTensor,
// quantize_int8, dequantize, LoRALinear, QLinear, QLoRALinear). Differences, all on the
// storage side:
//   * the quantized weight lives on the GPU as int8 values plus one IEEE binary16 scale
//     per block of 32 along a row of W[in, out] (the reference stores fp32 scales and
//     defaults to block 64); only block 32 is provided;
//   * no dequantized fp32 copy of the weight is cached (the reference keeps Wdq_):
//     forward and backward expand the blocks on the fly for the GEMM and drop them;
//   * dequantisation is exactly float(q) * float(scale), so it is bit-identical to the
//     reference's dequantize() applied to the same q and (fp16-rounded) scales.
#include <cstdint>
#include <vector>

#include "microtorch/nn.hpp"

namespace microtorch {

struct QuantizedTensor {
    std::vector<int8_t> q;      // rows*cols values, row-major (host copy)
    std::vector<float> scales;  // one per block, already rounded to binary16
    size_t rows = 0, cols = 0;
    size_t block = 32;
    size_t nbytes() const { return q.size() + scales.size() * 2; }
};

// Device-resident Q8_0 weight.
struct Q8Weight {
    Tensor q;       // int8 [rows, cols] (byte buffer)
    Tensor scales;  // binary16 [rows, cols/32] (byte buffer)
    size_t rows = 0, cols = 0;
    static Q8Weight from_matrix(const Matrix& W);
    Tensor dequantize(DType dt) const;  // transient expansion
    size_t nbytes() const { return rows * cols + rows * (cols / 32) * 2; }
};

// Block must be 32 (Q8_0); cols must be a multiple of 32.
QuantizedTensor quantize_int8(const Matrix& m, size_t block = 32);
Matrix dequantize(const QuantizedTensor& t);

namespace ops {
// y = x deq(Wq) (+ bias) (+ residual); no gradient flows to the quantized weight.
Var q8_linear(const Var& x, const std::shared_ptr<Q8Weight>& Wq, const Var& bias = nullptr,
              const Var& residual = nullptr);
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
    QLinear(const Matrix& W, Matrix b, size_t block = 32);
    explicit QLinear(const Matrix& W, size_t block = 32);
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
    QLoRALinear(const Matrix& W, Matrix b, size_t rank, float alpha, size_t block = 32, unsigned seed = 0);
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
