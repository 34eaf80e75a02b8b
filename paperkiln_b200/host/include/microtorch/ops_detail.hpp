#pragma once
// Building blocks shared by the translation units that define tape ops (ops.cpp,
// quant.cpp). Not part of the public surface.
#include <functional>
#include <vector>

#include "microtorch/autograd.hpp"

namespace microtorch {
namespace ops {
namespace detail {

// Tape node around `result` unless grad is off or no parent requires it. Null parents
// are dropped. `bw` reads self->grad and accumulates into self->parents.
Var record_node(Tensor result, std::vector<Var> parents, std::function<void(Variable*)> bw);
// Tape node of a projection whose [rows, cols] value `produce` computes. Outside a recomputed
// segment produce() runs at once; inside one it runs when the first consumer reads the value
// (Value::deferred), i.e. never for the segment's last projection. `produce` must not depend on
// buffers that an in-place op rewrites between this call and the first read.
Var record_projection(size_t rows, size_t cols, std::function<Tensor()> produce, std::vector<Var> parents,
                      std::function<void(Variable*)> bw);
// Upstream gradient of a node as a tensor in the compute dtype.
Tensor upstream(Variable* self);
// C (+)= op(A).op(B) (+ bias) (+ residual) through pk_gemm.
void gemm_raw(const Tensor& A, bool ta, const Tensor& B, bool tb, Tensor& C, bool accumulate,
              const float* bias = nullptr, const Tensor* residual = nullptr);
// target.grad += op(A).op(B), in the GEMM epilogue when the gradient buffer exists.
void gemm_into_grad(const Var& target, const Tensor& A, bool ta, const Tensor& B, bool tb);
// grad(b) += column sums of g
void colsum_into_grad(const Var& b, const Tensor& g);
// Rotary embedding: the (cos, sin) table [positions, head_dim] for theta_base and the positions on
// the device; rotation of the first n_rot heads of t in place (inverse: by the negative angle).
void rope_operands(const std::vector<int>& pos, float theta_base, size_t head_dim, Tensor& table, Tensor& dpos);
// False when MICROTORCH_ROPE_IN_GEMM=0: the projections then rotate in a second pass (for
// measuring what the fusion is worth; the results are the same bits).
bool rope_in_gemm();
void rope_inplace(Tensor& t, size_t n_rot, size_t head_dim, const std::vector<int>& pos, float theta_base, bool inverse);

}  // namespace detail
}  // namespace ops
}  // namespace microtorch
