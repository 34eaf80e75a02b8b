#pragma once
// Tape ops: forward on the GPU through libpk + a backward closure per op.
//
// The first group keeps the names, argument meaning and error behaviour of the
// reference's op set (include/microtorch/ops.hpp:12-163; formulas in src/ops.cpp),
// restricted to the ops the transformer-block training step uses. The second group
// are the fused forms the models in this library are written against; each one is
// mathematically the composition named in its comment.
#include <vector>

#include "microtorch/autograd.hpp"

namespace microtorch {
namespace ops {

// ---- reference op set (hot-path subset) ---------------------------------------
Var matmul(const Var& a, const Var& b);      // [m,k]x[k,n]; dA = dC B^T, dB = A^T dC
Var add(const Var& a, const Var& b);
Var sub(const Var& a, const Var& b);
Var mul(const Var& a, const Var& b);         // hadamard
Var add_bias(const Var& x, const Var& b);    // b [1,n]; db = column sum
Var gelu(const Var& x);                      // tanh form, exact derivative
Var relu(const Var& x);
Var silu(const Var& x);
Var mean(const Var& x);                      // -> [1,1]
Var scale(const Var& x, float s);
Var transpose(const Var& x);
Var slice_cols(const Var& x, size_t j0, size_t j1);
Var concat_cols(const std::vector<Var>& xs);
Var layernorm(const Var& x, const Var& gamma, const Var& beta, float eps = 1e-5f);
Var rmsnorm(const Var& x, const Var& w);     // eps fixed at 1e-5 like the reference (src/ops.cpp:435)
Var embedding(const Var& table, const std::vector<int>& ids);
Var cross_entropy(const Var& logits, const std::vector<int>& targets);
// mean cross entropy of (h W) or (h W^T) against targets, computed over row chunks so that the
// [rows, vocab] logits never exist as a whole; W is [in, out], or [out, in] when transposed_w.
Var linear_cross_entropy(const Var& h, const Var& W, bool transposed_w, const std::vector<int>& targets,
                         size_t chunk_rows = 16384);
// qk is the fused [T, 3d] q|k|v layout. Like the reference (src/ops.cpp:495-511) this
// rotates the first head_dim columns of q and of k only.
Var apply_rope(const Var& qk, const std::vector<int>& pos, float theta_base, size_t head_dim);
// One head: Y = softmax(scale Q K^T + block-causal mask) V as one tape node.
Var fused_attention(const Var& q, const Var& k, const Var& v, float scale, size_t seq_len, bool causal);
float clip_grad_norm(const std::vector<Var>& params, float max_norm);
Matrix attention_mask(size_t rows, size_t seq_len, bool causal);
Var softmax_row(const Var& x);               // dX = S .* (dY - rowsum(dY .* S))
// Inverted dropout (src/ops.cpp:760-786): keep with probability 1 - p, kept values scaled by
// 1 / (1 - p); the mask is a pure function of (seed, element index), drawn on the host with the
// reference's generator (std::mt19937_64 + uniform_real_distribution<float>, row-major) and
// applied on the device; backward replays it. p == 0 returns x. Not allowed inside checkpoint().
Var dropout(const Var& x, float p, unsigned long long seed);

// ---- declared for source compatibility, not provided -------------------------------
// Research mechanisms of the reference outside the checkpointed transformer-block training
// path. The declarations let code written against the reference's headers (its Python
// bindings, its model zoo header) compile unchanged; calling one throws std::runtime_error.
// (four parameters: the arity the reference's python/bindings.cpp binds)
Var kimi_attention(const Var& q, const Var& k, const Var& v, bool causal);

// ---- fused forms ------------------------------------------------------------------
// y = x W (+ bias) (+ residual): matmul + add_bias + add in one GEMM epilogue.
// W is [in, out] (transposed_w = false) or [out, in] (true: y = x W^T, the tied head).
Var linear(const Var& x, const Var& W, const Var& bias = nullptr, const Var& residual = nullptr,
           bool transposed_w = false);
// All heads at once on the [T, H*dk] layout (q: Hq heads; k, v: Hkv heads, Hq % Hkv == 0).
// Equals the per-head slice_cols + fused_attention + concat_cols loop of the
// reference's blocks (src/llama.cpp:44-52, src/nn.cpp:144-150).
Var attention(const Var& q, const Var& k, const Var& v, size_t n_heads, size_t n_kv_heads, size_t seq_len,
              bool causal);
// attention(slice_cols(qkv, 0, d), slice_cols(qkv, d, 2 d), slice_cols(qkv, 2 d, 3 d), n_heads, n_heads, ...)
// for a packed [T, 3 d] projection, without the slices: the same values, read and written in place.
Var attention_packed(const Var& qkv, size_t n_heads, size_t seq_len, bool causal);
// Rotates the first `n_rot` heads (width head_dim) of x [T, H*head_dim] IN PLACE and
// returns a node that shares x's buffer. x must have no other consumer and must be the
// output of an op whose backward does not read its own output (a linear / matmul).
Var rope_(const Var& x, const std::vector<int>& pos, float theta_base, size_t head_dim, size_t n_rot);
// silu(gate) .* up in one pass (ops::mul(ops::silu(g), u)).
Var swiglu(const Var& gate, const Var& up);
// swiglu(x Wg, x Wu) as ONE node: in bf16 mode both projections and the activation run in one
// GEMM kernel that reads x once (pk_gemm_swiglu); the two products are kept only when a backward
// pass will need them, and their gradients are written over them. Same values, bit for bit, as
// swiglu(linear(x, Wg), linear(x, Wu)); falls back to exactly that where the kernel does not apply.
Var linear_swiglu(const Var& x, const Var& Wg, const Var& Wu);
// rope_(linear(x, W), pos, theta_base, head_dim, n_rot) with the rotation in the GEMM's epilogue
// where the kernel takes the shape (bf16, head_dim 64 or 128); the same bits either way.
Var linear_rope(const Var& x, const Var& W, const std::vector<int>& pos, float theta_base, size_t head_dim, size_t n_rot);

}  // namespace ops
}  // namespace microtorch
