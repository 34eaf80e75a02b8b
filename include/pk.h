/*
 * pk.h -- C ABI of libpk, the sm_100a kernel library behind the microtorch
 * tape (activation-checkpointed transformer-block training step).
 *
 * Conventions
 *   - every entry returns an int status (PK_OK == 0); none throws, exits,
 *     traps the device or allocates device memory unless its name says so
 *     (pk_malloc / pk_free / pk_host_alloc).
 *   - every pointer is a DEVICE pointer unless the parameter name ends in _h.
 *   - `stream` is a cudaStream_t passed as void*; work is asynchronous on it.
 *   - matrices are row-major; `ld*` are row strides in ELEMENTS.
 *   - `dtype` is PK_F32 or PK_BF16 and names the storage type of activations;
 *     all arithmetic is fp32 (fp64 where the reference sums in double).
 *   - scratch buffers are caller-provided; the matching *_scratch_bytes()
 *     call gives the size. Results never depend on scratch contents on entry.
 *   - all kernels are deterministic: the same call on the same inputs gives
 *     the same bits, which is what makes a recomputed activation identical to
 *     the one the forward pass produced.
 *
 * Each group cites the interface of the reference (paperkiln / microtorch,
 * paths relative to its repository root) that the entries stand in for.
 */
#ifndef PK_H_
#define PK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PK_ABI_VERSION 1

enum pk_dtype { PK_F32 = 0, PK_BF16 = 1 };

enum pk_status {
    PK_OK = 0,
    PK_ERR_INVALID = 1,     /* bad argument (shape, alignment, null pointer) */
    PK_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed; see pk_last_error */
    PK_ERR_UNSUPPORTED = 3, /* valid request this build has no kernel for */
    PK_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up */
    PK_ERR_INDEX = 5,       /* an id / target was out of range (device status word) */
    PK_ERR_COMM = 6         /* a collective failed or its communicator was aborted */
};

/* ---- library / runtime ----------------------------------------------------
 * Stands in for the process-global device switch and CUDA error convention of
 * include/microtorch/device.hpp:20-33 and src/cuda_ops.cu:34-38 (exceptions
 * there, status codes here). */
int pk_abi_version(void);
const char* pk_last_error(void);           /* message of the last failing call on this thread */
int pk_device_count(int* count_h);
int pk_set_device(int device);
int pk_device_name(int device, char* name_h, size_t cap);
int pk_mem_info(size_t* free_h, size_t* total_h);
int pk_malloc(void** ptr_h, size_t bytes);
int pk_free(void* ptr);
int pk_host_alloc(void** ptr_h, size_t bytes); /* pinned host memory */
int pk_host_free(void* ptr_h);
int pk_memcpy_h2d(void* dst, const void* src_h, size_t bytes, void* stream);
int pk_memcpy_d2h(void* dst_h, const void* src, size_t bytes, void* stream);
int pk_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int pk_memset(void* dst, int value, size_t bytes, void* stream);
int pk_stream_create(void** stream_h);
int pk_stream_destroy(void* stream);
int pk_stream_sync(void* stream);
int pk_device_sync(void);
/* Device status word: kernels that detect an out-of-range id or a wait that
 * ran out OR a code into *status (int32 on the device) instead of trapping. */

/* ---- per-kernel-class timing -------------------------------------------------
 * With profiling enabled every launch of a timed class is bracketed by CUDA events on
 * its own stream. pk_prof_summary(kind) synchronises the device and returns the summed
 * duration (ms), the summed algorithmic work (FLOPs) and the launch count since the last
 * pk_prof_reset. kind: 0 tcgen05 GEMM, 1 SIMT GEMM, 2 attention forward, 3 attention
 * backward. (The reference prints per-call timings under MATMUL_PROFILE,
 * third_party/transformer_cpp/src/cuda/matrix_ops.cu:173-181.) */
int pk_prof_enable(int on);
int pk_prof_reset(void);
int pk_prof_summary(int kind, double* ms_h, double* work_h, int64_t* launches_h);

/* ---- GEMM ------------------------------------------------------------------
 * C[M,N] (+)= op(A) . op(B) (+ bias) (+ residual), fp32 accumulation.
 * Replaces device::gemm(A, devA, tA, B, devB, tB) -- include/microtorch/
 * device_cache.hpp:63-71, call sites src/ops.cpp:45,50-55 -- and the kernels
 * gemm_tiled / gemm_tiled_ops in src/cuda_resident.cu:53-76,141-171.
 *   ab_dtype : storage type of A and B (PK_F32 or PK_BF16)
 *   c_dtype  : storage type of C and of `residual`
 *   trans_a  : 0 -> A is [M,K] (lda >= K); 1 -> A is stored [K,M] (lda >= M)
 *   trans_b  : 0 -> B is [K,N] (ldb >= N); 1 -> B is stored [N,K] (ldb >= K)
 *   accumulate: 0 -> C = ..., 1 -> C += ... (C read-modify-write, fixed order)
 *   bias     : fp32 [N] or NULL; residual: [M,N] with row stride ldr or NULL
 * bf16 inputs take the tcgen05 tensor-core kernel when M,N,K and the leading
 * dimensions meet its alignment (multiples of 8 elements, 16-byte aligned
 * bases); other shapes take a SIMT kernel. pk_gemm_last_path() tells which
 * one the last call on this thread used (0 SIMT fp32, 1 SIMT bf16, 2 tcgen05, 3 tcgen05 on
 * CTA pairs, 4 the Q8_0 kernel of pk_gemm_q8_lora). */
int pk_gemm(void* stream, int ab_dtype, int c_dtype, int trans_a, int trans_b,
            int64_t M, int64_t N, int64_t K,
            const void* A, int64_t lda, const void* B, int64_t ldb,
            void* C, int64_t ldc, int accumulate,
            const float* bias, const void* residual, int64_t ldr);
/* y = silu(A Wg) .* (A Wu): the gate and up projections of a SwiGLU feed-forward layer and the
 * activation in ONE pass over A (bf16; A [M, K], Wg and Wu [K, N] row-major, y [M, N]). A CTA pair
 * computes 128 columns of G = A Wg and the same 128 columns of U = A Wu side by side in tensor
 * memory and the epilogue forms y; G and U (both or neither; row stride ldgu) are also stored
 * when the caller needs them for the backward pass. G, U and y have exactly the bits of
 * pk_gemm + pk_gemm + pk_swiglu_fwd: a forward pass that keeps nothing (a checkpointed segment
 * under NoGrad) and a recomputation that keeps G and U produce the same y. Replaces
 * ops::mul(ops::silu(gate), up) over two ops::matmul (src/llama.cpp:55-58; src/ops.cpp:404-424,
 * 76-83). Needs M >= 256, N a multiple of 8 and >= 128, 16-byte aligned bases, leading dimensions
 * multiples of 8; otherwise PK_ERR_UNSUPPORTED (use the three separate calls). */
int pk_gemm_swiglu(void* stream, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* Wg, int64_t ldg,
                   const void* Wu, int64_t ldu, void* G, void* U, int64_t ldgu, void* Y, int64_t ldy);
int pk_gemm_last_path(void);
/* Launch counts per kernel path since the last reset, for a host that wants to know which
 * kernels a whole step ran on (the last-path calls only see one launch). counts_h[0..n):
 * 0 GEMM SIMT fp32, 1 GEMM SIMT bf16, 2 GEMM tcgen05 (one CTA per tile), 3 GEMM tcgen05 on CTA
 * pairs, 4 Q8_0 dequantise-GEMM, 5 attention forward SIMT, 6 attention forward tcgen05,
 * 7 attention backward SIMT, 8 attention backward tcgen05. reset != 0 zeroes them afterwards.
 * Host-side counters; not synchronised between threads. */
int pk_launch_counts(int64_t* counts_h, int n, int reset);
/* Status word of the tensor-core kernel: non-zero (PK_ERR_TIMEOUT) when one of its
 * bounded mbarrier waits gave up. Synchronises the device; clear != 0 resets it. */
int pk_gemm_tc_status(int* status_h, int clear);
/* Force the SIMT kernels (1) or restore automatic selection (0); used by the
 * parity tests to compare the tensor-core kernel with the SIMT one. */
int pk_gemm_force_simt(int on);
/* 1: shapes with enough 256 x 256 output tiles run on CTA pairs (tcgen05 cta_group::2: two SMs
 * per tile, each loading half of B; default); 0: always one CTA per 128 x 256 tile. pk_gemm_last_path
 * reports 3 for the pair kernel. Results are identical bit for bit. */
int pk_gemm_pair_mode(int on);
/* Split-K for products with few output tiles and a long k extent (the weight gradients of
 * narrow projections: dW[d, dkv] = X^T dY over all rows): the k range is cut into up to 8 parts
 * that run side by side, each writing an fp32 partial tile into the caller's workspace, and a
 * second kernel adds the partials in ascending order (so the result is reproducible) together
 * with bias / residual / accumulate. Off until a workspace is given (ptr 16-byte aligned, device
 * memory; null switches it off); 128 MiB covers every shape of the configurations in this repo.
 * The workspace is shared by all calls: they must be issued on one stream. No counterpart in the
 * reference, whose device::gemm is a single SIMT kernel (src/cuda_resident.cu:226-263).
 * pk_gemm_last_splits: parts used by the last tensor-core launch of this thread (1 = not split). */
int pk_gemm_set_workspace(void* ptr, size_t bytes);
int pk_gemm_last_splits(void);

/* ---- normalisation ----------------------------------------------------------
 * RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w; rinv[R] is saved for backward.
 * Replaces ops::rmsnorm (src/ops.cpp:426-479), devops::rmsnorm_fwd/bwd
 * (include/microtorch/device_cache.hpp:122-126) and k_rmsnorm_* in
 * src/cuda_ops.cu:321-381. w and dw are fp32 [C]. dw is ACCUMULATED (+=).
 * dx and dw may each be NULL to skip. */
int pk_rmsnorm_fwd(void* stream, int dtype, const void* x, const float* w, void* y,
                   float* rinv, int64_t R, int64_t C, float eps);
size_t pk_rmsnorm_bwd_scratch_bytes(int64_t R, int64_t C);
int pk_rmsnorm_bwd(void* stream, int dtype, const void* dy, const void* x, const float* w,
                   const float* rinv, void* dx, float* dw, void* scratch,
                   int64_t R, int64_t C);
/* pk_rmsnorm_bwd for hosts that cannot allocate device memory. (No counterpart in the
 * reference: this entry exists only in this library.)
 * Who needs it: a host that gave the whole GPU to its own memory pool before this library was
 * loaded has no memory left to allocate the dw scratch from, and a latency-critical loop
 * cannot afford cudaMalloc, which synchronises the device. This variant takes no scratch
 * argument and calls no allocator (CUDA's or anyone else's): the per-block partial sums of dw
 * go to a fixed buffer inside the library image (~9.3 MiB of device memory held by every GPU
 * that loads libpk, until the process exits).
 * Limits and rules:
 *   - C is limited by that buffer: pk_rmsnorm_bwd_scratch_bytes(R, C) must not exceed
 *     592*4096*4 bytes (C <= 4096 on a 148-SM GPU); larger C returns PK_ERR_UNSUPPORTED with
 *     a message, and pk_rmsnorm_bwd with caller scratch remains available.
 *   - The first call on a device resolves the buffer's device address (a CUDA runtime query,
 *     made with that device current): make that first call before starting any stream capture.
 *   - All calls share the one buffer and it keeps whatever the last call wrote. Nothing has
 *     to be cleared between calls (each call overwrites what it reads), but two calls that
 *     overlap on the GPU (different streams) race on it: serialise them.
 * Results are identical to pk_rmsnorm_bwd, bit for bit. */
int pk_rmsnorm_bwd_noalloc(void* stream, int dtype, const void* dy, const void* x, const float* w,
                           const float* rinv, void* dx, float* dw, int64_t R, int64_t C);
/* LayerNorm (biased variance). Saves mean[R] and rstd[R] instead of the
 * reference's xhat [R,C]. Replaces ops::layernorm (src/ops.cpp:248-327),
 * devops::layernorm_fwd/bwd and k_layernorm_* / k_colsum_dgb in
 * src/cuda_ops.cu:221-318. dgamma/dbeta are ACCUMULATED. */
int pk_layernorm_fwd(void* stream, int dtype, const void* x, const float* gamma,
                     const float* beta, void* y, float* mean, float* rstd,
                     int64_t R, int64_t C, float eps);
size_t pk_layernorm_bwd_scratch_bytes(int64_t R, int64_t C);
int pk_layernorm_bwd(void* stream, int dtype, const void* dy, const void* x,
                     const float* gamma, const float* mean, const float* rstd,
                     void* dx, float* dgamma, float* dbeta, void* scratch,
                     int64_t R, int64_t C);

/* ---- rotary embedding -------------------------------------------------------
 * In-place interleaved-pair rotation (x[2j], x[2j+1]) of `n_heads` heads of
 * width head_dim starting at column col0 of a [R, ld] buffer. The angle table
 * cos_sin is fp32 [n_pos, head_dim/2, 2] built on the host with the reference's
 * float expressions; pos is int32 [R]. inverse != 0 rotates by -theta (the
 * backward). Replaces ops::apply_rope (src/ops.cpp:481-537), which rotates
 * ONE head of q and one of k: call with n_heads = 1 for that behaviour. */
int pk_rope(void* stream, int dtype, void* x, int64_t ld, int64_t col0, int n_heads,
            int head_dim, const int32_t* pos, const float* cos_sin, int64_t n_pos,
            int64_t R, int inverse);

/* C = rope(A . op(B) + bias) for bf16 operands and output: pk_gemm followed by pk_rope on columns
 * [0, n_heads * head_dim) of C, in one launch -- the rotation happens in the GEMM's epilogue on the
 * value rounded to bf16, so the result is bit-identical to the two calls (the q and k
 * projections of src/llama.cpp:30-36, which concatenates q, k, v and calls ops::apply_rope). trans_b as in pk_gemm. Takes
 * head_dim 64 or 128 and the shapes the CTA-pair kernel takes (M, N >= 256, enough 256 x 256
 * tiles, 16-byte aligned operands); otherwise PK_ERR_UNSUPPORTED and the caller makes the two calls. */
int pk_gemm_rope(void* stream, int trans_b, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                 const void* B, int64_t ldb, void* C, int64_t ldc, const float* bias, const int32_t* pos,
                 const float* cos_sin, int64_t n_pos, int n_heads, int head_dim, int inverse);

/* ---- activations / elementwise ---------------------------------------------
 * SwiGLU y = silu(g) * u and its backward: ops::silu + ops::mul
 * (src/ops.cpp:404-424, 76-83). GELU (tanh form, correct derivative):
 * ops::gelu (src/ops.cpp:106-138), k_gelu_fwd/bwd (src/cuda_ops.cu:125-150).
 * ReLU: ops::relu (src/ops.cpp:788-801). n = element count. Every backward of this group may
 * write its result over one of its inputs (dg == g and du == u for SwiGLU): an element is read
 * before it is written and belongs to one thread. */
int pk_swiglu_fwd(void* stream, int dtype, const void* g, const void* u, void* y, int64_t n);
int pk_swiglu_bwd(void* stream, int dtype, const void* dy, const void* g, const void* u,
                  void* dg, void* du, int64_t n);
int pk_silu_fwd(void* stream, int dtype, const void* x, void* y, int64_t n);
int pk_silu_bwd(void* stream, int dtype, const void* dy, const void* x, void* dx, int64_t n);
int pk_gelu_fwd(void* stream, int dtype, const void* x, void* y, int64_t n);
int pk_gelu_bwd(void* stream, int dtype, const void* dy, const void* x, void* dx, int64_t n);
int pk_relu_fwd(void* stream, int dtype, const void* x, void* y, int64_t n);
int pk_relu_bwd(void* stream, int dtype, const void* dy, const void* x, void* dx, int64_t n);
/* Row softmax y[i,:] = softmax(x[i,:]) (maximum subtracted) and its backward
 * dx = s .* (dy - rowsum(dy .* s)) with s the forward's output: ops::softmax_row
 * (src/ops.cpp:140-167), devops::softmax_fwd / softmax_bwd. */
int pk_softmax_fwd(void* stream, int dtype, const void* x, void* y, int64_t R, int64_t C);
int pk_softmax_bwd(void* stream, int dtype, const void* s, const void* dy, void* dx, int64_t R, int64_t C);
/* y = a (op) b, op: 0 add, 1 sub, 2 mul. ops::add/sub/mul (src/ops.cpp:60-83),
 * devops::add/sub/mul (device_cache.hpp:99-101). */
int pk_binary(void* stream, int dtype, int op, const void* a, const void* b, void* y, int64_t n);
/* y = alpha * x (ops::scale, src/ops.cpp:184-190); y may alias x. */
int pk_scale(void* stream, int dtype, const void* x, float alpha, void* y, int64_t n);
/* y += alpha * x, the gradient-accumulate shape (devops::axpy; Variable::accumulate,
 * src/autograd.cpp:16-24). x has dtype x_dtype, y has dtype y_dtype. */
int pk_axpy(void* stream, int y_dtype, void* y, int x_dtype, const void* x, float alpha, int64_t n);
int pk_cast(void* stream, int src_dtype, const void* src, int dst_dtype, void* dst, int64_t n);
/* y[R,C] = x[R,C] + b[C] (ops::add_bias, src/ops.cpp:85-104); b fp32. */
int pk_add_bias(void* stream, int dtype, const void* x, const float* b, void* y, int64_t R, int64_t C);
/* out[C] += column sums of x[R,C] (the db of add_bias), fp32 out, deterministic. */
size_t pk_colsum_scratch_bytes(int64_t R, int64_t C);
int pk_colsum(void* stream, int dtype, const void* x, float* out, void* scratch, int64_t R, int64_t C);
/* dst[r, dcol0 + j] (+)= src[r, scol0 + j], j < ncols: ops::slice_cols /
 * ops::concat_cols and their backward scatters (src/ops.cpp:200-246). */
int pk_copy_cols(void* stream, int dtype, const void* src, int64_t lds, int64_t scol0,
                 void* dst, int64_t ldd, int64_t dcol0, int64_t R, int64_t ncols, int accumulate);
/* y[C,R] = x[R,C]^T (ops::transpose, src/ops.cpp:192-198). */
int pk_transpose(void* stream, int dtype, const void* x, void* y, int64_t R, int64_t C);

/* ---- attention ---------------------------------------------------------------
 * Causal (or bidirectional) softmax attention over B stacked sequences of
 * length S, all heads in one call, never materialising the score matrix.
 * q is [B*S, Hq*dk] with row stride ldq, k/v are [B*S, Hkv*dk]; query head h
 * reads kv head h / (Hq/Hkv). out has q's shape (row stride ldo); lse is fp32
 * [B*S, Hq] (log-sum-exp of the scaled scores), saved for backward.
 * Replaces the per-head slice_cols + ops::fused_attention loop
 * (src/llama.cpp:44-52, src/nn.cpp:144-150; op at src/ops.cpp:863-934). A
 * row attends keys [sequence start, i] when causal, the whole sequence
 * otherwise; rows of different sequences never see each other. */
int pk_attn_fwd(void* stream, int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk,
                const void* v, int64_t ldv, void* out, int64_t ldo, float* lse,
                int64_t B, int64_t S, int Hq, int Hkv, int dk, float scale, int causal);
/* delta is fp32 scratch [B*S, Hq]. dq/dk/dv are overwritten (row strides lddq, lddk, lddv). */
size_t pk_attn_bwd_scratch_bytes(int64_t B, int64_t S, int Hq);
int pk_attn_bwd(void* stream, int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk,
                const void* v, int64_t ldv, const void* out, int64_t ldo, const float* lse,
                const void* dout, int64_t lddo, void* dq, int64_t lddq, void* dk_, int64_t lddk,
                void* dv, int64_t lddv, void* scratch,
                int64_t B, int64_t S, int Hq, int Hkv, int dk, float scale, int causal);
/* 0 = SIMT fp32-math kernel, 1 = tensor-core kernel (last call on this thread). bf16 with
 * head_dim 64 or 128 and 16-byte aligned rows takes the tcgen05 kernels. */
int pk_attn_last_path(void);
/* Status word of the tensor-core attention kernels (PK_ERR_TIMEOUT when a bounded wait
 * gave up). Synchronises the device; clear != 0 resets it. A host that launches these kernels
 * should read (and clear) the word wherever it synchronises anyway: a launch that timed out
 * has left its outputs incomplete. */
int pk_attn_tc_status(int* status_h, int clear);
int pk_attn_force_simt(int on);
/* All status words of the tensor-core kernels (GEMM and attention) ORed together, without a
 * device synchronisation: for a host that has just synchronised the stream it launched on (a
 * training step reading its loss back). clear != 0 resets the words that were set. */
int pk_kernel_status(int* status_h, int clear);
/* Limit of the bounded device-side waits of every tensor-core kernel (GEMM and attention): a
 * wait on an mbarrier that lasts longer gives up, ORs PK_ERR_TIMEOUT into its family's status
 * word and lets the kernel drain and return (no trap, tensor memory released). Default 2 s;
 * the limit is given in microseconds and converted to SM clock cycles at the highest clock, so
 * a wait never gives up earlier than asked. Applies to launches made after the call. */
int pk_set_wait_limit_us(double microseconds);
/* Self-test of that path: one warp waits on an mbarrier nobody arrives at, under the current
 * limit. On return *status_h holds the status the wait recorded (PK_ERR_TIMEOUT expected; the
 * word is cleared) and *waited_us_h how long the warp waited. Synchronises the stream and
 * allocates 8 bytes for the duration of the call. The status words of the GEMM and attention
 * kernels are separate and stay untouched. */
int pk_wait_selftest(void* stream, int* status_h, double* waited_us_h);

/* ---- embedding / loss --------------------------------------------------------
 * Row gather out[i,:] = table[ids[i],:] (pure copy; table has the out dtype).
 * ops::embedding forward (src/ops.cpp:329-337). An id outside [0,V) ORs
 * PK_ERR_INDEX into *status (int32, device) and writes zeros. */
int pk_embedding_fwd(void* stream, int dtype, const void* table, const int32_t* ids, void* out,
                     int64_t R, int64_t d, int64_t V, int32_t* status);
/* dtable[uniq[u],:] += sum over p in order[seg[u]..seg[u+1]) of dy[p,:], summed in
 * ascending position order (the order the reference's scatter-add loop uses,
 * src/ops.cpp:338-347). order/seg/uniq are built on the host from the ids. */
int pk_embedding_bwd(void* stream, int dtype, const void* dy, const int32_t* order,
                     const int32_t* seg, const int32_t* uniq, int64_t n_uniq, float* dtable,
                     int64_t d);
/* Cross entropy over rows of logits [R,V]: row_loss[i] = -log(max(softmax_i[t_i], 1e-12)).
 * When want_grad != 0 the logits are OVERWRITTEN with (softmax - onehot) * grad_scale.
 * ops::cross_entropy (src/ops.cpp:350-376). A target outside [0,V) sets *status. */
int pk_cross_entropy(void* stream, int dtype, void* logits, int64_t ld, const int32_t* targets,
                     float* row_loss, int64_t R, int64_t V, float grad_scale, int want_grad,
                     int32_t* status);
/* out[0] (double) = sum of x[0..n) in a fixed tree order, accumulated in fp64
 * (the reference sums the NLL and the grad norm in double). square != 0 sums x^2.
 * add != 0 adds to out[0] instead of overwriting. scratch: pk_reduce_scratch_bytes(). */
size_t pk_reduce_scratch_bytes(void);
int pk_reduce_sum_f64(void* stream, const float* x, int64_t n, int square, int add, double* out,
                      void* scratch);

/* out[0] = float(sum[0] / denom): turns the fp64 NLL sum into the mean loss without a
 * host round trip (ops::cross_entropy, src/ops.cpp:368: out = float(nll / R)). */
int pk_sum_to_mean(void* stream, const double* sum, double denom, float* out);
/* dst[0..n) = value (devops::fill, include/microtorch/device_cache.hpp:104). */
int pk_fill(void* stream, int dtype, void* dst, float value, int64_t n);

/* ---- optimizer ---------------------------------------------------------------
 * AdamW::step (src/nn.cpp:301-321) over a flat fp32 buffer: m,v EMA, bias
 * correction c1 = 1-b1^t, c2 = 1-b2^t computed by the caller in float,
 * p -= lr * ((m/c1)/(sqrt(v/c2)+eps) + wd*p). p_bf16 (nullable) receives the
 * rounded copy of the new p in the same pass. */
int pk_adamw(void* stream, float* p, const float* g, float* m, float* v, int64_t n,
             float lr, float b1, float b2, float eps, float wd, float c1, float c2,
             void* p_bf16);
/* Q8_0: blocks of 32 along a row of W[rows, cols] (cols % 32 == 0), int8 values and an
 * fp16 scale = fp16(absmax/127) (1.0 for an all-zero block); q = round-half-away(clamp(x/s)).
 * quantize_int8 / dequantize (src/quant.cpp:11-48) with block 32 and the scale stored as fp16.
 * Dequantisation is one fp32 multiply float(q) * float(scale), then a cast to out_dtype. */
int pk_q8_quantize(void* stream, const float* W, int8_t* q, uint16_t* scales, int64_t rows, int64_t cols);
int pk_q8_dequantize(void* stream, const int8_t* q, const uint16_t* scales, int out_dtype, void* out,
                     int64_t rows, int64_t cols);
/* The reference's own block quantisation (src/quant.cpp:11-48) for any block length, a short last
 * block included: fp32 scale = absmax / 127 per block (1.0 for an all-zero block), scales
 * [rows, ceil(cols / block)], q = round-half-away(clamp(x / s, -127, 127)); dequantisation is
 * float(q) * scale. Bit-identical to the reference on the same input. */
int pk_q8_quantize_block(void* stream, const float* W, int8_t* q, float* scales, int64_t rows, int64_t cols,
                         int64_t block);
int pk_q8_dequantize_block(void* stream, const int8_t* q, const float* scales, int64_t block, int out_dtype, void* out,
                           int64_t rows, int64_t cols);
/* Fused dequantise-GEMM over a frozen Q8_0 weight with the LoRA side path in the same accumulator:
 *     C[M,N] (+)= A[M,K] . deq(W) + XA[M,r] . L (+ bias) (+ residual)
 * A, XA, L are bf16; accumulation is fp32 in tensor memory; C / residual have c_dtype.
 *   trans_w = 0   W is the quantised matrix [K, N] with scales [K, N/32]; L is [r, N].
 *                 The forward of QLinear / QLoRALinear: y = x deq(W) + (s x A) B with XA = s x A,
 *                 L = B (src/quant.cpp:91-119; the reference multiplies by a dequantised fp32 copy).
 *   trans_w = 1   W is [N, K] with scales [N, K/32] and is used transposed; L is [N, r], used
 *                 transposed. The input gradient: dx = dy deq(W)^T + (s dy B^T) A^T.
 * XA == NULL (r = 0) leaves the LoRA term out. The int8 tiles and their fp16 scales are brought
 * into shared memory, expanded there to bf16 -- float(q) * float(scale) in fp32, one rounding to
 * bf16, the bits pk_q8_dequantize writes -- straight into the swizzled operand buffer that
 * tcgen05.mma reads; the weight never exists in bf16 in global memory. The result equals
 * pk_gemm over [A | XA] and [deq(W); L] bit for bit (same products, same k order).
 * Needs: W's column count a multiple of 128 (trans_w = 0) or of 64 (trans_w = 1), N a multiple
 * of 8, 16-byte aligned bases, lda / ldxa / ldl / ldc / ldr multiples of 8, r a multiple of 8
 * and <= 64. Other requests return PK_ERR_UNSUPPORTED; the
 * caller can always dequantise and call pk_gemm. pk_gemm_last_path reports 4. */
int pk_gemm_q8_lora(void* stream, int c_dtype, int trans_w, int64_t M, int64_t N, int64_t K,
                    const void* A, int64_t lda, const int8_t* Wq, const uint16_t* scales,
                    const void* XA, int64_t ldxa, const void* L, int64_t ldl, int r,
                    void* C, int64_t ldc, int accumulate, const float* bias, const void* residual, int64_t ldr);


/* ---- collectives -------------------------------------------------------------
 * Sum all-reduce of fp32 gradient ranges between the ranks of a data-parallel job (one process
 * per GPU), asynchronous behind the compute stream so that the exchange of one block's gradients
 * overlaps the recompute + backward of the next. The reference has no multi-GPU path; the
 * identity used -- every rank pre-scales its loss and the gradients are summed -- is the one of
 * its gradient accumulation loop (tools/mtstudio.cpp:456-474).
 *   pk_comm_unique_id   rank 0 draws the 128-byte NCCL id; the host distributes it (any channel)
 *   pk_comm_init        every rank, with its GPU current: builds the NCCL communicator and a
 *                       private communication stream. max_ctas > 0 caps the CTAs NCCL's kernels
 *                       use (SMs they take from the kernels they overlap); 0 = NCCL's default.
 *                       NCCL is opened at run time (libnccl.so.2); absent -> PK_ERR_COMM.
 *   pk_comm_init_file   CPU ranks exchanging HOST buffers through an existing directory: for
 *                       exercising the host-side protocol without GPUs. The files stay there.
 *   pk_allreduce_async  buf[0..count) = sum over ranks, in place. NCCL backend: starts once the
 *                       work enqueued so far on compute_stream has finished; returns at once.
 *   pk_comm_wait        orders compute_stream behind every collective started so far (no host
 *                       block) and reports an asynchronous communicator error if there is one.
 *                       File backend: completes the collectives on the host.
 *   pk_comm_wait_host   blocks the host until they have finished, polling the communicator's
 *                       error state; after the time limit (pk_comm_set_timeout, default 30 s) it
 *                       aborts the communicator and returns PK_ERR_TIMEOUT.
 *   pk_comm_abort       ncclCommAbort: ends the communicator's kernels; every later call on the
 *                       handle returns PK_ERR_COMM. pk_comm_destroy frees the handle.
 * All ranks must start the same collectives in the same order. One host thread per handle. */
int pk_comm_unique_id(void* id_h, size_t cap);
int pk_comm_init(const void* id_h, int rank, int world, int max_ctas, void** comm_h);
int pk_comm_init_file(const char* dir, int rank, int world, void** comm_h);
int pk_comm_set_timeout(void* comm, double seconds);
int pk_comm_info(void* comm, int* rank_h, int* world_h, int* backend_h, int* alive_h);
int pk_allreduce_async(void* comm, float* buf, int64_t count, void* compute_stream);
int pk_comm_wait(void* comm, void* compute_stream);
int pk_comm_wait_host(void* comm);
int pk_comm_abort(void* comm);
int pk_comm_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif /* PK_H_ */
