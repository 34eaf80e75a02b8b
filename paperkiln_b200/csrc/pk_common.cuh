// Shared helpers for the libpk kernels: error reporting, 128-bit vector IO for
// fp32 / bf16 storage with fp32 arithmetic, warp and block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#include "pk.h"

namespace pk {

void set_error(const char* fmt, ...);

#define PK_CHECK_CUDA(expr)                                                             \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess) {                                                        \
            pk::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),       \
                          __FILE__, __LINE__);                                          \
            return PK_ERR_CUDA;                                                         \
        }                                                                               \
    } while (0)

#define PK_REQUIRE(cond, msg)                                           \
    do {                                                                \
        if (!(cond)) {                                                  \
            pk::set_error("%s: %s (%s)", __func__, msg, #cond);         \
            return PK_ERR_INVALID;                                      \
        }                                                               \
    } while (0)

#define PK_LAUNCH_CHECK()                                                              \
    do {                                                                               \
        cudaError_t _e = cudaGetLastError();                                           \
        if (_e != cudaSuccess) {                                                       \
            pk::set_error("%s: launch failed: %s", __func__, cudaGetErrorString(_e));  \
            return PK_ERR_CUDA;                                                        \
        }                                                                              \
    } while (0)

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline size_t dtype_size(int dt) { return dt == PK_BF16 ? 2 : 4; }
inline bool valid_dtype(int dt) { return dt == PK_F32 || dt == PK_BF16; }

// Optional per-kernel-class timing with CUDA events on the launching stream (off by
// default). A ProfScope placed around a launch records the pair of events; the totals
// are read with pk_prof_summary().
enum ProfKind { PROF_GEMM_TC = 0, PROF_GEMM_SIMT = 1, PROF_ATTN_FWD = 2, PROF_ATTN_BWD = 3, PROF_KINDS = 4 };
struct ProfScope {
    ProfScope(int kind, double work, cudaStream_t st);
    ~ProfScope();
    int slot;
    cudaStream_t st;
};

// Launches per kernel path since the last reset (pk_launch_counts): which kernel a call took is
// otherwise visible only for the last call of a thread.
enum PathSlot {
    PATH_GEMM_SIMT_F32 = 0, PATH_GEMM_SIMT_BF16 = 1, PATH_GEMM_TC = 2, PATH_GEMM_TC_PAIR = 3, PATH_GEMM_Q8 = 4,
    PATH_ATTN_FWD_SIMT = 5, PATH_ATTN_FWD_TC = 6, PATH_ATTN_BWD_SIMT = 7, PATH_ATTN_BWD_TC = 8, PATH_SLOTS = 9
};
void note_launch(int slot);

// Number of SMs of the current device (cached); grids of the bandwidth-bound
// kernels are sized in multiples of it.
int sm_count();

// Split-K support shared by the two tensor-core GEMM kernels (defined with the one-CTA kernel):
// the caller's workspace, the second stage that adds `splits` fp32 partial slabs in ascending
// order and applies bias / residual / accumulate, and the count reported by pk_gemm_last_splits.
float* gemm_splitk_workspace(size_t* bytes);
int gemm_splitk_reduce(cudaStream_t st, int c_dtype, const float* partial, int splits, int64_t slab, int64_t pstride,
                       int64_t M, int64_t N, void* C, int64_t ldc, int accumulate, const float* bias,
                       const void* residual, int64_t ldr);
void gemm_note_splits(int splits);


typedef __nv_bfloat16 bf16;

// ---- scalar conversions -----------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- 16-byte vector IO ---------------------------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ __forceinline__ static void store(float* p, const float (&f)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
    // The 16 bytes as loaded, and their conversion: lets a kernel keep a row packed in registers.
    __device__ __forceinline__ static uint4 load_raw(const float* p) {
        return *reinterpret_cast<const uint4*>(p);
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static uint4 load_raw(const bf16* p) {
        return *reinterpret_cast<const uint4*>(p);
    }
    __device__ __forceinline__ static void load(const bf16* p, float (&f)[8]) {
        unpack(load_raw(p), f);
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // bf16 -> fp32 is a 16-bit left shift
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static void store(bf16* p, const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// Rotary embedding applied by a GEMM epilogue to columns [0, cols) of its output.
struct RopeEpilogue {
    const float* cos_sin;   // (cos, sin) per [position, pair]
    const int32_t* pos;     // position of every output row
    int64_t n_pos;
    int half;               // pairs per head
    int64_t cols;           // rotated columns: heads * 2 * half
    float sign;             // +1, or -1 for the inverse rotation
};

// One rotary pair: (x0, x1) turned by the angle whose (cos, sin) is (c, s). Shared by the RoPE
// kernels and by the GEMM epilogue that rotates q / k on their way out, so that all three
// form the same products and sums.
// Every product and sum is rounded on its own (no fused multiply-add), as the reference's CPU loop
// does (src/ops.cpp:495-511), so the three sites cannot contract differently.
__device__ __forceinline__ void rope_rotate(float x0, float x1, float c, float s, float& o0, float& o1) {
    o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    o1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

__host__ __device__ inline bool aligned16(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// ---- reductions ------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Block-wide sum, result broadcast to all threads. `red` is >= 32 floats of smem.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

}  // namespace pk
