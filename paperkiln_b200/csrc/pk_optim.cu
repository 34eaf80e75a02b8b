// AdamW over a flat fp32 parameter buffer (with an optional bf16 shadow written in the
// same pass) and the Q8_0 block quantizer / dequantizer.
//
// Reference behaviour: AdamW::step (src/nn.cpp:301-321); quantize_int8 / dequantize
// (src/quant.cpp:11-48) at block 32 with the per-block scale stored as IEEE binary16.
#include <cuda_fp16.h>

#include "pk_common.cuh"

namespace pk {

__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
             float* __restrict__ v, int64_t n, float lr, float b1, float b2, float eps, float wd,
             float c1, float c2, bf16* __restrict__ shadow, bool vec) {
    const float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t nv = vec ? n / 4 : 0;
    for (int64_t i = tid; i < nv; i += stride) {
        float pp[4], gg[4], mm[4], vv[4];
        Vec<float>::load(p + i * 4, pp);
        Vec<float>::load(g + i * 4, gg);
        Vec<float>::load(m + i * 4, mm);
        Vec<float>::load(v + i * 4, vv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            mm[e] = b1 * mm[e] + omb1 * gg[e];
            vv[e] = b2 * vv[e] + omb2 * gg[e] * gg[e];
            const float upd = (mm[e] / c1) / (sqrtf(vv[e] / c2) + eps);
            pp[e] -= lr * (upd + wd * pp[e]);
        }
        Vec<float>::store(p + i * 4, pp);
        Vec<float>::store(m + i * 4, mm);
        Vec<float>::store(v + i * 4, vv);
        if (shadow) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(pp[0], pp[1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(pp[2], pp[3]);
            uint2 w;
            w.x = *reinterpret_cast<uint32_t*>(&h0);
            w.y = *reinterpret_cast<uint32_t*>(&h1);
            *reinterpret_cast<uint2*>(shadow + i * 4) = w;
        }
    }
    for (int64_t i = nv * 4 + tid; i < n; i += stride) {
        const float gi = g[i];
        const float mi = b1 * m[i] + omb1 * gi;
        const float vi = b2 * v[i] + omb2 * gi * gi;
        m[i] = mi;
        v[i] = vi;
        const float upd = (mi / c1) / (sqrtf(vi / c2) + eps);
        const float pi = p[i] - lr * (upd + wd * p[i]);
        p[i] = pi;
        if (shadow) shadow[i] = __float2bfloat16_rn(pi);
    }
}

// One warp per block of 32 values.
__global__ void __launch_bounds__(256)
q8_quantize_kernel(const float* __restrict__ W, int8_t* __restrict__ q, __half* __restrict__ scales,
                   int64_t nblocks) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); b < nblocks; b += warps) {
        const float x = W[b * 32 + lane];
        const float amax = warp_max(fabsf(x));
        const float s = amax > 0.0f ? amax / 127.0f : 1.0f;
        __half h = __float2half_rn(s);
        if (__half2float(h) == 0.0f) h = __float2half_rn(6.103515625e-05f);
        const float s16 = __half2float(h);
        const float v = fmaxf(-127.0f, fminf(127.0f, x / s16));
        q[b * 32 + lane] = static_cast<int8_t>(static_cast<int>(roundf(v)));
        if (lane == 0) scales[b] = h;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
q8_dequantize_kernel(const int8_t* __restrict__ q, const __half* __restrict__ scales, T* __restrict__ out,
                     int64_t n) {
    // 16 values per thread: one 128-bit load of int8, half a block of 32
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n / 16; i += stride) {
        const uint4 raw = *reinterpret_cast<const uint4*>(q + i * 16);
        const float s = __half2float(scales[i / 2]);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float f[16];
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                f[k * 4 + e] = static_cast<float>(static_cast<int8_t>((w[k] >> (8 * e)) & 0xff)) * s;
#pragma unroll
        for (int e = 0; e < 16; ++e) out[i * 16 + e] = from_f32<T>(f[e]);
    }
}

// Block quantisation with any block length and fp32 scales (the reference's quantize_int8,
// src/quant.cpp:11-37): one warp per (row, block); the last block of a row may be short.
__global__ void __launch_bounds__(256)
q8_quantize_block_kernel(const float* __restrict__ W, int8_t* __restrict__ q, float* __restrict__ scales,
                         int64_t rows, int64_t cols, int64_t block, int64_t bpr) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * 8, n = rows * bpr;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); b < n; b += warps) {
        const int64_t row = b / bpr, j0 = (b % bpr) * block;
        const int64_t j1 = j0 + block < cols ? j0 + block : cols;
        const float* src = W + row * cols;
        float amax = 0.0f;
        for (int64_t j = j0 + lane; j < j1; j += 32) amax = fmaxf(amax, fabsf(src[j]));
        amax = warp_max(amax);
        const float s = amax > 0.0f ? amax / 127.0f : 1.0f;
        for (int64_t j = j0 + lane; j < j1; j += 32) {
            const float v = fmaxf(-127.0f, fminf(127.0f, src[j] / s));
            q[row * cols + j] = static_cast<int8_t>(static_cast<int>(roundf(v)));
        }
        if (lane == 0) scales[b] = s;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
q8_dequantize_block_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, T* __restrict__ out,
                           int64_t rows, int64_t cols, int64_t block, int64_t bpr) {
    const int64_t n = rows * cols, stride = static_cast<int64_t>(gridDim.x) * 256;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += stride) {
        const int64_t row = i / cols, col = i % cols;
        out[i] = from_f32<T>(static_cast<float>(q[i]) * scales[row * bpr + col / block]);
    }
}

}  // namespace pk

using namespace pk;

extern "C" {

int pk_adamw(void* stream, float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1,
             float b2, float eps, float wd, float c1, float c2, void* p_bf16) {
    PK_REQUIRE(n >= 0, "negative size");
    if (n == 0) return PK_OK;
    PK_REQUIRE(p && g && m && v, "null pointer");
    const bool vec = aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v) &&
                     (p_bf16 == nullptr || (reinterpret_cast<uintptr_t>(p_bf16) & 7u) == 0);
    int64_t blocks = ((vec ? n / 4 : n) + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    adamw_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
        p, g, m, v, n, lr, b1, b2, eps, wd, c1, c2, static_cast<bf16*>(p_bf16), vec);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_q8_quantize(void* stream, const float* W, int8_t* q, uint16_t* scales, int64_t rows, int64_t cols) {
    PK_REQUIRE(rows >= 0 && cols >= 0 && cols % 32 == 0, "cols must be a multiple of 32");
    const int64_t nblocks = rows * cols / 32;
    if (nblocks == 0) return PK_OK;
    PK_REQUIRE(W && q && scales, "null pointer");
    int64_t blocks = (nblocks + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    q8_quantize_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
        W, q, reinterpret_cast<__half*>(scales), nblocks);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_q8_dequantize(void* stream, const int8_t* q, const uint16_t* scales, int out_dtype, void* out,
                     int64_t rows, int64_t cols) {
    PK_REQUIRE(valid_dtype(out_dtype), "bad dtype");
    PK_REQUIRE(rows >= 0 && cols >= 0 && cols % 32 == 0, "cols must be a multiple of 32");
    const int64_t n = rows * cols;
    if (n == 0) return PK_OK;
    PK_REQUIRE(q && scales && out, "null pointer");
    PK_REQUIRE(aligned16(q), "q must be 16-byte aligned");
    int64_t blocks = (n / 16 + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (out_dtype == PK_F32)
        q8_dequantize_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            q, reinterpret_cast<const __half*>(scales), static_cast<float*>(out), n);
    else
        q8_dequantize_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            q, reinterpret_cast<const __half*>(scales), static_cast<bf16*>(out), n);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_q8_quantize_block(void* stream, const float* W, int8_t* q, float* scales, int64_t rows, int64_t cols,
                         int64_t block) {
    PK_REQUIRE(rows >= 0 && cols >= 0 && block > 0, "bad shape");
    const int64_t bpr = (cols + block - 1) / block, n = rows * bpr;
    if (n == 0) return PK_OK;
    PK_REQUIRE(W && q && scales, "null pointer");
    int64_t blocks = (n + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    q8_quantize_block_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(W, q, scales, rows, cols, block, bpr);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_q8_dequantize_block(void* stream, const int8_t* q, const float* scales, int64_t block, int out_dtype, void* out,
                           int64_t rows, int64_t cols) {
    PK_REQUIRE(valid_dtype(out_dtype), "bad dtype");
    PK_REQUIRE(rows >= 0 && cols >= 0 && block > 0, "bad shape");
    const int64_t n = rows * cols, bpr = (cols + block - 1) / block;
    if (n == 0) return PK_OK;
    PK_REQUIRE(q && scales && out, "null pointer");
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (out_dtype == PK_F32)
        q8_dequantize_block_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            q, scales, static_cast<float*>(out), rows, cols, block, bpr);
    else
        q8_dequantize_block_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            q, scales, static_cast<bf16*>(out), rows, cols, block, bpr);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // extern "C"
