// Row softmax forward / backward (ops::softmax_row of the reference, src/ops.cpp:140-167;
// device seam devops::softmax_fwd / softmax_bwd, include/microtorch/device_cache.hpp:97-127).
// Not on the fused-attention path -- the attention kernels never materialise scores -- but part
// of the op set the reference's bindings and layer tests call. One warp per row, the row read
// three times (maximum, sum, normalise); fp32 arithmetic, fixed shuffle order: deterministic.
#include "pk_common.cuh"

namespace pk {

template <typename T>
__global__ void __launch_bounds__(256)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t R, int64_t C) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < R; r += warps) {
        const T* xr = x + r * C;
        float m = -INFINITY;
        for (int64_t j = lane; j < C; j += 32) m = fmaxf(m, to_f32(xr[j]));
        m = warp_max(m);
        float s = 0.0f;
        for (int64_t j = lane; j < C; j += 32) s += expf(to_f32(xr[j]) - m);
        s = warp_sum(s);
        const float inv = 1.0f / s;
        for (int64_t j = lane; j < C; j += 32) y[r * C + j] = from_f32<T>(expf(to_f32(xr[j]) - m) * inv);
    }
}

// dx = s .* (dy - rowsum(dy .* s))
template <typename T>
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const T* __restrict__ s, const T* __restrict__ dy, T* __restrict__ dx, int64_t R, int64_t C) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < R; r += warps) {
        float dot = 0.0f;
        for (int64_t j = lane; j < C; j += 32) dot += to_f32(dy[r * C + j]) * to_f32(s[r * C + j]);
        dot = warp_sum(dot);
        for (int64_t j = lane; j < C; j += 32)
            dx[r * C + j] = from_f32<T>(to_f32(s[r * C + j]) * (to_f32(dy[r * C + j]) - dot));
    }
}

}  // namespace pk

using namespace pk;

extern "C" {

int pk_softmax_fwd(void* stream, int dtype, const void* x, void* y, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C >= 0, "negative shape");
    if (R == 0 || C == 0) return PK_OK;
    PK_REQUIRE(x && y, "null pointer");
    int64_t blocks = (R + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == PK_F32)
        softmax_fwd_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<const float*>(x), static_cast<float*>(y), R, C);
    else
        softmax_fwd_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(x), static_cast<bf16*>(y), R, C);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_softmax_bwd(void* stream, int dtype, const void* s, const void* dy, void* dx, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C >= 0, "negative shape");
    if (R == 0 || C == 0) return PK_OK;
    PK_REQUIRE(s && dy && dx, "null pointer");
    int64_t blocks = (R + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == PK_F32)
        softmax_bwd_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<const float*>(s), static_cast<const float*>(dy), static_cast<float*>(dx), R, C);
    else
        softmax_bwd_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(s), static_cast<const bf16*>(dy), static_cast<bf16*>(dx), R, C);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // extern "C"
