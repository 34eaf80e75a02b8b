// Embedding gather / deterministic scatter-add, row-wise cross entropy with the
// gradient written in place, and a fixed-order fp64 sum reduction.
//
// Reference behaviour: ops::embedding (src/ops.cpp:329-348) and ops::cross_entropy
// (src/ops.cpp:350-376, softmax from third_party/transformer_cpp/src/components.cpp:229-252).
// Out-of-range ids / targets do not trap: they OR PK_ERR_INDEX into a device status word.
#include "pk_common.cuh"

namespace pk {

template <typename T>
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, T* __restrict__ out,
                     int64_t R, int64_t d, int64_t V, int32_t* status, bool vec) {
    constexpr int N = Vec<T>::N;
    const int64_t per_row = vec ? d / N : d;
    const int64_t total = R * per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t row = i / per_row, c = i % per_row;
        const int64_t id = ids[row];
        const bool ok = id >= 0 && id < V;
        if (!ok && c == 0 && status) atomicOr(status, PK_ERR_INDEX);
        if (vec) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (ok) v = *reinterpret_cast<const uint4*>(table + id * d + c * N);
            *reinterpret_cast<uint4*>(out + row * d + c * N) = v;
        } else {
            out[row * d + c] = ok ? table[id * d + c] : from_f32<T>(0.0f);
        }
    }
}

// One block per distinct id; threads own columns; rows are added in the order given.
template <typename T>
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const T* __restrict__ dy, const int32_t* __restrict__ order,
                     const int32_t* __restrict__ seg, const int32_t* __restrict__ uniq,
                     float* __restrict__ dtable, int64_t d) {
    const int64_t u = blockIdx.x;
    const int64_t id = uniq[u];
    const int32_t p0 = seg[u], p1 = seg[u + 1];
    for (int64_t c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = dtable[id * d + c];
        for (int32_t p = p0; p < p1; ++p) acc += to_f32(dy[static_cast<int64_t>(order[p]) * d + c]);
        dtable[id * d + c] = acc;
    }
}

// One block per row, the row read ONCE: thread t keeps vectors t, t + blockDim, ... (at most
// CE_VPT of them, packed as loaded) in registers across the three phases (max, sum of exp,
// write). Used when the row fits: V / N <= blockDim * CE_VPT; longer rows take the sweep kernel
// below (same arithmetic per element; the threads' partial sums group differently).
constexpr int CE_VPT = 8;

// exp(x - mx): fp32 logits take expf (the reference's std::exp to within an ulp or two); bf16
// logits carry 8 bits, so ex2.approx of the pre-scaled difference is far inside their noise.
template <typename T> struct CeExp {
    float mx;
    __device__ __forceinline__ explicit CeExp(float m) : mx(m) {}
    __device__ __forceinline__ float operator()(float x) const { return expf(x - mx); }
};
template <> struct CeExp<bf16> {
    float neg_mx2;
    __device__ __forceinline__ explicit CeExp(float m) : neg_mx2(-m * 1.4426950408889634f) {}
    __device__ __forceinline__ float operator()(float x) const {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmaf(x, 1.4426950408889634f, neg_mx2)));
        return y;
    }
};

template <typename T>
__global__ void __launch_bounds__(512, 2)
cross_entropy_row_kernel(T* __restrict__ logits, int64_t ld, const int32_t* __restrict__ targets,
                         float* __restrict__ row_loss, int64_t R, int64_t V, float gscale, int want_grad,
                         int32_t* status) {
    constexpr int N = Vec<T>::N;
    __shared__ float red[32];
    const int64_t nv = V / N;
    for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
        T* lr = logits + row * ld;
        uint4 raw[CE_VPT];
#pragma unroll
        for (int k = 0; k < CE_VPT; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
            if (i < nv) raw[k] = Vec<T>::load_raw(lr + i * N);
        }
        float mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < CE_VPT; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
            if (i < nv) {
                float f[N];
                Vec<T>::unpack(raw[k], f);
#pragma unroll
                for (int e = 0; e < N; ++e) mx = fmaxf(mx, f[e]);
            }
        }
        for (int64_t c = nv * N + threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, to_f32(lr[c]));
        mx = block_max(mx, red);
        const CeExp<T> ex(mx);
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < CE_VPT; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
            if (i < nv) {
                float f[N];
                Vec<T>::unpack(raw[k], f);
#pragma unroll
                for (int e = 0; e < N; ++e) sum += ex(f[e]);
            }
        }
        for (int64_t c = nv * N + threadIdx.x; c < V; c += blockDim.x) sum += ex(to_f32(lr[c]));
        sum = block_sum(sum, red);
        int64_t t = targets[row];
        const bool ok = t >= 0 && t < V;
        if (!ok) {
            if (threadIdx.x == 0 && status) atomicOr(status, PK_ERR_INDEX);
            t = 0;
        }
        if (threadIdx.x == 0) {
            const float pt = ex(to_f32(lr[t])) / sum;
            row_loss[row] = ok ? -logf(fmaxf(pt, 1e-12f)) : 0.0f;
        }
        if (want_grad) {
            __syncthreads();  // lr[t] has been read before anyone overwrites it
            const float inv = 1.0f / sum;
#pragma unroll
            for (int k = 0; k < CE_VPT; ++k) {
                const int64_t i = threadIdx.x + static_cast<int64_t>(k) * blockDim.x;
                if (i < nv) {
                    float f[N];
                    Vec<T>::unpack(raw[k], f);
                    const int64_t te = t - i * N;  // the target's slot in this vector, if any
#pragma unroll
                    for (int e = 0; e < N; ++e) {
                        float p = ex(f[e]) * inv;
                        if (te == e) p -= 1.0f;
                        f[e] = p * gscale;
                    }
                    Vec<T>::store(lr + i * N, f);
                }
            }
            for (int64_t c = nv * N + threadIdx.x; c < V; c += blockDim.x) {
                float p = ex(to_f32(lr[c])) * inv;
                if (c == t) p -= 1.0f;
                lr[c] = from_f32<T>(p * gscale);
            }
        }
        __syncthreads();
    }
}

// One block per row. Three sweeps over the row (max, sum of exp, write), the last two
// served from L2. p = exp(l - max) / sum; loss = -log(max(p_t, 1e-12)).
template <typename T>
__global__ void __launch_bounds__(512)
cross_entropy_kernel(T* __restrict__ logits, int64_t ld, const int32_t* __restrict__ targets,
                     float* __restrict__ row_loss, int64_t R, int64_t V, float gscale, int want_grad,
                     int32_t* status, bool vec) {
    constexpr int N = Vec<T>::N;
    __shared__ float red[32];
    for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
        T* lr = logits + row * ld;
        const int64_t nv = vec ? V / N : 0;
        float mx = -INFINITY;
        for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
            float f[N];
            Vec<T>::load(lr + i * N, f);
#pragma unroll
            for (int e = 0; e < N; ++e) mx = fmaxf(mx, f[e]);
        }
        for (int64_t c = nv * N + threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, to_f32(lr[c]));
        mx = block_max(mx, red);
        const CeExp<T> ex(mx);
        float sum = 0.0f;
        for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
            float f[N];
            Vec<T>::load(lr + i * N, f);
#pragma unroll
            for (int e = 0; e < N; ++e) sum += ex(f[e]);
        }
        for (int64_t c = nv * N + threadIdx.x; c < V; c += blockDim.x) sum += ex(to_f32(lr[c]));
        sum = block_sum(sum, red);
        int64_t t = targets[row];
        const bool ok = t >= 0 && t < V;
        if (!ok) {
            if (threadIdx.x == 0 && status) atomicOr(status, PK_ERR_INDEX);
            t = 0;
        }
        if (threadIdx.x == 0) {
            const float pt = ex(to_f32(lr[t])) / sum;
            row_loss[row] = ok ? -logf(fmaxf(pt, 1e-12f)) : 0.0f;
        }
        if (want_grad) {
            __syncthreads();  // lr[t] has been read before anyone overwrites it
            const float inv = 1.0f / sum;
            for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
                float f[N];
                Vec<T>::load(lr + i * N, f);
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    float p = ex(f[e]) * inv;
                    if (i * N + e == t) p -= 1.0f;
                    f[e] = p * gscale;
                }
                Vec<T>::store(lr + i * N, f);
            }
            for (int64_t c = nv * N + threadIdx.x; c < V; c += blockDim.x) {
                float p = ex(to_f32(lr[c])) * inv;
                if (c == t) p -= 1.0f;
                lr[c] = from_f32<T>(p * gscale);
            }
        }
        __syncthreads();
    }
}

constexpr int RED_BLOCKS = 512;
__global__ void __launch_bounds__(256)
reduce_stage1(const float* __restrict__ x, int64_t n, int square, double* __restrict__ partial) {
    __shared__ double red[8];
    double acc = 0.0;
    // contiguous chunk per block, strided by thread inside the chunk
    const int64_t chunk = (n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = chunk * blockIdx.x;
    int64_t hi = lo + chunk;
    if (hi > n) hi = n;
    for (int64_t i = lo + threadIdx.x; i < hi; i += 256) {
        const double v = x[i];
        acc += square ? v * v : v;
    }
    acc = warp_sum_f64(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}
__global__ void reduce_stage2(const double* __restrict__ partial, int nparts, int add, double* out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    double t = 0.0;
    for (int i = 0; i < nparts; ++i) t += partial[i];
    out[0] = add ? out[0] + t : t;
}

__global__ void sum_to_mean_kernel(const double* sum, double denom, float* out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = static_cast<float>(sum[0] / denom);
}

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* p, float v, int64_t n) {
    const T tv = from_f32<T>(v);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * 256)
        p[i] = tv;
}

}  // namespace pk

using namespace pk;

extern "C" {

int pk_embedding_fwd(void* stream, int dtype, const void* table, const int32_t* ids, void* out,
                     int64_t R, int64_t d, int64_t V, int32_t* status) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && d > 0 && V > 0, "bad shape");
    if (R == 0) return PK_OK;
    PK_REQUIRE(table && ids && out, "null pointer");
    const int nvec = dtype == PK_F32 ? 4 : 8;
    const bool vec = d % nvec == 0 && aligned16(table) && aligned16(out);
    const int64_t total = R * (vec ? d / nvec : d);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == PK_F32)
        embedding_fwd_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<const float*>(table), ids, static_cast<float*>(out), R, d, V, status, vec);
    else
        embedding_fwd_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(table), ids, static_cast<bf16*>(out), R, d, V, status, vec);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_embedding_bwd(void* stream, int dtype, const void* dy, const int32_t* order, const int32_t* seg,
                     const int32_t* uniq, int64_t n_uniq, float* dtable, int64_t d) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(n_uniq >= 0 && d > 0, "bad shape");
    if (n_uniq == 0) return PK_OK;
    PK_REQUIRE(dy && order && seg && uniq && dtable, "null pointer");
    const int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
    if (dtype == PK_F32)
        embedding_bwd_kernel<float><<<static_cast<unsigned>(n_uniq), threads, 0, as_stream(stream)>>>(
            static_cast<const float*>(dy), order, seg, uniq, dtable, d);
    else
        embedding_bwd_kernel<bf16><<<static_cast<unsigned>(n_uniq), threads, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(dy), order, seg, uniq, dtable, d);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_cross_entropy(void* stream, int dtype, void* logits, int64_t ld, const int32_t* targets,
                     float* row_loss, int64_t R, int64_t V, float grad_scale, int want_grad,
                     int32_t* status) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && V > 0 && ld >= V, "bad shape");
    if (R == 0) return PK_OK;
    PK_REQUIRE(logits && targets && row_loss, "null pointer");
    const int nvec = dtype == PK_F32 ? 4 : 8;
    // rows start on 16-byte boundaries when ld is a multiple of the vector width; a ragged
    // tail of V is handled element by element
    const bool vec = ld % nvec == 0 && aligned16(logits);
    int64_t blocks = R;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const int threads = V >= 4096 ? 512 : (V >= 1024 ? 256 : 128);
    if (vec && V / nvec <= static_cast<int64_t>(threads) * CE_VPT) {
        if (dtype == PK_F32)
            cross_entropy_row_kernel<float><<<static_cast<unsigned>(blocks), threads, 0, as_stream(stream)>>>(
                static_cast<float*>(logits), ld, targets, row_loss, R, V, grad_scale, want_grad, status);
        else
            cross_entropy_row_kernel<bf16><<<static_cast<unsigned>(blocks), threads, 0, as_stream(stream)>>>(
                static_cast<bf16*>(logits), ld, targets, row_loss, R, V, grad_scale, want_grad, status);
        PK_LAUNCH_CHECK();
        return PK_OK;
    }
    if (dtype == PK_F32)
        cross_entropy_kernel<float><<<static_cast<unsigned>(blocks), threads, 0, as_stream(stream)>>>(
            static_cast<float*>(logits), ld, targets, row_loss, R, V, grad_scale, want_grad, status, vec);
    else
        cross_entropy_kernel<bf16><<<static_cast<unsigned>(blocks), threads, 0, as_stream(stream)>>>(
            static_cast<bf16*>(logits), ld, targets, row_loss, R, V, grad_scale, want_grad, status, vec);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

size_t pk_reduce_scratch_bytes(void) { return RED_BLOCKS * sizeof(double); }

int pk_reduce_sum_f64(void* stream, const float* x, int64_t n, int square, int add, double* out,
                      void* scratch) {
    PK_REQUIRE(n >= 0 && out && scratch, "bad argument");
    PK_REQUIRE(n == 0 || x, "null pointer");
    int blocks = RED_BLOCKS;
    if (n < static_cast<int64_t>(blocks) * 256) blocks = static_cast<int>((n + 255) / 256);
    if (blocks < 1) blocks = 1;
    double* partial = static_cast<double*>(scratch);
    reduce_stage1<<<blocks, 256, 0, as_stream(stream)>>>(x, n, square, partial);
    PK_LAUNCH_CHECK();
    reduce_stage2<<<1, 32, 0, as_stream(stream)>>>(partial, blocks, add, out);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_sum_to_mean(void* stream, const double* sum, double denom, float* out) {
    PK_REQUIRE(sum && out && denom != 0.0, "bad argument");
    sum_to_mean_kernel<<<1, 32, 0, as_stream(stream)>>>(sum, denom, out);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int pk_fill(void* stream, int dtype, void* dst, float value, int64_t n) {
    PK_REQUIRE(valid_dtype(dtype) && n >= 0, "bad argument");
    if (n == 0) return PK_OK;
    PK_REQUIRE(dst != nullptr, "null pointer");
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == PK_F32)
        fill_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(static_cast<float*>(dst), value, n);
    else
        fill_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(static_cast<bf16*>(dst), value, n);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // extern "C"
