// Bandwidth-bound elementwise kernels: activations (SwiGLU, SiLU, GELU, ReLU) with
// their backward formulas, binary ops, scale, axpy, casts, bias add, column sums,
// column-range copies and transpose. Every kernel moves 8 elements per thread per
// iteration with 128-bit accesses when the buffers are 16-byte aligned and falls
// back to scalar accesses otherwise; arithmetic is fp32 whatever the storage type.
//
// Formulas follow the reference tape ops (src/ops.cpp: silu 404-424, mul 76-83,
// gelu 106-138, relu 788-801, add/sub 60-74, scale 184-190, add_bias 85-104,
// slice_cols/concat_cols 200-246, transpose 192-198).
#include "pk_common.cuh"

namespace pk {

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&f)[8]) {
    Vec<bf16>::load(p, f);
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float (&f)[8]) {
    Vec<bf16>::store(p, f);
}

constexpr int EW_THREADS = 256;

// Generic map kernel: NIN inputs of type TI, NOUT outputs of type TO. F::apply takes
// the inputs of one element and writes its outputs.
template <typename TI, typename TO, int NIN, int NOUT>
struct EwPtrs {
    const TI* in[NIN];
    TO* out[NOUT];
};

template <typename TI, typename TO, int NIN, int NOUT, typename F>
__global__ void __launch_bounds__(EW_THREADS)
ew_kernel(F f, EwPtrs<TI, TO, NIN, NOUT> p, int64_t nvec, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * EW_THREADS;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * EW_THREADS + threadIdx.x;
    for (int64_t i = tid; i < nvec; i += stride) {
        float in[NIN][8], out[NOUT][8];
#pragma unroll
        for (int k = 0; k < NIN; ++k) load8<TI>(p.in[k] + i * 8, in[k]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float a[NIN], o[NOUT];
#pragma unroll
            for (int k = 0; k < NIN; ++k) a[k] = in[k][e];
            f.apply(a, o);
#pragma unroll
            for (int k = 0; k < NOUT; ++k) out[k][e] = o[k];
        }
#pragma unroll
        for (int k = 0; k < NOUT; ++k) store8<TO>(p.out[k] + i * 8, out[k]);
    }
    for (int64_t i = nvec * 8 + tid; i < n; i += stride) {
        float a[NIN], o[NOUT];
#pragma unroll
        for (int k = 0; k < NIN; ++k) a[k] = to_f32(p.in[k][i]);
        f.apply(a, o);
#pragma unroll
        for (int k = 0; k < NOUT; ++k) p.out[k][i] = from_f32<TO>(o[k]);
    }
}

template <typename TI, typename TO, int NIN, int NOUT, typename F>
int launch_ew(cudaStream_t st, F f, EwPtrs<TI, TO, NIN, NOUT> p, int64_t n) {
    if (n <= 0) return PK_OK;
    bool al = true;
    for (int k = 0; k < NIN; ++k) al = al && aligned16(p.in[k]);
    for (int k = 0; k < NOUT; ++k) al = al && aligned16(p.out[k]);
    const int64_t nvec = al ? n / 8 : 0;
    const int64_t work = nvec + (n - nvec * 8);
    int64_t blocks = (work + EW_THREADS - 1) / EW_THREADS;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    ew_kernel<TI, TO, NIN, NOUT, F><<<static_cast<unsigned>(blocks), EW_THREADS, 0, st>>>(f, p, nvec, n);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

// ---- functors ---------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

struct SiluFwd {
    __device__ void apply(const float (&a)[1], float (&o)[1]) const { o[0] = a[0] / (1.0f + expf(-a[0])); }
};
struct SiluBwd {  // in: dy, x
    __device__ void apply(const float (&a)[2], float (&o)[1]) const {
        const float v = a[1], s = sigmoidf_(v);
        o[0] = a[0] * (s * (1.0f + v * (1.0f - s)));
    }
};
struct SwigluFwd {  // in: g, u
    __device__ void apply(const float (&a)[2], float (&o)[1]) const {
        o[0] = (a[0] / (1.0f + expf(-a[0]))) * a[1];
    }
};
struct SwigluBwd {  // in: dy, g, u -> dg, du
    __device__ void apply(const float (&a)[3], float (&o)[2]) const {
        const float dy = a[0], g = a[1], u = a[2];
        const float s = sigmoidf_(g);
        const float ds = dy * u;  // gradient reaching silu(g)
        o[0] = ds * (s * (1.0f + g * (1.0f - s)));
        o[1] = dy * (g / (1.0f + expf(-g)));
    }
};
constexpr float kGeluK = 0.7978845608028654f;
struct GeluFwd {
    __device__ void apply(const float (&a)[1], float (&o)[1]) const {
        const float v = a[0];
        const float cdf = 0.5f * (1.0f + tanhf(kGeluK * (v + 0.044715f * v * v * v)));
        o[0] = v * cdf;
    }
};
struct GeluBwd {  // in: dy, x
    __device__ void apply(const float (&a)[2], float (&o)[1]) const {
        const float v = a[1];
        const float u = kGeluK * (v + 0.044715f * v * v * v);
        const float t = tanhf(u);
        const float cdf = 0.5f * (1.0f + t);
        const float pdf = 0.5f * (1.0f - t * t) * kGeluK * (1.0f + 0.134145f * v * v);
        o[0] = a[0] * (cdf + v * pdf);
    }
};
struct ReluFwd {
    __device__ void apply(const float (&a)[1], float (&o)[1]) const { o[0] = fmaxf(0.0f, a[0]); }
};
struct ReluBwd {  // in: dy, x
    __device__ void apply(const float (&a)[2], float (&o)[1]) const { o[0] = a[1] > 0.0f ? a[0] : 0.0f; }
};
struct BinaryOp {
    int op;
    __device__ void apply(const float (&a)[2], float (&o)[1]) const {
        o[0] = op == 0 ? a[0] + a[1] : (op == 1 ? a[0] - a[1] : a[0] * a[1]);
    }
};
struct ScaleOp {
    float alpha;
    __device__ void apply(const float (&a)[1], float (&o)[1]) const { o[0] = a[0] * alpha; }
};
struct CastOp {
    __device__ void apply(const float (&a)[1], float (&o)[1]) const { o[0] = a[0]; }
};

template <typename F>
int unary(void* stream, int dtype, const void* x, void* y, int64_t n, F f) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(n == 0 || (x && y), "null pointer");
    if (dtype == PK_F32) {
        EwPtrs<float, float, 1, 1> p{{static_cast<const float*>(x)}, {static_cast<float*>(y)}};
        return launch_ew(as_stream(stream), f, p, n);
    }
    EwPtrs<bf16, bf16, 1, 1> p{{static_cast<const bf16*>(x)}, {static_cast<bf16*>(y)}};
    return launch_ew(as_stream(stream), f, p, n);
}
template <typename F>
int binary(void* stream, int dtype, const void* a, const void* b, void* y, int64_t n, F f) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(n == 0 || (a && b && y), "null pointer");
    if (dtype == PK_F32) {
        EwPtrs<float, float, 2, 1> p{{static_cast<const float*>(a), static_cast<const float*>(b)},
                                     {static_cast<float*>(y)}};
        return launch_ew(as_stream(stream), f, p, n);
    }
    EwPtrs<bf16, bf16, 2, 1> p{{static_cast<const bf16*>(a), static_cast<const bf16*>(b)},
                               {static_cast<bf16*>(y)}};
    return launch_ew(as_stream(stream), f, p, n);
}

// ---- axpy with independent dtypes ---------------------------------------------
template <typename TY, typename TX>
__global__ void __launch_bounds__(EW_THREADS)
axpy_kernel(TY* y, const TX* x, float alpha, int64_t nvec, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * EW_THREADS;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * EW_THREADS + threadIdx.x;
    for (int64_t i = tid; i < nvec; i += stride) {
        float a[8], b[8];
        load8<TY>(y + i * 8, a);
        load8<TX>(x + i * 8, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] + alpha * b[e];
        store8<TY>(y + i * 8, a);
    }
    for (int64_t i = nvec * 8 + tid; i < n; i += stride)
        y[i] = from_f32<TY>(to_f32(y[i]) + alpha * to_f32(x[i]));
}
template <typename TY, typename TX>
int launch_axpy(cudaStream_t st, TY* y, const TX* x, float alpha, int64_t n) {
    if (n <= 0) return PK_OK;
    const int64_t nvec = (aligned16(y) && aligned16(x)) ? n / 8 : 0;
    const int64_t work = nvec + (n - nvec * 8);
    int64_t blocks = (work + EW_THREADS - 1) / EW_THREADS;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    axpy_kernel<TY, TX><<<static_cast<unsigned>(blocks), EW_THREADS, 0, st>>>(y, x, alpha, nvec, n);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

// ---- bias add: y[r,c] = x[r,c] + b[c] ---------------------------------------------
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
add_bias_kernel(const T* x, const float* b, T* y, int64_t R, int64_t C, bool vec) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * EW_THREADS;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * EW_THREADS + threadIdx.x;
    if (vec) {
        const int64_t cv = C / 8, nvec = R * cv;
        for (int64_t i = tid; i < nvec; i += stride) {
            const int64_t c0 = (i % cv) * 8;
            float a[8], bb[8];
            load8<T>(x + i * 8, a);
            load8<float>(b + c0, bb);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] += bb[e];
            store8<T>(y + i * 8, a);
        }
    } else {
        const int64_t n = R * C;
        for (int64_t i = tid; i < n; i += stride) y[i] = from_f32<T>(to_f32(x[i]) + b[i % C]);
    }
}

// ---- column sums, two deterministic stages ---------------------------------------------
// Stage 1: a block owns a group of columns (COLSUM_THREADS x 16 bytes of a row) and the rows
// b, b+G, b+2G, ... of stripe b; a thread keeps the sums of its 16 bytes of columns in
// registers and has four rows in flight. partial[b, c] is the stripe's sum of column c.
// Stage 2: out[c] += sum_b partial[b, c], four interleaved running sums combined in a fixed order.
// (The previous form read one element per thread and row: 63 us for 16384 x 3072 bf16, a
// tenth of a GPT-2 step went into bias gradients.)
constexpr int COLSUM_THREADS = 128;
struct ColsumGrid {
    int col_groups;   // gridDim.y
    int stripes;      // gridDim.x = G
};
inline ColsumGrid colsum_grid(int64_t R, int64_t C, int per_thread) {
    ColsumGrid g;
    const int64_t cols_per_block = static_cast<int64_t>(COLSUM_THREADS) * per_thread;
    g.col_groups = static_cast<int>((C + cols_per_block - 1) / cols_per_block);
    int64_t st = (static_cast<int64_t>(sm_count()) * 4 + g.col_groups - 1) / g.col_groups;
    if (st > R) st = R;
    if (st < 1) st = 1;
    g.stripes = static_cast<int>(st);
    return g;
}
// the scratch is sized for the larger of the two layouts (scalar fallback: one column per thread)
inline int colsum_stripes_max(int64_t R, int64_t C) {
    const int a = colsum_grid(R, C, 8).stripes, b = colsum_grid(R, C, 1).stripes;
    return a > b ? a : b;
}
template <typename T, int N>
__device__ __forceinline__ void colsum_load(const T* p, float (&v)[N]) {
    if constexpr (N == 1) v[0] = to_f32(p[0]);
    else Vec<T>::load(p, v);
}
template <typename T, int N>   // N columns (16 bytes) per thread when the rows are 16-byte aligned, else 1
__global__ void __launch_bounds__(COLSUM_THREADS)
colsum_stage1(const T* __restrict__ x, float* __restrict__ partial, int64_t R, int64_t C) {
    const int64_t c0 = (static_cast<int64_t>(blockIdx.y) * COLSUM_THREADS + threadIdx.x) * N;
    if (c0 >= C) return;
    float acc[N];
#pragma unroll
    for (int e = 0; e < N; ++e) acc[e] = 0.0f;
    const int64_t G = gridDim.x;
    int64_t r = blockIdx.x;
    for (; r + 3 * G < R; r += 4 * G) {   // four rows in flight, added in row order
        float v[4][N];
#pragma unroll
        for (int k = 0; k < 4; ++k) colsum_load<T, N>(x + (r + k * G) * C + c0, v[k]);
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int e = 0; e < N; ++e) acc[e] += v[k][e];
    }
    for (; r < R; r += G) {
        float v[N];
        colsum_load<T, N>(x + r * C + c0, v);
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] += v[e];
    }
#pragma unroll
    for (int e = 0; e < N; ++e) partial[static_cast<int64_t>(blockIdx.x) * C + c0 + e] = acc[e];
}
__global__ void __launch_bounds__(256)
colsum_stage2(const float* __restrict__ partial, float* out, int nparts, int64_t C) {
    const int64_t c = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (c >= C) return;
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    int b = 0;
    for (; b + 3 < nparts; b += 4) {
        a0 += partial[static_cast<int64_t>(b) * C + c];
        a1 += partial[static_cast<int64_t>(b + 1) * C + c];
        a2 += partial[static_cast<int64_t>(b + 2) * C + c];
        a3 += partial[static_cast<int64_t>(b + 3) * C + c];
    }
    for (; b < nparts; ++b) a0 += partial[static_cast<int64_t>(b) * C + c];
    out[c] += (a0 + a1) + (a2 + a3);
}

// ---- column-range copy -----------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
copy_cols_kernel(const T* src, int64_t lds, int64_t sc0, T* dst, int64_t ldd, int64_t dc0,
                 int64_t R, int64_t nc, bool acc, bool vec) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * EW_THREADS;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * EW_THREADS + threadIdx.x;
    if (vec) {
        constexpr int N = Vec<T>::N;
        const int64_t cv = nc / N, nvec = R * cv;
        for (int64_t i = tid; i < nvec; i += stride) {
            const int64_t r = i / cv, c = (i % cv) * N;
            float a[N];
            Vec<T>::load(src + r * lds + sc0 + c, a);
            if (acc) {
                float d[N];
                Vec<T>::load(dst + r * ldd + dc0 + c, d);
#pragma unroll
                for (int e = 0; e < N; ++e) a[e] += d[e];
            }
            Vec<T>::store(dst + r * ldd + dc0 + c, a);
        }
    } else {
        const int64_t n = R * nc;
        for (int64_t i = tid; i < n; i += stride) {
            const int64_t r = i / nc, c = i % nc;
            float a = to_f32(src[r * lds + sc0 + c]);
            if (acc) a += to_f32(dst[r * ldd + dc0 + c]);
            dst[r * ldd + dc0 + c] = from_f32<T>(a);
        }
    }
}

// ---- transpose through a padded shared tile ---------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* x, T* y, int64_t R, int64_t C) {
    __shared__ T tile[32][33];
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32, r0 = static_cast<int64_t>(blockIdx.y) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int j = ty; j < 32; j += 8) {
        const int64_t r = r0 + j, c = c0 + tx;
        if (r < R && c < C) tile[j][tx] = x[r * C + c];
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int64_t c = c0 + j, r = r0 + tx;  // output row = input column
        if (c < C && r < R) y[c * R + r] = tile[tx][j];
    }
}

template <typename T>
int grid_for(int64_t work) {
    int64_t blocks = (work + EW_THREADS - 1) / EW_THREADS;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace pk

using namespace pk;

extern "C" {

int pk_swiglu_fwd(void* stream, int dtype, const void* g, const void* u, void* y, int64_t n) {
    return binary(stream, dtype, g, u, y, n, SwigluFwd{});
}
int pk_swiglu_bwd(void* stream, int dtype, const void* dy, const void* g, const void* u, void* dg,
                  void* du, int64_t n) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(n == 0 || (dy && g && u && dg && du), "null pointer");
    if (dtype == PK_F32) {
        EwPtrs<float, float, 3, 2> p{{static_cast<const float*>(dy), static_cast<const float*>(g),
                                      static_cast<const float*>(u)},
                                     {static_cast<float*>(dg), static_cast<float*>(du)}};
        return launch_ew(as_stream(stream), SwigluBwd{}, p, n);
    }
    EwPtrs<bf16, bf16, 3, 2> p{{static_cast<const bf16*>(dy), static_cast<const bf16*>(g),
                                static_cast<const bf16*>(u)},
                               {static_cast<bf16*>(dg), static_cast<bf16*>(du)}};
    return launch_ew(as_stream(stream), SwigluBwd{}, p, n);
}
int pk_silu_fwd(void* stream, int dtype, const void* x, void* y, int64_t n) {
    return unary(stream, dtype, x, y, n, SiluFwd{});
}
int pk_silu_bwd(void* stream, int dtype, const void* dy, const void* x, void* dx, int64_t n) {
    return binary(stream, dtype, dy, x, dx, n, SiluBwd{});
}
int pk_gelu_fwd(void* stream, int dtype, const void* x, void* y, int64_t n) {
    return unary(stream, dtype, x, y, n, GeluFwd{});
}
int pk_gelu_bwd(void* stream, int dtype, const void* dy, const void* x, void* dx, int64_t n) {
    return binary(stream, dtype, dy, x, dx, n, GeluBwd{});
}
int pk_relu_fwd(void* stream, int dtype, const void* x, void* y, int64_t n) {
    return unary(stream, dtype, x, y, n, ReluFwd{});
}
int pk_relu_bwd(void* stream, int dtype, const void* dy, const void* x, void* dx, int64_t n) {
    return binary(stream, dtype, dy, x, dx, n, ReluBwd{});
}
int pk_binary(void* stream, int dtype, int op, const void* a, const void* b, void* y, int64_t n) {
    PK_REQUIRE(op >= 0 && op <= 2, "op must be 0 (add), 1 (sub) or 2 (mul)");
    return binary(stream, dtype, a, b, y, n, BinaryOp{op});
}
int pk_scale(void* stream, int dtype, const void* x, float alpha, void* y, int64_t n) {
    return unary(stream, dtype, x, y, n, ScaleOp{alpha});
}
int pk_axpy(void* stream, int y_dtype, void* y, int x_dtype, const void* x, float alpha, int64_t n) {
    PK_REQUIRE(valid_dtype(y_dtype) && valid_dtype(x_dtype), "bad dtype");
    PK_REQUIRE(n == 0 || (x && y), "null pointer");
    cudaStream_t st = as_stream(stream);
    if (y_dtype == PK_F32 && x_dtype == PK_F32)
        return launch_axpy(st, static_cast<float*>(y), static_cast<const float*>(x), alpha, n);
    if (y_dtype == PK_F32)
        return launch_axpy(st, static_cast<float*>(y), static_cast<const bf16*>(x), alpha, n);
    if (x_dtype == PK_F32)
        return launch_axpy(st, static_cast<bf16*>(y), static_cast<const float*>(x), alpha, n);
    return launch_axpy(st, static_cast<bf16*>(y), static_cast<const bf16*>(x), alpha, n);
}
int pk_cast(void* stream, int src_dtype, const void* src, int dst_dtype, void* dst, int64_t n) {
    PK_REQUIRE(valid_dtype(src_dtype) && valid_dtype(dst_dtype), "bad dtype");
    PK_REQUIRE(n == 0 || (src && dst), "null pointer");
    cudaStream_t st = as_stream(stream);
    if (src_dtype == dst_dtype) {
        if (src != dst) PK_CHECK_CUDA(cudaMemcpyAsync(dst, src, n * dtype_size(src_dtype), cudaMemcpyDeviceToDevice, st));
        return PK_OK;
    }
    if (src_dtype == PK_F32) {
        EwPtrs<float, bf16, 1, 1> p{{static_cast<const float*>(src)}, {static_cast<bf16*>(dst)}};
        return launch_ew(st, CastOp{}, p, n);
    }
    EwPtrs<bf16, float, 1, 1> p{{static_cast<const bf16*>(src)}, {static_cast<float*>(dst)}};
    return launch_ew(st, CastOp{}, p, n);
}
int pk_add_bias(void* stream, int dtype, const void* x, const float* b, void* y, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C >= 0, "negative shape");
    if (R == 0 || C == 0) return PK_OK;
    PK_REQUIRE(x && b && y, "null pointer");
    const bool vec = (C % 8 == 0) && aligned16(x) && aligned16(y) && aligned16(b);
    const int64_t work = vec ? R * C / 8 : R * C;
    const int blocks = grid_for<float>(work);
    if (dtype == PK_F32)
        add_bias_kernel<float><<<blocks, EW_THREADS, 0, as_stream(stream)>>>(
            static_cast<const float*>(x), b, static_cast<float*>(y), R, C, vec);
    else
        add_bias_kernel<bf16><<<blocks, EW_THREADS, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(x), b, static_cast<bf16*>(y), R, C, vec);
    PK_LAUNCH_CHECK();
    return PK_OK;
}
size_t pk_colsum_scratch_bytes(int64_t R, int64_t C) {
    if (R <= 0 || C <= 0) return 0;
    return static_cast<size_t>(colsum_stripes_max(R, C)) * static_cast<size_t>(C) * sizeof(float);
}
int pk_colsum(void* stream, int dtype, const void* x, float* out, void* scratch, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    if (R <= 0 || C <= 0) return PK_OK;
    PK_REQUIRE(x && out && scratch, "null pointer");
    float* partial = static_cast<float*>(scratch);
    cudaStream_t st = as_stream(stream);
    constexpr int NB = Vec<bf16>::N, NF = Vec<float>::N;
    const bool vec = aligned16(x) && C % (dtype == PK_F32 ? NF : NB) == 0;
    const ColsumGrid cg = colsum_grid(R, C, vec ? (dtype == PK_F32 ? NF : NB) : 1);
    const dim3 grid(static_cast<unsigned>(cg.stripes), static_cast<unsigned>(cg.col_groups));
    const int g = cg.stripes;
    if (dtype == PK_F32) {
        if (vec) colsum_stage1<float, NF><<<grid, COLSUM_THREADS, 0, st>>>(static_cast<const float*>(x), partial, R, C);
        else colsum_stage1<float, 1><<<grid, COLSUM_THREADS, 0, st>>>(static_cast<const float*>(x), partial, R, C);
    } else {
        if (vec) colsum_stage1<bf16, NB><<<grid, COLSUM_THREADS, 0, st>>>(static_cast<const bf16*>(x), partial, R, C);
        else colsum_stage1<bf16, 1><<<grid, COLSUM_THREADS, 0, st>>>(static_cast<const bf16*>(x), partial, R, C);
    }
    PK_LAUNCH_CHECK();
    colsum_stage2<<<static_cast<unsigned>((C + 255) / 256), 256, 0, as_stream(stream)>>>(partial, out, g, C);
    PK_LAUNCH_CHECK();
    return PK_OK;
}
int pk_copy_cols(void* stream, int dtype, const void* src, int64_t lds, int64_t scol0, void* dst,
                 int64_t ldd, int64_t dcol0, int64_t R, int64_t ncols, int accumulate) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && ncols >= 0 && scol0 >= 0 && dcol0 >= 0, "negative shape");
    if (R == 0 || ncols == 0) return PK_OK;
    PK_REQUIRE(src && dst, "null pointer");
    PK_REQUIRE(scol0 + ncols <= lds && dcol0 + ncols <= ldd, "column range exceeds row stride");
    const int nv = dtype == PK_F32 ? 4 : 8;
    const size_t es = dtype_size(dtype);
    const bool vec = ncols % nv == 0 && lds % nv == 0 && ldd % nv == 0 && scol0 % nv == 0 &&
                     dcol0 % nv == 0 && aligned16(src) && aligned16(dst);
    (void)es;
    const int64_t work = vec ? R * ncols / nv : R * ncols;
    const int blocks = grid_for<float>(work);
    if (dtype == PK_F32)
        copy_cols_kernel<float><<<blocks, EW_THREADS, 0, as_stream(stream)>>>(
            static_cast<const float*>(src), lds, scol0, static_cast<float*>(dst), ldd, dcol0, R, ncols,
            accumulate != 0, vec);
    else
        copy_cols_kernel<bf16><<<blocks, EW_THREADS, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(src), lds, scol0, static_cast<bf16*>(dst), ldd, dcol0, R, ncols,
            accumulate != 0, vec);
    PK_LAUNCH_CHECK();
    return PK_OK;
}
int pk_transpose(void* stream, int dtype, const void* x, void* y, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    if (R <= 0 || C <= 0) return PK_OK;
    PK_REQUIRE(x && y, "null pointer");
    dim3 grid(static_cast<unsigned>((C + 31) / 32), static_cast<unsigned>((R + 31) / 32));
    PK_REQUIRE(grid.y <= 65535u, "too many rows for one transpose launch");
    if (dtype == PK_F32)
        transpose_kernel<float><<<grid, 256, 0, as_stream(stream)>>>(static_cast<const float*>(x), static_cast<float*>(y), R, C);
    else
        transpose_kernel<bf16><<<grid, 256, 0, as_stream(stream)>>>(static_cast<const bf16*>(x), static_cast<bf16*>(y), R, C);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // extern "C"
