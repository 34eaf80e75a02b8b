// RMSNorm / LayerNorm forward and backward, and the rotary-embedding rotation.
//
// Row kernels come in two shapes:
//   * "warp" kernels: one warp owns a row, the row lives in registers between
//     the reduction and the normalisation (one HBM read per element), 128-bit
//     accesses, warp-shuffle reductions. Used when C is a multiple of the vector
//     width and fits 32 lanes x 8 vectors.
//   * "generic" kernels: one block per row, scalar accesses, any C.
// Parameter gradients (dw, dgamma, dbeta) are column sums over all rows. They are
// produced in two fixed-order stages -- per-block partial sums in scratch, then
// one pass over the partials -- so the result does not depend on scheduling.
//
// Formulas: ops::rmsnorm (src/ops.cpp:426-479), ops::layernorm (src/ops.cpp:248-327),
// ops::apply_rope (src/ops.cpp:481-537) of the reference.
#include "pk_common.cuh"

namespace pk {

constexpr int NORM_WPB = 4;               // warps per block in the warp kernels
constexpr int NORM_THREADS = NORM_WPB * 32;
constexpr int NORM_MAX_VPL = 8;           // vectors per lane

template <typename T>
inline int norm_vpl(int64_t C, const void* a, const void* b, const void* c) {
    constexpr int N = Vec<T>::N;
    if (C % N != 0) return 0;
    if (!aligned16(a) || (b && !aligned16(b)) || (c && !aligned16(c))) return 0;
    const int64_t nv = C / N;
    for (int v = 1; v <= NORM_MAX_VPL; v *= 2)
        if (nv <= 32 * v) return v;
    return 0;
}

inline int norm_partial_blocks() { return sm_count() * 4; }

// Loads the fp32 parameter vector segment matching one storage vector.
template <int N>
__device__ __forceinline__ void load_param(const float* p, float (&f)[N]) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + i);
        f[i] = v.x; f[i + 1] = v.y; f[i + 2] = v.z; f[i + 3] = v.w;
    }
}

// ---------------------------------------------------------------- forward, warp per row
template <typename T, int VPL, bool LN>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_warp(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
              T* __restrict__ y, float* __restrict__ stat0, float* __restrict__ stat1,
              int64_t R, int64_t C, float eps) {
    constexpr int N = Vec<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * NORM_WPB + warp;
    if (row >= R) return;
    const T* xr = x + row * C;
    float v[VPL][N];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int64_t col = (static_cast<int64_t>(i) * 32 + lane) * N;
        if (col < C) {
            Vec<T>::load(xr + col, v[i]);
        } else {
#pragma unroll
            for (int e = 0; e < N; ++e) v[i][e] = 0.0f;
        }
    }
    const float inv_c = 1.0f / static_cast<float>(C);
    float mu = 0.0f, rs;
    if (LN) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VPL; ++i)
#pragma unroll
            for (int e = 0; e < N; ++e) s += v[i][e];
        mu = warp_sum(s) / static_cast<float>(C);
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int64_t col = (static_cast<int64_t>(i) * 32 + lane) * N;
            if (col < C) {
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float d = v[i][e] - mu;
                    q += d * d;
                }
            }
        }
        const float var = warp_sum(q) / static_cast<float>(C);
        rs = 1.0f / sqrtf(var + eps);
        if (lane == 0) {
            stat0[row] = mu;
            stat1[row] = rs;
        }
    } else {
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < VPL; ++i)
#pragma unroll
            for (int e = 0; e < N; ++e) q += v[i][e] * v[i][e];
        const float ms = warp_sum(q) / static_cast<float>(C);
        rs = 1.0f / sqrtf(ms + eps);
        if (lane == 0) stat0[row] = rs;
    }
    (void)inv_c;
    T* yr = y + row * C;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int64_t col = (static_cast<int64_t>(i) * 32 + lane) * N;
        if (col < C) {
            float ww[N], o[N];
            load_param<N>(w + col, ww);
            if (LN) {
                float bb[N];
                load_param<N>(b + col, bb);
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = ww[e] * ((v[i][e] - mu) * rs) + bb[e];
            } else {
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = v[i][e] * rs * ww[e];
            }
            Vec<T>::store(yr + col, o);
        }
    }
}

// ---------------------------------------------------------------- forward, generic
template <typename T, bool LN>
__global__ void __launch_bounds__(256)
norm_fwd_generic(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                 T* __restrict__ y, float* __restrict__ stat0, float* __restrict__ stat1,
                 int64_t R, int64_t C, float eps) {
    __shared__ float red[32];
    for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
        const T* xr = x + row * C;
        float mu = 0.0f, rs;
        if (LN) {
            float s = 0.0f;
            for (int64_t c = threadIdx.x; c < C; c += blockDim.x) s += to_f32(xr[c]);
            mu = block_sum(s, red) / static_cast<float>(C);
            float q = 0.0f;
            for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
                const float d = to_f32(xr[c]) - mu;
                q += d * d;
            }
            rs = 1.0f / sqrtf(block_sum(q, red) / static_cast<float>(C) + eps);
            if (threadIdx.x == 0) {
                stat0[row] = mu;
                stat1[row] = rs;
            }
        } else {
            float q = 0.0f;
            for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
                const float t = to_f32(xr[c]);
                q += t * t;
            }
            rs = 1.0f / sqrtf(block_sum(q, red) / static_cast<float>(C) + eps);
            if (threadIdx.x == 0) stat0[row] = rs;
        }
        T* yr = y + row * C;
        for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
            const float t = to_f32(xr[c]);
            yr[c] = from_f32<T>(LN ? w[c] * ((t - mu) * rs) + b[c] : t * rs * w[c]);
        }
    }
}

// ---------------------------------------------------------------- backward, warp per row
// A warp keeps its row packed as loaded (x and dy, 16 bytes per vector) and converts it twice:
// once for the row sums and the parameter gradients, once for dx. A lane sees the same columns
// in every row, so its share of dw / dgamma / dbeta accumulates in registers over the warp's
// rows (row order ascending) when that fits (ACC_REG), else in shared memory; at the end the
// warps of a block are combined in warp order through shared memory:
// NORM_WPB x (LN ? 2 : 1) x SLOTS floats, laid out [warp][which][vec-slot][element][lane].
template <typename T, int VPL, bool LN>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_warp(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ w,
              const float* __restrict__ stat0, const float* __restrict__ stat1,
              T* __restrict__ dx, float* __restrict__ partial, int want_dparam,
              int64_t R, int64_t C) {
    constexpr int N = Vec<T>::N;
    constexpr int SLOTS = VPL * N * 32;  // >= C
    constexpr bool ACC_REG = (LN ? 2 : 1) * VPL * N <= 64;
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* acc_w = smem + static_cast<size_t>(warp) * (LN ? 2 : 1) * SLOTS;
    float* acc_b = acc_w + SLOTS;  // only when LN
    float rw[ACC_REG ? VPL : 1][N], rb[ACC_REG && LN ? VPL : 1][N];
    if (ACC_REG) {
#pragma unroll
        for (int i = 0; i < (ACC_REG ? VPL : 1); ++i)
#pragma unroll
            for (int e = 0; e < N; ++e) {
                rw[i][e] = 0.0f;
                if (LN) rb[i][e] = 0.0f;
            }
    } else if (want_dparam) {
        for (int i = lane; i < (LN ? 2 : 1) * SLOTS; i += 32) acc_w[i] = 0.0f;
        __syncwarp();
    }
    const int64_t total_warps = static_cast<int64_t>(gridDim.x) * NORM_WPB;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * NORM_WPB + warp; row < R; row += total_warps) {
        const T* xr = x + row * C;
        const T* gr = dy + row * C;
        uint4 xq[VPL], gq[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int64_t col = (static_cast<int64_t>(i) * 32 + lane) * N;
            if (col < C) {
                xq[i] = Vec<T>::load_raw(xr + col);
                gq[i] = Vec<T>::load_raw(gr + col);
            } else {
                xq[i] = make_uint4(0u, 0u, 0u, 0u);
                gq[i] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        const float rs = LN ? stat1[row] : stat0[row];
        const float mu = LN ? stat0[row] : 0.0f;
        // gw = dy * w is the gradient reaching the normalised value; xh = xhat (LN) or x
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int64_t col = (static_cast<int64_t>(i) * 32 + lane) * N;
            if (col < C) {
                float ww[N], xv[N], gv[N];
                load_param<N>(w + col, ww);
                Vec<T>::unpack(xq[i], xv);
                Vec<T>::unpack(gq[i], gv);
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float g = gv[e];
                    const float xh = LN ? (xv[e] - mu) * rs : xv[e];
                    if (want_dparam) {
                        if (ACC_REG) {
                            if (LN) {
                                rw[ACC_REG ? i : 0][e] += g * xh;
                                rb[ACC_REG && LN ? i : 0][e] += g;
                            } else {
                                rw[ACC_REG ? i : 0][e] += g * xh * rs;
                            }
                        } else {
                            const int slot = (i * N + e) * 32 + lane;
                            if (LN) {
                                acc_w[slot] += g * xh;
                                acc_b[slot] += g;
                            } else {
                                acc_w[slot] += g * xh * rs;
                            }
                        }
                    }
                    const float gw = g * ww[e];
                    if (LN) s1 += gw;
                    s2 += gw * xh;
                }
            }
        }
        if (dx != nullptr) {
            s2 = warp_sum(s2);
            if (LN) s1 = warp_sum(s1);
            const float inv_c = 1.0f / static_cast<float>(C);
            const float m1 = s1 * inv_c, m2 = s2 * inv_c;
            const float rr = rs * rs;
            T* dr = dx + row * C;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int64_t col = (static_cast<int64_t>(i) * 32 + lane) * N;
                if (col < C) {
                    float ww[N], xv[N], gv[N], o[N];
                    load_param<N>(w + col, ww);
                    Vec<T>::unpack(xq[i], xv);
                    Vec<T>::unpack(gq[i], gv);
#pragma unroll
                    for (int e = 0; e < N; ++e) {
                        const float xh = LN ? (xv[e] - mu) * rs : xv[e];
                        const float gw = gv[e] * ww[e];
                        if (LN) o[e] = rs * (gw - m1 - xh * m2);
                        else o[e] = rs * (gw - xh * rr * s2 * inv_c);
                    }
                    Vec<T>::store(dr + col, o);
                }
            }
        }
    }
    if (!want_dparam) return;
    if (ACC_REG) {
#pragma unroll
        for (int i = 0; i < (ACC_REG ? VPL : 1); ++i)
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const int slot = (i * N + e) * 32 + lane;
                acc_w[slot] = rw[i][e];
                if (LN) acc_b[slot] = rb[ACC_REG && LN ? i : 0][e];
            }
    }
    __syncthreads();
    // Combine the warps of this block in warp order and write the block's partial row(s).
    float* pw = partial + static_cast<size_t>(blockIdx.x) * (LN ? 2 : 1) * C;
    for (int64_t c = threadIdx.x; c < C; c += NORM_THREADS) {
        const int64_t vec = c / N;
        const int e = static_cast<int>(c % N);
        const int i = static_cast<int>(vec / 32), ln = static_cast<int>(vec % 32);
        const int slot = (i * N + e) * 32 + ln;
        float a = 0.0f, bsum = 0.0f;
#pragma unroll
        for (int wv = 0; wv < NORM_WPB; ++wv) {
            const float* base = smem + static_cast<size_t>(wv) * (LN ? 2 : 1) * SLOTS;
            a += base[slot];
            if (LN) bsum += base[SLOTS + slot];
        }
        pw[c] = a;
        if (LN) pw[C + c] = bsum;
    }
}

// ---------------------------------------------------------------- backward, generic
// Block b owns rows b, b+G, ...; thread t owns columns t, t+blockDim, ... of the block's
// partial row(s), which it updates in place (read-modify-write by a single thread).
template <typename T, bool LN>
__global__ void __launch_bounds__(256)
norm_bwd_generic(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ w,
                 const float* __restrict__ stat0, const float* __restrict__ stat1,
                 T* __restrict__ dx, float* __restrict__ partial, int want_dparam,
                 int64_t R, int64_t C) {
    __shared__ float red[32];
    float* pw = partial + static_cast<size_t>(blockIdx.x) * (LN ? 2 : 1) * C;
    if (want_dparam)
        for (int64_t c = threadIdx.x; c < (LN ? 2 : 1) * C; c += blockDim.x) pw[c] = 0.0f;
    for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
        const T* xr = x + row * C;
        const T* gr = dy + row * C;
        const float rs = LN ? stat1[row] : stat0[row];
        const float mu = LN ? stat0[row] : 0.0f;
        float s1 = 0.0f, s2 = 0.0f;
        for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
            const float g = to_f32(gr[c]);
            const float xh = LN ? (to_f32(xr[c]) - mu) * rs : to_f32(xr[c]);
            if (want_dparam) {
                if (LN) {
                    pw[c] += g * xh;
                    pw[C + c] += g;
                } else {
                    pw[c] += g * xh * rs;
                }
            }
            const float gw = g * w[c];
            s1 += gw;
            s2 += gw * xh;
        }
        if (dx != nullptr) {
            s2 = block_sum(s2, red);
            if (LN) s1 = block_sum(s1, red);
            const float inv_c = 1.0f / static_cast<float>(C);
            const float m1 = s1 * inv_c, m2 = s2 * inv_c, rr = rs * rs;
            T* dr = dx + row * C;
            for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
                const float gw = to_f32(gr[c]) * w[c];
                const float xh = LN ? (to_f32(xr[c]) - mu) * rs : to_f32(xr[c]);
                dr[c] = from_f32<T>(LN ? rs * (gw - m1 - xh * m2) : rs * (gw - xh * rr * s2 * inv_c));
            }
        }
    }
}

// out[c] += sum over blocks of partial[b, which, c]. A block of 8 warps owns 32 columns; warp j
// adds blocks j, j+8, ... in ascending order with four independent running sums (blocks
// j+8(4i+k) go to sum k), then the four sums and the eight warps are combined in a fixed
// order, so the result depends only on nblocks.
__global__ void __launch_bounds__(256)
norm_dparam_stage2(const float* __restrict__ partial, int nblocks, int nwhich, int which,
                   float* __restrict__ out, int64_t C) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + lane;
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    if (c < C) {
        const size_t pitch = static_cast<size_t>(nwhich) * C;
        const float* p = partial + static_cast<size_t>(which) * C + c;
        int b = warp;
        for (; b + 24 < nblocks; b += 32) {
            a0 += p[static_cast<size_t>(b) * pitch];
            a1 += p[static_cast<size_t>(b + 8) * pitch];
            a2 += p[static_cast<size_t>(b + 16) * pitch];
            a3 += p[static_cast<size_t>(b + 24) * pitch];
        }
        if (b < nblocks) a0 += p[static_cast<size_t>(b) * pitch];
        if (b + 8 < nblocks) a1 += p[static_cast<size_t>(b + 8) * pitch];
        if (b + 16 < nblocks) a2 += p[static_cast<size_t>(b + 16) * pitch];
    }
    part[warp][lane] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (warp == 0 && c < C) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += part[j][lane];
        out[c] += acc;
    }
}

template <typename T, bool LN>
int norm_fwd_dispatch(cudaStream_t st, const T* x, const float* w, const float* b, T* y, float* s0,
                      float* s1, int64_t R, int64_t C, float eps) {
    int vpl = norm_vpl<T>(C, x, y, nullptr);
    if (!aligned16(w) || (LN && !aligned16(b))) vpl = 0;
    const unsigned grid = static_cast<unsigned>((R + NORM_WPB - 1) / NORM_WPB);
    switch (vpl) {
        case 1: norm_fwd_warp<T, 1, LN><<<grid, NORM_THREADS, 0, st>>>(x, w, b, y, s0, s1, R, C, eps); break;
        case 2: norm_fwd_warp<T, 2, LN><<<grid, NORM_THREADS, 0, st>>>(x, w, b, y, s0, s1, R, C, eps); break;
        case 4: norm_fwd_warp<T, 4, LN><<<grid, NORM_THREADS, 0, st>>>(x, w, b, y, s0, s1, R, C, eps); break;
        case 8: norm_fwd_warp<T, 8, LN><<<grid, NORM_THREADS, 0, st>>>(x, w, b, y, s0, s1, R, C, eps); break;
        default: {
            int64_t g = static_cast<int64_t>(sm_count()) * 8;
            if (g > R) g = R;
            norm_fwd_generic<T, LN><<<static_cast<unsigned>(g), 256, 0, st>>>(x, w, b, y, s0, s1, R, C, eps);
        }
    }
    PK_LAUNCH_CHECK();
    return PK_OK;
}

template <typename T, int VPL, bool LN>
int launch_bwd_warp(cudaStream_t st, const T* dy, const T* x, const float* w, const float* s0,
                    const float* s1, T* dx, float* partial, int want, int64_t R, int64_t C, int grid,
                    int* grid_out) {
    const size_t smem = static_cast<size_t>(NORM_WPB) * (LN ? 2 : 1) * VPL * Vec<T>::N * 32 * sizeof(float);
    auto kern = norm_bwd_warp<T, VPL, LN>;
    if (smem > 48 * 1024)
        PK_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    // The rows are dealt out evenly over the grid, so a grid of more blocks than fit on the
    // GPU at once ends in a thin second wave: keep it to one wave of resident blocks.
    static int resident = 0;  // per instantiation; the same on every device of one machine
    if (resident == 0) {
        int per_sm = 0;
        PK_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NORM_THREADS, smem));
        resident = per_sm > 0 ? per_sm : 1;
    }
    const int64_t wave = static_cast<int64_t>(resident) * sm_count();
    if (grid > wave) grid = static_cast<int>(wave);
    *grid_out = grid;
    kern<<<grid, NORM_THREADS, smem, st>>>(dy, x, w, s0, s1, dx, partial, want, R, C);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

// dparams: out0 (dw / dgamma) and out1 (dbeta, LN only) are accumulated; either may be null.
template <typename T, bool LN>
int norm_bwd_dispatch(cudaStream_t st, const T* dy, const T* x, const float* w, const float* s0,
                      const float* s1, T* dx, float* out0, float* out1, float* partial,
                      int64_t R, int64_t C) {
    const int want = (out0 != nullptr || out1 != nullptr) ? 1 : 0;
    if (!want && dx == nullptr) return PK_OK;
    int vpl = norm_vpl<T>(C, x, dy, dx);
    if (!aligned16(w)) vpl = 0;
    int grid;
    int rc = PK_OK;
    if (vpl > 0) {
        int64_t g = norm_partial_blocks();
        const int64_t need = (R + NORM_WPB - 1) / NORM_WPB;
        if (g > need) g = need;
        grid = static_cast<int>(g);
        switch (vpl) {
            case 1: rc = launch_bwd_warp<T, 1, LN>(st, dy, x, w, s0, s1, dx, partial, want, R, C, grid, &grid); break;
            case 2: rc = launch_bwd_warp<T, 2, LN>(st, dy, x, w, s0, s1, dx, partial, want, R, C, grid, &grid); break;
            case 4: rc = launch_bwd_warp<T, 4, LN>(st, dy, x, w, s0, s1, dx, partial, want, R, C, grid, &grid); break;
            default: rc = launch_bwd_warp<T, 8, LN>(st, dy, x, w, s0, s1, dx, partial, want, R, C, grid, &grid); break;
        }
        if (rc != PK_OK) return rc;
    } else {
        int64_t g = norm_partial_blocks();
        if (g > R) g = R;
        grid = static_cast<int>(g);
        norm_bwd_generic<T, LN><<<grid, 256, 0, st>>>(dy, x, w, s0, s1, dx, partial, want, R, C);
        PK_LAUNCH_CHECK();
    }
    if (want) {
        const unsigned g2 = static_cast<unsigned>((C + 31) / 32);
        if (out0) norm_dparam_stage2<<<g2, 256, 0, st>>>(partial, grid, LN ? 2 : 1, 0, out0, C);
        if (LN && out1) norm_dparam_stage2<<<g2, 256, 0, st>>>(partial, grid, 2, 1, out1, C);
        PK_LAUNCH_CHECK();
    }
    return PK_OK;
}

// ---------------------------------------------------------------- rotary embedding
template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(T* __restrict__ x, int64_t ld, int64_t col0, int n_heads, int half, const int32_t* __restrict__ pos,
            const float* __restrict__ cs, int64_t n_pos, int64_t R, float sin_sign) {
    const int64_t per_row = static_cast<int64_t>(n_heads) * half;
    const int64_t total = R * per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t row = i / per_row;
        const int rem = static_cast<int>(i % per_row);
        const int h = rem / half, j = rem % half;
        int64_t p = pos[row];
        if (p < 0) p = 0;
        if (p >= n_pos) p = n_pos - 1;
        const float2 c = *reinterpret_cast<const float2*>(cs + (p * half + j) * 2);
        T* px = x + row * ld + col0 + static_cast<int64_t>(h) * (2 * half) + 2 * j;
        const float x0 = to_f32(px[0]), x1 = to_f32(px[1]);
        const float sn = c.y * sin_sign;
        float o0, o1;
        rope_rotate(x0, x1, c.x, sn, o0, o1);
        px[0] = from_f32<T>(o0);
        px[1] = from_f32<T>(o1);
    }
}

// bf16, 8 elements (4 rotation pairs, 16 bytes) per thread and iteration: same arithmetic per pair
// as rope_kernel, with 16-byte accesses and 32-bit index arithmetic inside a row.
__global__ void __launch_bounds__(256)
rope_vec8_kernel(bf16* __restrict__ x, int64_t ld, int64_t col0, int n_heads, int half, const int32_t* __restrict__ pos,
                 const float* __restrict__ cs, int64_t n_pos, int64_t R, float sin_sign) {
    const int vec_per_head = half / 4;                       // 4 pairs per vector
    const int vec_per_row = n_heads * vec_per_head;
    const int64_t total = R * vec_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t row = i / vec_per_row;
        const int rem = static_cast<int>(i - row * vec_per_row);
        const int h = rem / vec_per_head, j4 = (rem - h * vec_per_head) * 4;   // first pair of this vector
        int64_t p = pos[row];
        if (p < 0) p = 0;
        if (p >= n_pos) p = n_pos - 1;
        const float4* c4 = reinterpret_cast<const float4*>(cs + (p * half + j4) * 2);
        const float4 ca = c4[0], cb = c4[1];                 // (cos, sin) of pairs j4 .. j4+3
        bf16* px = x + row * ld + col0 + static_cast<int64_t>(h) * (2 * half) + 2 * j4;
        float v[8];
        Vec<bf16>::load(px, v);
        const float cc[4] = {ca.x, ca.z, cb.x, cb.z};
        const float ss[4] = {ca.y * sin_sign, ca.w * sin_sign, cb.y * sin_sign, cb.w * sin_sign};
        float o[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            rope_rotate(v[2 * e], v[2 * e + 1], cc[e], ss[e], o[2 * e], o[2 * e + 1]);
        }
        Vec<bf16>::store(px, o);
    }
}

}  // namespace pk

using namespace pk;

extern "C" {

int pk_rmsnorm_fwd(void* stream, int dtype, const void* x, const float* w, void* y, float* rinv,
                   int64_t R, int64_t C, float eps) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C > 0, "bad shape");
    if (R == 0) return PK_OK;
    PK_REQUIRE(x && w && y && rinv, "null pointer");
    if (dtype == PK_F32)
        return norm_fwd_dispatch<float, false>(as_stream(stream), static_cast<const float*>(x), w, nullptr,
                                               static_cast<float*>(y), rinv, nullptr, R, C, eps);
    return norm_fwd_dispatch<bf16, false>(as_stream(stream), static_cast<const bf16*>(x), w, nullptr,
                                          static_cast<bf16*>(y), rinv, nullptr, R, C, eps);
}

size_t pk_rmsnorm_bwd_scratch_bytes(int64_t R, int64_t C) {
    (void)R;
    return static_cast<size_t>(norm_partial_blocks()) * static_cast<size_t>(C) * sizeof(float);
}

int pk_rmsnorm_bwd(void* stream, int dtype, const void* dy, const void* x, const float* w,
                   const float* rinv, void* dx, float* dw, void* scratch, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C > 0, "bad shape");
    if (R == 0) return PK_OK;
    PK_REQUIRE(dy && x && w && rinv, "null pointer");
    PK_REQUIRE(dw == nullptr || scratch != nullptr, "dw needs scratch");
    if (dtype == PK_F32)
        return norm_bwd_dispatch<float, false>(as_stream(stream), static_cast<const float*>(dy),
                                               static_cast<const float*>(x), w, rinv, nullptr,
                                               static_cast<float*>(dx), dw, nullptr,
                                               static_cast<float*>(scratch), R, C);
    return norm_bwd_dispatch<bf16, false>(as_stream(stream), static_cast<const bf16*>(dy),
                                          static_cast<const bf16*>(x), w, rinv, nullptr,
                                          static_cast<bf16*>(dx), dw, nullptr,
                                          static_cast<float*>(scratch), R, C);
}

// ---- RMSNorm backward for callers that cannot allocate -----------------------------------
// pk_rmsnorm_bwd needs a scratch buffer for the per-block partial sums of dw, and expects the
// caller to allocate it. Some hosts cannot: a runtime that claimed the whole GPU for its own
// memory pool before loading this library has nothing left for cudaMalloc to hand out, and a
// latency-critical loop must not call cudaMalloc at all because it synchronises the device.
// For them the partial sums live in a fixed array that is part of the library image.
//
// The array below is device memory reserved by the module itself (~9.3 MiB on every GPU that
// loads the library, until the process exits). Its name is only a host-side handle: the
// device address is looked up once per device with cudaGetSymbolAddress and that pointer is
// what the kernels receive.
constexpr size_t PK_STATIC_SCRATCH_FLOATS = size_t(592) * 4096;  // 592 partial rows of up to 4096 columns
static __device__ __align__(256) float g_rmsnorm_static_scratch[PK_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int PK_MAX_DEVICES = 64;
float* g_static_scratch_ptr[PK_MAX_DEVICES] = {};  // device address per ordinal, resolved lazily
}  // namespace

int pk_rmsnorm_bwd_noalloc(void* stream, int dtype, const void* dy, const void* x, const float* w,
                           const float* rinv, void* dx, float* dw, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C > 0, "bad shape");
    // the same partial-row count pk_rmsnorm_bwd_scratch_bytes() is based on
    const size_t need = static_cast<size_t>(norm_partial_blocks()) * static_cast<size_t>(C);
    if (need > PK_STATIC_SCRATCH_FLOATS) {
        set_error("pk_rmsnorm_bwd_noalloc: %lld columns need %zu floats of scratch, the built-in buffer holds %zu "
                  "(about %zu columns on this GPU); use pk_rmsnorm_bwd with caller-provided scratch",
                  static_cast<long long>(C), need, PK_STATIC_SCRATCH_FLOATS,
                  PK_STATIC_SCRATCH_FLOATS / static_cast<size_t>(norm_partial_blocks()));
        return PK_ERR_UNSUPPORTED;
    }
    if (R == 0) return PK_OK;
    PK_REQUIRE(dy && x && w && rinv, "null pointer");
    int dev = 0;
    PK_CHECK_CUDA(cudaGetDevice(&dev));
    PK_REQUIRE(dev >= 0 && dev < PK_MAX_DEVICES, "device ordinal out of range");
    if (g_static_scratch_ptr[dev] == nullptr) {
        // First call on this device (it is the current one): resolve the symbol. This is a
        // runtime query, so make this first call outside any stream capture.
        void* p = nullptr;
        PK_CHECK_CUDA(cudaGetSymbolAddress(&p, g_rmsnorm_static_scratch));
        g_static_scratch_ptr[dev] = static_cast<float*>(p);
    }
    float* scratch = g_static_scratch_ptr[dev];
    // Nothing needs clearing: every partial row that the second stage reads is written in
    // full by the first stage of the same call, whatever an earlier call left behind.
    if (dtype == PK_F32)
        return norm_bwd_dispatch<float, false>(as_stream(stream), static_cast<const float*>(dy),
                                               static_cast<const float*>(x), w, rinv, nullptr,
                                               static_cast<float*>(dx), dw, nullptr, scratch, R, C);
    return norm_bwd_dispatch<bf16, false>(as_stream(stream), static_cast<const bf16*>(dy),
                                          static_cast<const bf16*>(x), w, rinv, nullptr,
                                          static_cast<bf16*>(dx), dw, nullptr, scratch, R, C);
}

int pk_layernorm_fwd(void* stream, int dtype, const void* x, const float* gamma, const float* beta,
                     void* y, float* mean, float* rstd, int64_t R, int64_t C, float eps) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C > 0, "bad shape");
    if (R == 0) return PK_OK;
    PK_REQUIRE(x && gamma && beta && y && mean && rstd, "null pointer");
    if (dtype == PK_F32)
        return norm_fwd_dispatch<float, true>(as_stream(stream), static_cast<const float*>(x), gamma, beta,
                                              static_cast<float*>(y), mean, rstd, R, C, eps);
    return norm_fwd_dispatch<bf16, true>(as_stream(stream), static_cast<const bf16*>(x), gamma, beta,
                                         static_cast<bf16*>(y), mean, rstd, R, C, eps);
}

size_t pk_layernorm_bwd_scratch_bytes(int64_t R, int64_t C) {
    (void)R;
    return 2 * static_cast<size_t>(norm_partial_blocks()) * static_cast<size_t>(C) * sizeof(float);
}

int pk_layernorm_bwd(void* stream, int dtype, const void* dy, const void* x, const float* gamma,
                     const float* mean, const float* rstd, void* dx, float* dgamma, float* dbeta,
                     void* scratch, int64_t R, int64_t C) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(R >= 0 && C > 0, "bad shape");
    if (R == 0) return PK_OK;
    PK_REQUIRE(dy && x && gamma && mean && rstd, "null pointer");
    PK_REQUIRE((dgamma == nullptr && dbeta == nullptr) || scratch != nullptr, "dgamma/dbeta need scratch");
    if (dtype == PK_F32)
        return norm_bwd_dispatch<float, true>(as_stream(stream), static_cast<const float*>(dy),
                                              static_cast<const float*>(x), gamma, mean, rstd,
                                              static_cast<float*>(dx), dgamma, dbeta,
                                              static_cast<float*>(scratch), R, C);
    return norm_bwd_dispatch<bf16, true>(as_stream(stream), static_cast<const bf16*>(dy),
                                         static_cast<const bf16*>(x), gamma, mean, rstd,
                                         static_cast<bf16*>(dx), dgamma, dbeta,
                                         static_cast<float*>(scratch), R, C);
}

int pk_rope(void* stream, int dtype, void* x, int64_t ld, int64_t col0, int n_heads, int head_dim,
            const int32_t* pos, const float* cos_sin, int64_t n_pos, int64_t R, int inverse) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "head_dim must be even");
    PK_REQUIRE(n_heads >= 0 && col0 >= 0 && col0 + static_cast<int64_t>(n_heads) * head_dim <= ld,
               "rotated columns exceed the row stride");
    if (R <= 0 || n_heads == 0) return PK_OK;
    PK_REQUIRE(x && pos && cos_sin && n_pos > 0, "null pointer");
    const int half = head_dim / 2;
    const int64_t total = R * n_heads * half;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    const float sgn = inverse ? -1.0f : 1.0f;
    if (dtype == PK_BF16 && half % 4 == 0 && ld % 8 == 0 && col0 % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(cos_sin) & 15u) == 0) {
        const int64_t vtotal = total / 4;
        int64_t vblocks = (vtotal + 255) / 256;
        if (vblocks > cap) vblocks = cap;
        rope_vec8_kernel<<<static_cast<unsigned>(vblocks), 256, 0, as_stream(stream)>>>(
            static_cast<bf16*>(x), ld, col0, n_heads, half, pos, cos_sin, n_pos, R, sgn);
        PK_LAUNCH_CHECK();
        return PK_OK;
    }
    if (dtype == PK_F32)
        rope_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<float*>(x), ld, col0, n_heads, half, pos, cos_sin, n_pos, R, sgn);
    else
        rope_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
            static_cast<bf16*>(x), ld, col0, n_heads, half, pos, cos_sin, n_pos, R, sgn);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // extern "C"
