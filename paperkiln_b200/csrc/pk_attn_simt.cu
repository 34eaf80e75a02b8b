// Flash-style attention with fp32 arithmetic on the SIMT pipes: forward, and a
// backward split into a dQ pass and a dK/dV pass so that no gradient needs an
// unordered atomic (every output element is owned by one thread and summed in a
// fixed order). Serves the fp32 precision mode and any head_dim in {8,16,32,64,128};
// the score matrix is never written to memory.
//
// Semantics follow ops::fused_attention of the reference (src/ops.cpp:863-934):
// rows are B stacked sequences of length S; row i of a sequence sees keys
// [sequence start, i] when causal, the whole sequence otherwise; the softmax is
// max-subtracted; dq, dk, dv are the hand-derived softmax-attention gradients.
// Query head h reads key/value head h / (Hq / Hkv).
#include "pk_common.cuh"

namespace pk {

constexpr int AT_ROWS = 32;   // rows (queries or keys) per block
constexpr int AT_TPR = 4;     // threads per row
constexpr int AT_THREADS = AT_ROWS * AT_TPR;
constexpr int AT_TILE = 32;   // rows of the streamed operand per shared-memory tile

__device__ __forceinline__ float group4_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// Cooperative load of `rows` rows x DK columns (head slice) into shared memory as fp32.
template <typename T, int DK>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int64_t ld, int64_t row0, int64_t row_end,
                                          int rows) {
    for (int i = threadIdx.x; i < rows * DK; i += AT_THREADS) {
        const int r = i / DK, c = i % DK;
        const int64_t gr = row0 + r;
        dst[r * DK + c] = gr < row_end ? to_f32(src[gr * ld + c]) : 0.0f;
    }
}

template <typename T, int EPT>
__global__ void __launch_bounds__(AT_THREADS)
attn_fwd_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                const T* __restrict__ v, int64_t ldv, T* __restrict__ out, int64_t ldo,
                float* __restrict__ lse, int64_t S, int Hq, int Hkv, float scale, int causal) {
    constexpr int DK = EPT * AT_TPR;
    __shared__ float Ks[AT_TILE * DK];
    __shared__ float Vs[AT_TILE * DK];
    const int part = threadIdx.x & 3, rloc = threadIdx.x >> 2;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (Hq / Hkv);
    const int64_t seq0 = static_cast<int64_t>(b) * S;
    const int64_t q0 = static_cast<int64_t>(blockIdx.x) * AT_ROWS;
    const int64_t qi = q0 + rloc;  // position inside the sequence
    const bool active = qi < S;
    float qr[EPT], o[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        qr[i] = active ? to_f32(q[(seq0 + qi) * ldq + h * DK + part + 4 * i]) : 0.0f;
        o[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    int64_t kv_end = causal ? q0 + AT_ROWS : S;
    if (kv_end > S) kv_end = S;
    for (int64_t kv0 = 0; kv0 < kv_end; kv0 += AT_TILE) {
        __syncthreads();
        load_tile<T, DK>(Ks, k + hk * DK, ldk, seq0 + kv0, seq0 + S, AT_TILE);
        load_tile<T, DK>(Vs, v + hk * DK, ldv, seq0 + kv0, seq0 + S, AT_TILE);
        __syncthreads();
        float s[AT_TILE];
        float mt = -INFINITY;
#pragma unroll
        for (int j = 0; j < AT_TILE; ++j) {
            float d = 0.0f;
#pragma unroll
            for (int i = 0; i < EPT; ++i) d = fmaf(qr[i], Ks[j * DK + part + 4 * i], d);
            d = group4_sum(d) * scale;
            const int64_t kj = kv0 + j;
            const bool vis = kj < S && (!causal || kj <= qi);
            s[j] = vis ? d : -INFINITY;
            mt = fmaxf(mt, s[j]);
        }
        const float m_new = fmaxf(m, mt);
        if (m_new > -INFINITY) {
            const float corr = expf(m - m_new);  // m == -inf gives 0
            l *= corr;
#pragma unroll
            for (int i = 0; i < EPT; ++i) o[i] *= corr;
#pragma unroll
            for (int j = 0; j < AT_TILE; ++j) {
                const float pj = expf(s[j] - m_new);  // masked entries give 0
                l += pj;
#pragma unroll
                for (int i = 0; i < EPT; ++i) o[i] = fmaf(pj, Vs[j * DK + part + 4 * i], o[i]);
            }
            m = m_new;
        }
    }
    if (active) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < EPT; ++i)
            out[(seq0 + qi) * ldo + h * DK + part + 4 * i] = from_f32<T>(o[i] * inv);
        if (part == 0) lse[(seq0 + qi) * Hq + h] = m + logf(l);
    }
}

// delta[row, h] = sum_c dout[row, h, c] * out[row, h, c]; one warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const T* __restrict__ out, int64_t ldo, const T* __restrict__ dout, int64_t lddo,
                  float* __restrict__ delta, int64_t R, int Hq, int dk) {
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (w >= R * Hq) return;
    const int64_t row = w / Hq;
    const int h = static_cast<int>(w % Hq);
    float acc = 0.0f;
    for (int c = lane; c < dk; c += 32)
        acc += to_f32(out[row * ldo + h * dk + c]) * to_f32(dout[row * lddo + h * dk + c]);
    acc = warp_sum(acc);
    if (lane == 0) delta[w] = acc;
}

template <typename T, int EPT>
__global__ void __launch_bounds__(AT_THREADS)
attn_bwd_dq_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                   const T* __restrict__ v, int64_t ldv, const float* __restrict__ lse,
                   const float* __restrict__ delta, const T* __restrict__ dout, int64_t lddo,
                   T* __restrict__ dq, int64_t lddq, int64_t S, int Hq, int Hkv, float scale, int causal) {
    constexpr int DK = EPT * AT_TPR;
    __shared__ float Ks[AT_TILE * DK];
    __shared__ float Vs[AT_TILE * DK];
    const int part = threadIdx.x & 3, rloc = threadIdx.x >> 2;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (Hq / Hkv);
    const int64_t seq0 = static_cast<int64_t>(b) * S;
    const int64_t q0 = static_cast<int64_t>(blockIdx.x) * AT_ROWS;
    const int64_t qi = q0 + rloc;
    const bool active = qi < S;
    float qr[EPT], dor[EPT], acc[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        qr[i] = active ? to_f32(q[(seq0 + qi) * ldq + h * DK + part + 4 * i]) : 0.0f;
        dor[i] = active ? to_f32(dout[(seq0 + qi) * lddo + h * DK + part + 4 * i]) : 0.0f;
        acc[i] = 0.0f;
    }
    const float lse_i = active ? lse[(seq0 + qi) * Hq + h] : 0.0f;
    const float del_i = active ? delta[(seq0 + qi) * Hq + h] : 0.0f;
    int64_t kv_end = causal ? q0 + AT_ROWS : S;
    if (kv_end > S) kv_end = S;
    for (int64_t kv0 = 0; kv0 < kv_end; kv0 += AT_TILE) {
        __syncthreads();
        load_tile<T, DK>(Ks, k + hk * DK, ldk, seq0 + kv0, seq0 + S, AT_TILE);
        load_tile<T, DK>(Vs, v + hk * DK, ldv, seq0 + kv0, seq0 + S, AT_TILE);
        __syncthreads();
#pragma unroll 4
        for (int j = 0; j < AT_TILE; ++j) {
            float d = 0.0f, dp = 0.0f;
#pragma unroll
            for (int i = 0; i < EPT; ++i) {
                d = fmaf(qr[i], Ks[j * DK + part + 4 * i], d);
                dp = fmaf(dor[i], Vs[j * DK + part + 4 * i], dp);
            }
            d = group4_sum(d) * scale;
            dp = group4_sum(dp);
            const int64_t kj = kv0 + j;
            const bool vis = active && kj < S && (!causal || kj <= qi);
            const float p = vis ? expf(d - lse_i) : 0.0f;
            const float ds = scale * p * (dp - del_i);
#pragma unroll
            for (int i = 0; i < EPT; ++i) acc[i] = fmaf(ds, Ks[j * DK + part + 4 * i], acc[i]);
        }
    }
    if (active) {
#pragma unroll
        for (int i = 0; i < EPT; ++i)
            dq[(seq0 + qi) * lddq + h * DK + part + 4 * i] = from_f32<T>(acc[i]);
    }
}

template <typename T, int EPT>
__global__ void __launch_bounds__(AT_THREADS)
attn_bwd_dkv_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                    const T* __restrict__ v, int64_t ldv, const float* __restrict__ lse,
                    const float* __restrict__ delta, const T* __restrict__ dout, int64_t lddo,
                    T* __restrict__ dk_, int64_t lddk, T* __restrict__ dv, int64_t lddv, int64_t S, int Hq,
                    int Hkv, float scale, int causal) {
    constexpr int DK = EPT * AT_TPR;
    __shared__ float Qs[AT_TILE * DK];
    __shared__ float Os[AT_TILE * DK];  // dout tile
    __shared__ float Ls[AT_TILE], Ds[AT_TILE];
    const int part = threadIdx.x & 3, rloc = threadIdx.x >> 2;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int group = Hq / Hkv;
    const int64_t seq0 = static_cast<int64_t>(b) * S;
    const int64_t k0 = static_cast<int64_t>(blockIdx.x) * AT_ROWS;
    const int64_t kj = k0 + rloc;
    const bool active = kj < S;
    float kr[EPT], vr[EPT], dka[EPT], dva[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        kr[i] = active ? to_f32(k[(seq0 + kj) * ldk + hk * DK + part + 4 * i]) : 0.0f;
        vr[i] = active ? to_f32(v[(seq0 + kj) * ldv + hk * DK + part + 4 * i]) : 0.0f;
        dka[i] = 0.0f;
        dva[i] = 0.0f;
    }
    const int64_t q_begin = causal ? (k0 / AT_TILE) * AT_TILE : 0;
    for (int g = 0; g < group; ++g) {
        const int h = hk * group + g;
        for (int64_t q0 = q_begin; q0 < S; q0 += AT_TILE) {
            __syncthreads();
            load_tile<T, DK>(Qs, q + h * DK, ldq, seq0 + q0, seq0 + S, AT_TILE);
            load_tile<T, DK>(Os, dout + h * DK, lddo, seq0 + q0, seq0 + S, AT_TILE);
            if (threadIdx.x < AT_TILE) {
                const int64_t qi = q0 + threadIdx.x;
                Ls[threadIdx.x] = qi < S ? lse[(seq0 + qi) * Hq + h] : 0.0f;
                Ds[threadIdx.x] = qi < S ? delta[(seq0 + qi) * Hq + h] : 0.0f;
            }
            __syncthreads();
#pragma unroll 4
            for (int i2 = 0; i2 < AT_TILE; ++i2) {
                float d = 0.0f, dp = 0.0f;
#pragma unroll
                for (int i = 0; i < EPT; ++i) {
                    d = fmaf(kr[i], Qs[i2 * DK + part + 4 * i], d);
                    dp = fmaf(vr[i], Os[i2 * DK + part + 4 * i], dp);
                }
                d = group4_sum(d) * scale;
                dp = group4_sum(dp);
                const int64_t qi = q0 + i2;
                const bool vis = active && qi < S && (!causal || kj <= qi);
                const float p = vis ? expf(d - Ls[i2]) : 0.0f;
                const float ds = scale * p * (dp - Ds[i2]);
#pragma unroll
                for (int i = 0; i < EPT; ++i) {
                    dva[i] = fmaf(p, Os[i2 * DK + part + 4 * i], dva[i]);
                    dka[i] = fmaf(ds, Qs[i2 * DK + part + 4 * i], dka[i]);
                }
            }
        }
    }
    if (active) {
#pragma unroll
        for (int i = 0; i < EPT; ++i) {
            dk_[(seq0 + kj) * lddk + hk * DK + part + 4 * i] = from_f32<T>(dka[i]);
            dv[(seq0 + kj) * lddv + hk * DK + part + 4 * i] = from_f32<T>(dva[i]);
        }
    }
}

static thread_local int g_attn_last_path = -1;
static int g_attn_force_simt = 0;
// tcgen05 kernels: forward in pk_attn_fwd_row.cu, backward in pk_attn_bwd_ws.cu
int attn_bwd_ws(cudaStream_t st, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                const void* out, int64_t ldo, const float* lse, const void* dout, int64_t lddo, void* dq, int64_t lddq,
                void* dk_, int64_t lddk, void* dv, int64_t lddv, float* scratch, int64_t B, int64_t S, int Hq, int Hkv,
                int dk, float scale, int causal);
size_t attn_bwd_ws_scratch_bytes(int64_t B, int64_t S, int Hq);
int attn_fwd_row(cudaStream_t st, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                 void* out, int64_t ldo, float* lse, int64_t B, int64_t S, int Hq, int Hkv, int dk, float scale,
                 int causal);
int attn_tc_supported(int dtype, int dk, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                      int64_t ldv, const void* out, int64_t ldo, int64_t B, int64_t S);  // pk_tc_host.cu

struct AttnArgs {
    const void *q, *k, *v, *out, *dout;
    void *o_w, *dq, *dk, *dv;
    int64_t ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv;
    float* lse_w;
    const float* lse;
    float* delta;
    int64_t B, S;
    int Hq, Hkv;
    float scale;
    int causal;
};

template <typename T, int EPT>
int attn_fwd_launch(cudaStream_t st, const AttnArgs& a) {
    dim3 grid(static_cast<unsigned>((a.S + AT_ROWS - 1) / AT_ROWS), a.Hq, static_cast<unsigned>(a.B));
    attn_fwd_kernel<T, EPT><<<grid, AT_THREADS, 0, st>>>(
        static_cast<const T*>(a.q), a.ldq, static_cast<const T*>(a.k), a.ldk, static_cast<const T*>(a.v), a.ldv,
        static_cast<T*>(a.o_w), a.ldo, a.lse_w, a.S, a.Hq, a.Hkv, a.scale, a.causal);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

template <typename T, int EPT>
int attn_bwd_launch(cudaStream_t st, const AttnArgs& a, int dk) {
    const int64_t R = a.B * a.S;
    attn_delta_kernel<T><<<static_cast<unsigned>((R * a.Hq + 7) / 8), 256, 0, st>>>(
        static_cast<const T*>(a.out), a.ldo, static_cast<const T*>(a.dout), a.lddo, a.delta, R, a.Hq, dk);
    PK_LAUNCH_CHECK();
    dim3 gq(static_cast<unsigned>((a.S + AT_ROWS - 1) / AT_ROWS), a.Hq, static_cast<unsigned>(a.B));
    attn_bwd_dq_kernel<T, EPT><<<gq, AT_THREADS, 0, st>>>(
        static_cast<const T*>(a.q), a.ldq, static_cast<const T*>(a.k), a.ldk, static_cast<const T*>(a.v), a.ldv,
        a.lse, a.delta, static_cast<const T*>(a.dout), a.lddo, static_cast<T*>(a.dq), a.lddq, a.S, a.Hq, a.Hkv,
        a.scale, a.causal);
    PK_LAUNCH_CHECK();
    dim3 gk(static_cast<unsigned>((a.S + AT_ROWS - 1) / AT_ROWS), a.Hkv, static_cast<unsigned>(a.B));
    attn_bwd_dkv_kernel<T, EPT><<<gk, AT_THREADS, 0, st>>>(
        static_cast<const T*>(a.q), a.ldq, static_cast<const T*>(a.k), a.ldk, static_cast<const T*>(a.v), a.ldv,
        a.lse, a.delta, static_cast<const T*>(a.dout), a.lddo, static_cast<T*>(a.dk), a.lddk,
        static_cast<T*>(a.dv), a.lddv, a.S, a.Hq, a.Hkv, a.scale, a.causal);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

template <typename T>
int attn_dispatch(cudaStream_t st, const AttnArgs& a, int dk, bool backward) {
    switch (dk) {
#define PK_CASE(D)                                                                   \
    case D:                                                                          \
        return backward ? attn_bwd_launch<T, D / 4>(st, a, dk) : attn_fwd_launch<T, D / 4>(st, a)
        PK_CASE(8);
        PK_CASE(16);
        PK_CASE(32);
        PK_CASE(64);
        PK_CASE(128);
#undef PK_CASE
        default:
            set_error("attention: head_dim %d is not one of 8, 16, 32, 64, 128", dk);
            return PK_ERR_UNSUPPORTED;
    }
}

static int check_common(int dtype, int64_t B, int64_t S, int Hq, int Hkv, int dk) {
    PK_REQUIRE(valid_dtype(dtype), "bad dtype");
    PK_REQUIRE(B >= 0 && S >= 0 && Hq > 0 && Hkv > 0 && dk > 0, "bad shape");
    PK_REQUIRE(Hq % Hkv == 0, "Hq must be a multiple of Hkv");
    PK_REQUIRE(B <= 65535 && Hq <= 65535, "batch or head count exceeds the launch grid");
    return PK_OK;
}

}  // namespace pk

using namespace pk;

extern "C" {

int pk_attn_fwd(void* stream, int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk,
                const void* v, int64_t ldv, void* out, int64_t ldo, float* lse, int64_t B, int64_t S,
                int Hq, int Hkv, int dk, float scale, int causal) {
    int rc = check_common(dtype, B, S, Hq, Hkv, dk);
    if (rc != PK_OK) return rc;
    if (B == 0 || S == 0) return PK_OK;
    PK_REQUIRE(q && k && v && out && lse, "null pointer");
    PK_REQUIRE(ldq >= Hq * dk && ldo >= Hq * dk && ldk >= Hkv * dk && ldv >= Hkv * dk, "row stride too small");
    AttnArgs a{};
    a.q = q; a.k = k; a.v = v; a.o_w = out; a.lse_w = lse;
    a.ldq = ldq; a.ldk = ldk; a.ldv = ldv; a.ldo = ldo;
    a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.scale = scale; a.causal = causal;
    // causal attention touches half of the score matrix: 2 GEMMs x 2 flops x S^2/2 x dk
    ProfScope prof(PROF_ATTN_FWD, (causal ? 2.0 : 4.0) * B * S * S * Hq * dk, as_stream(stream));
    if (!g_attn_force_simt && attn_tc_supported(dtype, dk, q, ldq, k, ldk, v, ldv, out, ldo, B, S)) {
        g_attn_last_path = 1;
        note_launch(PATH_ATTN_FWD_TC);
        return attn_fwd_row(as_stream(stream), q, ldq, k, ldk, v, ldv, out, ldo, lse, B, S, Hq, Hkv, dk, scale, causal);
    }
    g_attn_last_path = 0;
    note_launch(PATH_ATTN_FWD_SIMT);
    if (dtype == PK_F32) return attn_dispatch<float>(as_stream(stream), a, dk, false);
    return attn_dispatch<bf16>(as_stream(stream), a, dk, false);
}

size_t pk_attn_bwd_scratch_bytes(int64_t B, int64_t S, int Hq) {
    // delta [B*S, Hq] for the SIMT kernel; two head-major padded arrays for the tcgen05 ones
    const size_t plain = static_cast<size_t>(B) * static_cast<size_t>(S) * static_cast<size_t>(Hq) * sizeof(float);
    const size_t ws = attn_bwd_ws_scratch_bytes(B, S, Hq);
    return plain > ws ? plain : ws;
}

int pk_attn_bwd(void* stream, int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk,
                const void* v, int64_t ldv, const void* out, int64_t ldo, const float* lse, const void* dout,
                int64_t lddo, void* dq, int64_t lddq, void* dk_, int64_t lddk, void* dv, int64_t lddv,
                void* scratch, int64_t B, int64_t S, int Hq, int Hkv, int dk, float scale, int causal) {
    int rc = check_common(dtype, B, S, Hq, Hkv, dk);
    if (rc != PK_OK) return rc;
    if (B == 0 || S == 0) return PK_OK;
    PK_REQUIRE(q && k && v && out && lse && dout && dq && dk_ && dv && scratch, "null pointer");
    PK_REQUIRE(ldq >= Hq * dk && ldo >= Hq * dk && lddo >= Hq * dk && lddq >= Hq * dk, "row stride too small");
    PK_REQUIRE(ldk >= Hkv * dk && ldv >= Hkv * dk && lddk >= Hkv * dk && lddv >= Hkv * dk, "row stride too small");
    AttnArgs a{};
    a.q = q; a.k = k; a.v = v; a.out = out; a.dout = dout; a.lse = lse;
    a.dq = dq; a.dk = dk_; a.dv = dv; a.delta = static_cast<float*>(scratch);
    a.ldq = ldq; a.ldk = ldk; a.ldv = ldv; a.ldo = ldo; a.lddo = lddo; a.lddq = lddq; a.lddk = lddk; a.lddv = lddv;
    a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.scale = scale; a.causal = causal;
    // backward = 5 GEMM-shaped products on the visible half: 2.5 x the forward
    ProfScope prof(PROF_ATTN_BWD, (causal ? 5.0 : 10.0) * B * S * S * Hq * dk, as_stream(stream));
    if (!g_attn_force_simt && attn_tc_supported(dtype, dk, q, ldq, k, ldk, v, ldv, out, ldo, B, S) &&
        attn_tc_supported(dtype, dk, dout, lddo, dk_, lddk, dv, lddv, dq, lddq, B, S)) {
        g_attn_last_path = 1;
        note_launch(PATH_ATTN_BWD_TC);
        return attn_bwd_ws(as_stream(stream), q, ldq, k, ldk, v, ldv, out, ldo, lse, dout, lddo, dq, lddq, dk_, lddk,
                           dv, lddv, a.delta, B, S, Hq, Hkv, dk, scale, causal);
    }
    g_attn_last_path = 0;
    note_launch(PATH_ATTN_BWD_SIMT);
    if (dtype == PK_F32) return attn_dispatch<float>(as_stream(stream), a, dk, true);
    return attn_dispatch<bf16>(as_stream(stream), a, dk, true);
}

int pk_attn_last_path(void) { return g_attn_last_path; }
int pk_attn_force_simt(int on) {
    g_attn_force_simt = on ? 1 : 0;
    return PK_OK;
}

}  // extern "C"
