// Flash-attention backward on the tcgen05 tensor cores (bf16, head_dim 64 or 128).
//
// Two kernels, no atomics: every gradient element is owned by one CTA and summed in a fixed
// order, so the result is reproducible bit for bit.
//
//   dQ kernel     CTA = (128-query tile, head, sequence); streams key tiles of 64:
//                   S  = Q K^T, dP = dO V^T            [128 q x 64 keys] in tensor memory
//                   dS = P (dP - delta) scale          bf16 operand tile in shared memory
//                   dQ += dS K                          K re-read as an MN-major operand
//   dK/dV kernel  CTA = (128-key tile, kv head, sequence); streams query tiles of 64 of every
//                 query head of the group, in the TRANSPOSED form so that rows are keys:
//                   S^T = K Q^T, dP^T = V dO^T         [128 keys x 64 q] in tensor memory
//                   P^T, dS^T                           bf16 operand tiles (rows = keys)
//                   dV += P^T dO,  dK += dS^T Q        dO / Q re-read as MN-major operands
//   P is recomputed from the saved log-sum-exp: p = exp2(s*c - lse*log2 e).
//
// CTAs have 256 threads: warps w and w+4 share tensor-memory lane quadrant w and split the 64
// streamed columns, so a thread owns one row and 32 columns of each score tile. With
// head_dim 64 a CTA needs 256 tensor-memory columns and < 100 KB of shared memory, so two
// CTAs share an SM and one CTA's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded (status word, no trap).
//
// Formulas: backward of ops::fused_attention in the reference (src/ops.cpp:903-933).
#include "pk_tc.cuh"

namespace pk {

__device__ int g_attn_bwd_tc_status = 0;

#ifdef PK_ATTN_TIMING
__device__ long long g_attn_dbg[64];
#define PK_T(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && j == 5 && (tid == 0 || tid == 200)) g_attn_dbg[(tid != 0) * 16 + (i)] = clock64(); } while (0)
#else
#define PK_T(i) do { } while (0)
#endif

using namespace tc;

namespace {

constexpr int BW_ROWS = 128;   // rows of the owning tile
constexpr int BW_COLS = 64;    // rows of the streamed tile = columns of the score tile
constexpr int BW_THREADS = 256;
constexpr float LOG2E_ = 1.4426950408889634f;
constexpr uint32_t CH128 = 16384;  // chunk of a 128-row tile: 128 rows x 128 bytes
constexpr uint32_t CH64 = 8192;    // chunk of a 64-row tile

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
// K-major operand: k-step of 16 = 32 bytes inside a chunk, 4 k-steps per 64-wide chunk.
__device__ __forceinline__ uint64_t dk_major(uint32_t tile, int kstep, uint32_t chunk_pitch) {
    return smem_desc(tile + static_cast<uint32_t>(kstep >> 2) * chunk_pitch + static_cast<uint32_t>(kstep & 3) * 32u, 16u, 1024u);
}
// MN-major operand: rows are the contraction index, k-step of 16 rows = 2048 bytes; chunks
// (64 M/N elements each) are chunk_pitch apart.
__device__ __forceinline__ uint64_t dmn_major(uint32_t tile, int kstep, uint32_t chunk_pitch) {
    return smem_desc(tile + static_cast<uint32_t>(kstep) * 2048u, chunk_pitch, 1024u);
}
template <int DK>
__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* map, int col0, int64_t row, uint32_t bar,
                                         uint32_t chunk_pitch) {
#pragma unroll
    for (int c = 0; c < DK / 64; ++c) tma_load_2d(dst + c * chunk_pitch, map, col0 + c * 64, static_cast<int32_t>(row), bar);
}
__device__ __forceinline__ void st32_bf16(uint8_t* chunk, int row, int unit0, const float (&v)[32]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack2(v[g * 8 + 0], v[g * 8 + 1]);
        w.y = pack2(v[g * 8 + 2], v[g * 8 + 3]);
        w.z = pack2(v[g * 8 + 4], v[g * 8 + 5]);
        w.w = pack2(v[g * 8 + 6], v[g * 8 + 7]);
        st_swizzled(chunk, row, unit0 + g, w);
    }
}
__device__ __forceinline__ void st32_global(bf16* dst, const uint32_t (&r)[32]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
        w.y = pack2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
        w.z = pack2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
        w.w = pack2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
        *reinterpret_cast<uint4*>(dst + g * 8) = w;
    }
}

struct BwdParams {
    bf16* dq;
    int64_t lddq;
    bf16* dk;
    int64_t lddk;
    bf16* dv;
    int64_t lddv;
    const float* lse;
    const float* delta;
    int S;
    int Hq, Hkv;
    float scale, scale_log2;
    int causal;
};

// ------------------------------------------------------------------------------ dQ
template <int DK>
struct DqSmem {
    static constexpr int TILEQ = (DK / 64) * (int)CH128;
    static constexpr int TILEK = (DK / 64) * (int)CH64;
    static constexpr int NST = DK == 64 ? 2 : 1;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_DO = TILEQ;
    static constexpr int OFF_K = 2 * TILEQ;
    static constexpr int OFF_V = OFF_K + NST * TILEK;
    static constexpr int OFF_DS = OFF_V + NST * TILEK;
    static constexpr int OFF_BAR = OFF_DS + (int)CH128;
    static constexpr int BYTES = OFF_BAR + 128 + 1024;
};

template <int DK>
__global__ void __launch_bounds__(BW_THREADS, DK == 64 ? 2 : 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const BwdParams p) {
    using L = DqSmem<DK>;
    constexpr int NST = L::NST;
    constexpr uint32_t TMEM_COLS = 256;  // S 64 | dP 64 | dQ DK
    constexpr int OH = DK / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* bar_q = bars;
    uint64_t* bar_kv = bars + 1;  // [2]
    uint64_t* bar_s = bars + 3;
    uint64_t* bar_d = bars + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hf = warp >> 2;
    const int row = quad * 32 + lane;
    const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int64_t seq0 = static_cast<int64_t>(b) * p.S;
    const int q0 = qt * BW_ROWS;
    const int qi = q0 + row;
    const bool row_ok = qi < p.S;
    int nkv = (p.S + BW_COLS - 1) / BW_COLS;
    if (p.causal && 2 * (qt + 1) < nkv) nkv = 2 * (qt + 1);

    if (tid == 0) {
        mbar_init(smem_u32(bar_q), 1);
        mbar_init(smem_u32(&bar_kv[0]), 1);
        mbar_init(smem_u32(&bar_kv[1]), 1);
        mbar_init(smem_u32(bar_s), 1);
        mbar_init(smem_u32(bar_d), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem + lane_off + hf * 32, t_dp = tmem + 64 + lane_off + hf * 32;
    const uint32_t t_dq = tmem + 128;
    const uint32_t sQ = smem_u32(smem + L::OFF_Q), sDO = smem_u32(smem + L::OFF_DO);
    const uint32_t sK0 = smem_u32(smem + L::OFF_K), sV0 = smem_u32(smem + L::OFF_V), sDS = smem_u32(smem + L::OFF_DS);
    uint8_t* pDS = smem + L::OFF_DS;

    if (tid == 0) {
        mbar_expect_tx(smem_u32(bar_q), 2 * L::TILEQ);
        tma_tile<DK>(sQ, &map_q, h * DK, seq0 + q0, smem_u32(bar_q), CH128);
        tma_tile<DK>(sDO, &map_do, h * DK, seq0 + q0, smem_u32(bar_q), CH128);
        mbar_expect_tx(smem_u32(&bar_kv[0]), 2 * L::TILEK);
        tma_tile<DK>(sK0, &map_k, hk * DK, seq0, smem_u32(&bar_kv[0]), CH64);
        tma_tile<DK>(sV0, &map_v, hk * DK, seq0, smem_u32(&bar_kv[0]), CH64);
    }
    // rows past the end of the sequence get lse = +inf, i.e. p = 0 everywhere
    const float neg_lse2 = row_ok ? -p.lse[(seq0 + qi) * p.Hq + h] * LOG2E_ : -INFINITY;
    const float neg_delta_s = row_ok ? -p.delta[(seq0 + qi) * p.Hq + h] * p.scale : 0.0f;
    const uint32_t idesc_s = idesc_bf16(BW_COLS, 0, 0);
    const uint32_t idesc_q = idesc_bf16(DK, 0, 1);
    bool ok = true;

    for (int j = 0; j < nkv; ++j) {
        const int st = NST == 2 ? (j & 1) : 0;
        const uint32_t kv_phase = NST == 2 ? ((j >> 1) & 1) : (j & 1);
        const int kv0 = j * BW_COLS;
        PK_T(0);
        if (tid == 0) {
            if (NST == 1 && j > 0) {  // the single K/V stage is free once dQ of tile j-1 is done
                ok = ok && mbar_wait(smem_u32(bar_d), (j - 1) & 1, abort_flag, &g_attn_bwd_tc_status);
                if (ok) {
                    mbar_expect_tx(smem_u32(&bar_kv[0]), 2 * L::TILEK);
                    tma_tile<DK>(sK0, &map_k, hk * DK, seq0 + kv0, smem_u32(&bar_kv[0]), CH64);
                    tma_tile<DK>(sV0, &map_v, hk * DK, seq0 + kv0, smem_u32(&bar_kv[0]), CH64);
                }
            }
            if (ok && j == 0) ok = mbar_wait(smem_u32(bar_q), 0, abort_flag, &g_attn_bwd_tc_status);
            if (ok) ok = mbar_wait(smem_u32(&bar_kv[st]), kv_phase, abort_flag, &g_attn_bwd_tc_status);
            if (ok) {
                PK_T(1);
                fence_after();
                const uint32_t sK = sK0 + st * L::TILEK, sV = sV0 + st * L::TILEK;
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)
                    mma_bf16(tmem, dk_major(sQ, k, CH128), dk_major(sK, k, CH64), idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)
                    mma_bf16(tmem + 64, dk_major(sDO, k, CH128), dk_major(sV, k, CH64), idesc_s, k > 0 ? 1u : 0u);
                commit(smem_u32(bar_s));
                PK_T(2);
            }
        }
        if (!mbar_wait(smem_u32(bar_s), j & 1, abort_flag, &g_attn_bwd_tc_status)) ok = false;
        PK_T(3);
        // S_j complete implies dQ of tile j-1 (issued earlier on the same pipe) is complete:
        // the dS buffer and, with two stages, the other K/V stage are free again.
        fence_after();
        if (tid == 0 && ok && NST == 2 && j + 1 < nkv) {
            const int sn = st ^ 1;
            mbar_expect_tx(smem_u32(&bar_kv[sn]), 2 * L::TILEK);
            tma_tile<DK>(sK0 + sn * L::TILEK, &map_k, hk * DK, seq0 + kv0 + BW_COLS, smem_u32(&bar_kv[sn]), CH64);
            tma_tile<DK>(sV0 + sn * L::TILEK, &map_v, hk * DK, seq0 + kv0 + BW_COLS, smem_u32(&bar_kv[sn]), CH64);
        }
        {
            const bool need_mask = (p.causal && kv0 + BW_COLS - 1 > q0) || (kv0 + BW_COLS > p.S);
            const int key0 = kv0 + hf * 32;
            uint32_t rs[32], rd[32];
            tmem_ld32(t_s, rs);
            tmem_ld32(t_dp, rd);
            tmem_wait_ld();
            PK_T(4);
            // per element: p = 2^(s*c - lse2) (FFMA + MUFU), ds = p * (dp*scale - delta*scale) (FFMA + FMUL)
            float dsv[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                float pe = ex2_approx(fmaf(__uint_as_float(rs[e]), p.scale_log2, neg_lse2));
                if (need_mask) {
                    const bool vis = key0 + e < p.S && (!p.causal || key0 + e <= qi);
                    pe = vis ? pe : 0.0f;
                }
                dsv[e] = pe * fmaf(__uint_as_float(rd[e]), p.scale, neg_delta_s);
            }
            st32_bf16(pDS, row, hf * 4, dsv);
        }
        PK_T(5);
        fence_async_smem();
        fence_before();
        if (__syncthreads_or(!ok)) {  // CTA-uniform exit as soon as any thread's wait gave up
            ok = false;
            break;
        }
        PK_T(6);
        if (tid == 0) {
            fence_after();
            const uint32_t sK = sK0 + st * L::TILEK;
#pragma unroll
            for (int k = 0; k < BW_COLS / 16; ++k)
                mma_bf16(t_dq, dk_major(sDS, k, CH128), dmn_major(sK, k, CH64), idesc_q, (j > 0 || k > 0) ? 1u : 0u);
            commit(smem_u32(bar_d));
            PK_T(7);
        }
    }
    if (ok) ok = mbar_wait(smem_u32(bar_d), (nkv - 1) & 1, abort_flag, &g_attn_bwd_tc_status);
    if (ok) {
        fence_after();
        bf16* dst = p.dq + (seq0 + qi) * p.lddq + h * DK + hf * OH;
#pragma unroll
        for (int ch = 0; ch < OH / 32; ++ch) {
            uint32_t r[32];
            tmem_ld32(t_dq + lane_off + hf * OH + ch * 32, r);
            tmem_wait_ld();
            if (row_ok) st32_global(dst + ch * 32, r);
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------ dK / dV
template <int DK>
struct DkvSmem {
    static constexpr int TILEK = (DK / 64) * (int)CH128;  // K_j, V_j: 128 rows
    static constexpr int TILEQ = (DK / 64) * (int)CH64;   // Q_i, dO_i: 64 rows
    static constexpr int NST = DK == 64 ? 2 : 1;
    static constexpr int OFF_K = 0;
    static constexpr int OFF_V = TILEK;
    static constexpr int OFF_Q = 2 * TILEK;
    static constexpr int OFF_DO = OFF_Q + NST * TILEQ;
    static constexpr int OFF_P = OFF_DO + NST * TILEQ;
    static constexpr int OFF_DS = OFF_P + (int)CH128;
    static constexpr int OFF_X = OFF_DS + (int)CH128;  // [2 buffers][lse2 | delta][64] floats
    static constexpr int OFF_BAR = OFF_X + 1024;
    static constexpr int BYTES = OFF_BAR + 128 + 1024;
};

template <int DK>
__global__ void __launch_bounds__(BW_THREADS, DK == 64 ? 2 : 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                    const BwdParams p) {
    using L = DkvSmem<DK>;
    constexpr int NST = L::NST;
    constexpr uint32_t TMEM_COLS = DK == 64 ? 256 : 512;  // S^T 64 | dP^T 64 | dV DK | dK DK
    constexpr int OH = DK / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* bar_kv = bars;
    uint64_t* bar_q = bars + 1;  // [2]
    uint64_t* bar_s = bars + 3;
    uint64_t* bar_d = bars + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xb = reinterpret_cast<float*>(smem + L::OFF_X);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hf = warp >> 2;
    const int row = quad * 32 + lane;
    const int kt = blockIdx.x;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int group = p.Hq / p.Hkv;
    const int64_t seq0 = static_cast<int64_t>(b) * p.S;
    const int k0 = kt * BW_ROWS;
    const int kj = k0 + row;  // this thread's key
    const bool key_ok = kj < p.S;
    const int nq_all = (p.S + BW_COLS - 1) / BW_COLS;
    const int i_begin = p.causal ? 2 * kt : 0;
    const int per_head = nq_all - i_begin;
    const int nit = per_head > 0 ? per_head * group : 0;

    // per-query log-sum-exp (in log2 units) and delta of query tile (h, i) -> buffer `buf`
    auto stage_stats = [&](int buf, int h, int q0) {
        if (tid < 128) {
            const int c = tid & 63;
            const int q = q0 + c;
            // -lse*log2(e) (queries past the end: -inf, so that p = 0) and -delta*scale
            float v = tid < 64 ? -INFINITY : 0.0f;
            if (q < p.S)
                v = tid < 64 ? -p.lse[(seq0 + q) * p.Hq + h] * LOG2E_ : -p.delta[(seq0 + q) * p.Hq + h] * p.scale;
            xb[buf * 128 + (tid < 64 ? 0 : 64) + c] = v;
        }
    };

    if (tid == 0) {
        mbar_init(smem_u32(bar_kv), 1);
        mbar_init(smem_u32(&bar_q[0]), 1);
        mbar_init(smem_u32(&bar_q[1]), 1);
        mbar_init(smem_u32(bar_s), 1);
        mbar_init(smem_u32(bar_d), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    if (nit > 0) stage_stats(0, hk * group, i_begin * BW_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem + lane_off + hf * 32, t_dp = tmem + 64 + lane_off + hf * 32;
    const uint32_t t_dv = tmem + 128, t_dk = tmem + 128 + DK;
    const uint32_t sK = smem_u32(smem + L::OFF_K), sV = smem_u32(smem + L::OFF_V);
    const uint32_t sQ0 = smem_u32(smem + L::OFF_Q), sDO0 = smem_u32(smem + L::OFF_DO);
    const uint32_t sP = smem_u32(smem + L::OFF_P), sDS = smem_u32(smem + L::OFF_DS);
    uint8_t* pP = smem + L::OFF_P;
    uint8_t* pDS = smem + L::OFF_DS;

    if (tid == 0) {
        mbar_expect_tx(smem_u32(bar_kv), 2 * L::TILEK);
        tma_tile<DK>(sK, &map_k, hk * DK, seq0 + k0, smem_u32(bar_kv), CH128);
        tma_tile<DK>(sV, &map_v, hk * DK, seq0 + k0, smem_u32(bar_kv), CH128);
        if (nit > 0) {
            mbar_expect_tx(smem_u32(&bar_q[0]), 2 * L::TILEQ);
            tma_tile<DK>(sQ0, &map_q, (hk * group) * DK, seq0 + i_begin * BW_COLS, smem_u32(&bar_q[0]), CH64);
            tma_tile<DK>(sDO0, &map_do, (hk * group) * DK, seq0 + i_begin * BW_COLS, smem_u32(&bar_q[0]), CH64);
        }
    }
    const uint32_t idesc_s = idesc_bf16(BW_COLS, 0, 0);
    const uint32_t idesc_g = idesc_bf16(DK, 0, 1);
    bool ok = true;

    for (int it = 0; it < nit; ++it) {
        const int g = it / per_head, i = i_begin + it % per_head;
        const int h = hk * group + g;
        const int st = NST == 2 ? (it & 1) : 0;
        const uint32_t q_phase = NST == 2 ? ((it >> 1) & 1) : (it & 1);
        const int q0 = i * BW_COLS;
        if (tid == 0) {
            if (NST == 1 && it > 0) {  // single Q/dO stage: wait for dV/dK of the previous iteration
                ok = ok && mbar_wait(smem_u32(bar_d), (it - 1) & 1, abort_flag, &g_attn_bwd_tc_status);
                if (ok) {
                    mbar_expect_tx(smem_u32(&bar_q[0]), 2 * L::TILEQ);
                    tma_tile<DK>(sQ0, &map_q, h * DK, seq0 + q0, smem_u32(&bar_q[0]), CH64);
                    tma_tile<DK>(sDO0, &map_do, h * DK, seq0 + q0, smem_u32(&bar_q[0]), CH64);
                }
            }
            if (ok && it == 0) ok = mbar_wait(smem_u32(bar_kv), 0, abort_flag, &g_attn_bwd_tc_status);
            if (ok) ok = mbar_wait(smem_u32(&bar_q[st]), q_phase, abort_flag, &g_attn_bwd_tc_status);
            if (ok) {
                fence_after();
                const uint32_t sQ = sQ0 + st * L::TILEQ, sDO = sDO0 + st * L::TILEQ;
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)   // S^T = K Q^T
                    mma_bf16(tmem, dk_major(sK, k, CH128), dk_major(sQ, k, CH64), idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)   // dP^T = V dO^T
                    mma_bf16(tmem + 64, dk_major(sV, k, CH128), dk_major(sDO, k, CH64), idesc_s, k > 0 ? 1u : 0u);
                commit(smem_u32(bar_s));
            }
        }
        if (!mbar_wait(smem_u32(bar_s), it & 1, abort_flag, &g_attn_bwd_tc_status)) ok = false;
        // S^T of this iteration complete => dV/dK of the previous one (issued earlier) complete:
        // P^T, dS^T and the other Q/dO stage may be overwritten.
        fence_after();
        if (it + 1 < nit) {
            const int itn = it + 1;
            const int hn = hk * group + itn / per_head, in_ = i_begin + itn % per_head;
            if (tid == 0 && ok && NST == 2) {
                const int sn = st ^ 1;
                mbar_expect_tx(smem_u32(&bar_q[sn]), 2 * L::TILEQ);
                tma_tile<DK>(sQ0 + sn * L::TILEQ, &map_q, hn * DK, seq0 + in_ * BW_COLS, smem_u32(&bar_q[sn]), CH64);
                tma_tile<DK>(sDO0 + sn * L::TILEQ, &map_do, hn * DK, seq0 + in_ * BW_COLS, smem_u32(&bar_q[sn]), CH64);
            }
            stage_stats((it + 1) & 1, hn, in_ * BW_COLS);  // read after the barrier below
        }
        {
            const bool need_mask = (p.causal && k0 + BW_ROWS - 1 > q0) || (q0 + BW_COLS > p.S) || (k0 + BW_ROWS > p.S);
            const float* xs = xb + (it & 1) * 128 + hf * 32;
            const int qc0 = q0 + hf * 32;
            uint32_t rs[32], rd[32];
            tmem_ld32(t_s, rs);
            tmem_ld32(t_dp, rd);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < 4; ++g) {  // 8 queries -> one 16-byte unit of each operand tile
                float pe[8], de[8];
#pragma unroll
                for (int e8 = 0; e8 < 8; ++e8) {
                    const int e = g * 8 + e8;
                    float pq = ex2_approx(fmaf(__uint_as_float(rs[e]), p.scale_log2, xs[e]));
                    if (need_mask) {
                        const bool vis = key_ok && (!p.causal || kj <= qc0 + e);
                        pq = vis ? pq : 0.0f;
                    }
                    pe[e8] = pq;
                    de[e8] = pq * fmaf(__uint_as_float(rd[e]), p.scale, xs[64 + e]);
                }
                uint4 wp, wd;
                wp.x = pack2(pe[0], pe[1]); wp.y = pack2(pe[2], pe[3]); wp.z = pack2(pe[4], pe[5]); wp.w = pack2(pe[6], pe[7]);
                wd.x = pack2(de[0], de[1]); wd.y = pack2(de[2], de[3]); wd.z = pack2(de[4], de[5]); wd.w = pack2(de[6], de[7]);
                st_swizzled(pP, row, hf * 4 + g, wp);
                st_swizzled(pDS, row, hf * 4 + g, wd);
            }
        }
        fence_async_smem();
        fence_before();
        if (__syncthreads_or(!ok)) {  // CTA-uniform exit as soon as any thread's wait gave up
            ok = false;
            break;
        }
        if (tid == 0) {
            fence_after();
            const uint32_t sQ = sQ0 + st * L::TILEQ, sDO = sDO0 + st * L::TILEQ;
#pragma unroll
            for (int k = 0; k < BW_COLS / 16; ++k)   // dV += P^T dO   (contraction over the 64 queries)
                mma_bf16(t_dv, dk_major(sP, k, CH128), dmn_major(sDO, k, CH64), idesc_g, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
            for (int k = 0; k < BW_COLS / 16; ++k)   // dK += dS^T Q
                mma_bf16(t_dk, dk_major(sDS, k, CH128), dmn_major(sQ, k, CH64), idesc_g, (it > 0 || k > 0) ? 1u : 0u);
            commit(smem_u32(bar_d));
        }
    }
    if (ok && nit > 0) ok = mbar_wait(smem_u32(bar_d), (nit - 1) & 1, abort_flag, &g_attn_bwd_tc_status);
    if (ok) {
        fence_after();
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            bf16* dst = (which == 0 ? p.dv + (seq0 + kj) * p.lddv : p.dk + (seq0 + kj) * p.lddk) + hk * DK + hf * OH;
            const uint32_t t_src = (which == 0 ? t_dv : t_dk) + lane_off + hf * OH;
#pragma unroll
            for (int ch = 0; ch < OH / 32; ++ch) {
                uint32_t r[32];
                if (nit > 0) {
                    tmem_ld32(t_src + ch * 32, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) r[e] = 0u;
                }
                if (key_ok) st32_global(dst + ch * 32, r);
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

template <int DK>
int launch_bwd(cudaStream_t st, const CUtensorMap& mq128, const CUtensorMap& mdo128, const CUtensorMap& mk64,
               const CUtensorMap& mv64, const CUtensorMap& mq64, const CUtensorMap& mdo64, const CUtensorMap& mk128,
               const CUtensorMap& mv128, const BwdParams& p, int64_t B) {
    auto kq = attn_bwd_dq_kernel<DK>;
    auto kkv = attn_bwd_dkv_kernel<DK>;
    static bool attr = false;
    if (!attr) {
        PK_CHECK_CUDA(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<DK>::BYTES));
        PK_CHECK_CUDA(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<DK>::BYTES));
        attr = true;
    }
    const unsigned tiles = static_cast<unsigned>((p.S + BW_ROWS - 1) / BW_ROWS);
    dim3 gq(tiles, p.Hq, static_cast<unsigned>(B));
    kq<<<gq, BW_THREADS, DqSmem<DK>::BYTES, st>>>(mq128, mk64, mv64, mdo128, p);
    PK_LAUNCH_CHECK();
    dim3 gkv(tiles, p.Hkv, static_cast<unsigned>(B));
    kkv<<<gkv, BW_THREADS, DkvSmem<DK>::BYTES, st>>>(mq64, mk128, mv128, mdo64, p);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // namespace

int attn_tc_bwd(cudaStream_t st, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                const float* lse, const float* delta, const void* dout, int64_t lddo, void* dq, int64_t lddq,
                void* dk_, int64_t lddk, void* dv, int64_t lddv, int64_t B, int64_t S, int Hq, int Hkv, int dk,
                float scale, int causal) {
    CUtensorMap mq128, mdo128, mk64, mv64, mq64, mdo64, mk128, mv128;
    const int64_t R = B * S;
    const int64_t wq = static_cast<int64_t>(Hq) * dk, wk = static_cast<int64_t>(Hkv) * dk;
    int rc;
    if ((rc = make_tensor_map(&mq128, q, wq, R, ldq, 64, 128)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mdo128, dout, wq, R, lddo, 64, 128)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mk64, k, wk, R, ldk, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mv64, v, wk, R, ldv, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mq64, q, wq, R, ldq, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mdo64, dout, wq, R, lddo, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mk128, k, wk, R, ldk, 64, 128)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mv128, v, wk, R, ldv, 64, 128)) != PK_OK) return rc;
    BwdParams p;
    p.dq = static_cast<bf16*>(dq);
    p.lddq = lddq;
    p.dk = static_cast<bf16*>(dk_);
    p.lddk = lddk;
    p.dv = static_cast<bf16*>(dv);
    p.lddv = lddv;
    p.lse = lse;
    p.delta = delta;
    p.S = static_cast<int>(S);
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale = scale;
    p.scale_log2 = scale * LOG2E_;
    p.causal = causal;
    return dk == 64 ? launch_bwd<64>(st, mq128, mdo128, mk64, mv64, mq64, mdo64, mk128, mv128, p, B)
                    : launch_bwd<128>(st, mq128, mdo128, mk64, mv64, mq64, mdo64, mk128, mv128, p, B);
}

// Status word of the backward kernels, for pk_attn_tc_status.
int attn_bwd_tc_status(int* status_h, int clear) {
    PK_CHECK_CUDA(cudaMemcpyFromSymbol(status_h, g_attn_bwd_tc_status, sizeof(int)));
    if (clear) {
        const int zero = 0;
        PK_CHECK_CUDA(cudaMemcpyToSymbol(g_attn_bwd_tc_status, &zero, sizeof(int)));
    }
    return PK_OK;
}

#ifdef PK_ATTN_TIMING
extern "C" int pk_debug_read(long long* out_h) {
    cudaDeviceSynchronize();
    return cudaMemcpyFromSymbol(out_h, g_attn_dbg, sizeof(long long) * 64) == cudaSuccess ? 0 : 2;
}
#endif

}  // namespace pk
