// Flash attention forward on the tcgen05 tensor cores, one 128-query tile per CTA (bf16 operands,
// fp32 accumulation in tensor memory), head_dim 64 or 128, causal or full, grouped-query head
// mapping, B stacked sequences. This is forward variant 0 (pk_attn_fwd_variant); the default is
// the warp-specialised kernel in pk_attn_fwd_ws.cu. The file also holds the tensor-map helper
// shared by the attention kernels and the combined status word.
//
// CTAs have 256 threads working on a 128-row tile: warps w and w+4 share tensor-memory lane
// quadrant w (rows 32w..32w+31) and split the COLUMNS of every tile between them, so thread
// (row r, half hf) owns row r of the tile and 64 of its 128 score columns / half of its
// head_dim output columns. Thread 0 additionally issues the TMA loads and the MMAs.
// Per (128-query tile, head, sequence), per 128-key tile:
//     S = Q K^T                tcgen05.mma, operands TMA-loaded into 128B-swizzled smem
//     p = exp2(S*c - m)        one sweep over the thread's 64 columns held in registers; the
//                              row maximum is combined with the partner thread through smem
//     O_tile = P V             P written as a bf16 operand tile; V read MN-major (no transpose)
//     o = o*corr + O_tile      running output in registers, rescaled per tile
// Every mbarrier wait is bounded (status word, no trap).
//
// Semantics: ops::fused_attention of the reference (src/ops.cpp:863-934) applied per head.
#include "pk_tc.cuh"

#include <mutex>

namespace pk {

__device__ int g_attn_tc_status = 0;
#ifdef PK_ATTN_TIMING
__device__ long long g_attn_fwd_dbg[64];
#define PK_TF(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && j == 5 && (tid == 0 || tid == 200)) g_attn_fwd_dbg[(tid != 0) * 16 + (i)] = clock64(); } while (0)
extern "C" int pk_debug_read_fwd(long long* out_h) {
    cudaDeviceSynchronize();
    return cudaMemcpyFromSymbol(out_h, g_attn_fwd_dbg, sizeof(long long) * 64) == cudaSuccess ? 0 : 2;
}
#else
#define PK_TF(i) do { } while (0)
#endif
int attn_bwd_tc_status(int* status_h, int clear);  // pk_attn_bwd_tc.cu
int attn_fwd_ws_status(int* status_h, int clear);  // pk_attn_fwd_ws.cu
int attn_fwd_row_status(int* status_h, int clear);  // pk_attn_fwd_row.cu
int attn_bwd_ws_status(int* status_h, int clear);  // pk_attn_bwd_ws.cu

namespace tc {

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

int make_tensor_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_inner,
                    int box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return PK_ERR_CUDA;
    }
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
        return PK_ERR_CUDA;
    }
    return PK_OK;
}

}  // namespace tc

using namespace tc;

constexpr int AT_BM = 128;       // rows of the owning tile (queries, or keys in the dK/dV kernel)
constexpr int AT_BN = 128;       // rows of the streamed tile
constexpr int AT_THREADS_TC = 256;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
// Barrier among the 64 threads (warps w and w+4) that share a lane quadrant.
__device__ __forceinline__ void pair_sync(int quad) {
    asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");
}
template <int DK>
__device__ __forceinline__ void load_tile_tma(uint32_t dst, const CUtensorMap* map, int col0, int64_t row, uint32_t bar) {
#pragma unroll
    for (int c = 0; c < DK / 64; ++c) tma_load_2d(dst + c * CHUNK_BYTES, map, col0 + c * 64, static_cast<int32_t>(row), bar);
}
// Writes 32 values as bf16 into 4 consecutive 16-byte units (unit0 .. unit0+3) of a row.
__device__ __forceinline__ void store32_bf16(uint8_t* chunk, int row, int unit0, const float (&v)[32]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack_bf16(v[g * 8 + 0], v[g * 8 + 1]);
        w.y = pack_bf16(v[g * 8 + 2], v[g * 8 + 3]);
        w.z = pack_bf16(v[g * 8 + 4], v[g * 8 + 5]);
        w.w = pack_bf16(v[g * 8 + 6], v[g * 8 + 7]);
        st_swizzled(chunk, row, unit0 + g, w);
    }
}
// 32 fp32 accumulator values of tensor memory -> bf16 -> global (64 contiguous bytes).
__device__ __forceinline__ void store32_global(bf16* dst, const uint32_t (&r)[32], float mul) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack_bf16(__uint_as_float(r[g * 8 + 0]) * mul, __uint_as_float(r[g * 8 + 1]) * mul);
        w.y = pack_bf16(__uint_as_float(r[g * 8 + 2]) * mul, __uint_as_float(r[g * 8 + 3]) * mul);
        w.z = pack_bf16(__uint_as_float(r[g * 8 + 4]) * mul, __uint_as_float(r[g * 8 + 5]) * mul);
        w.w = pack_bf16(__uint_as_float(r[g * 8 + 6]) * mul, __uint_as_float(r[g * 8 + 7]) * mul);
        *reinterpret_cast<uint4*>(dst + g * 8) = w;
    }
}

// ================================================================================ forward
struct FwdParams {
    bf16* out;
    int64_t ldo;
    float* lse;
    int S;
    int Hq, Hkv;
    float scale_log2;  // scale * log2(e)
    int causal;
};

template <int DK>
struct FwdSmem {
    static constexpr int NCH = DK / 64;
    static constexpr int TILE = NCH * (int)CHUNK_BYTES;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = TILE;        // 2 stages
    static constexpr int OFF_V = 3 * TILE;    // 1 stage
    static constexpr int OFF_P = 4 * TILE;    // 2 chunks (128 keys)
    static constexpr int OFF_X = 4 * TILE + 2 * (int)CHUNK_BYTES;  // row max / row sum exchange: 2 x 128 floats
    static constexpr int OFF_BAR = OFF_X + 1024;
    static constexpr int BYTES = OFF_BAR + 128 + 1024;
};

template <int DK>
__global__ void __launch_bounds__(AT_THREADS_TC, DK == 64 ? 2 : 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
    using L = FwdSmem<DK>;
    constexpr uint32_t TMEM_COLS = 256;
    constexpr int OH = DK / 2;  // output columns per thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* bar_q = bars;
    uint64_t* bar_k = bars + 1;  // [2]
    uint64_t* bar_v = bars + 3;
    uint64_t* bar_s = bars + 4;
    uint64_t* bar_o = bars + 5;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(smem + L::OFF_X);  // [2][128]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hf = warp >> 2;
    const int row = quad * 32 + lane;
    const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int64_t seq0 = static_cast<int64_t>(b) * p.S;
    const int q0 = qt * AT_BM;
    const int qi = q0 + row;
    int nkv = (p.S + AT_BN - 1) / AT_BN;
    if (p.causal && qt + 1 < nkv) nkv = qt + 1;

    if (tid == 0) {
        mbar_init(smem_u32(bar_q), 1);
        mbar_init(smem_u32(&bar_k[0]), 1);
        mbar_init(smem_u32(&bar_k[1]), 1);
        mbar_init(smem_u32(bar_v), 1);
        mbar_init(smem_u32(bar_s), 1);
        mbar_init(smem_u32(bar_o), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem + lane_off + hf * 64;        // this thread's 64 score columns
    const uint32_t t_o = tmem + 128 + lane_off + hf * OH;  // this thread's output columns
    const uint32_t sQ = smem_u32(smem + L::OFF_Q), sK0 = smem_u32(smem + L::OFF_K), sV = smem_u32(smem + L::OFF_V);
    const uint32_t sP = smem_u32(smem + L::OFF_P);
    uint8_t* pP = smem + L::OFF_P + hf * CHUNK_BYTES;  // 64 keys = one chunk per half

    const uint32_t idesc_s = idesc_bf16(AT_BN, 0, 0);
    const uint32_t idesc_o = idesc_bf16(DK, 0, 1);

    float o[OH];
#pragma unroll
    for (int i = 0; i < OH; ++i) o[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;  // l: partial row sum over this thread's columns
    bool ok = true;

    // S of tile t: issued one tile ahead of its softmax, so that it runs on the tensor pipe
    // while the CTA is still busy with tile t-1 (only thread 0 calls this).
    auto issue_s = [&](int t) {
        const int st = t & 1;
        if (ok) ok = mbar_wait(smem_u32(&bar_k[st]), (t >> 1) & 1, abort_flag, &g_attn_tc_status);
        if (!ok) return;
        fence_after();
        const uint32_t sK = sK0 + st * L::TILE;
#pragma unroll
        for (int k = 0; k < DK / 16; ++k)
            mma_bf16(tmem, desc_kmajor(sQ, k), desc_kmajor(sK, k), idesc_s, k > 0 ? 1u : 0u);
        commit(smem_u32(bar_s));
    };
    auto load_k = [&](int t) {  // K of tile t into buffer t & 1
        mbar_expect_tx(smem_u32(&bar_k[t & 1]), L::TILE);
        load_tile_tma<DK>(sK0 + (t & 1) * L::TILE, &map_k, hk * DK, seq0 + static_cast<int64_t>(t) * AT_BN, smem_u32(&bar_k[t & 1]));
    };
    if (tid == 0) {
        mbar_expect_tx(smem_u32(bar_q), L::TILE);
        load_tile_tma<DK>(sQ, &map_q, h * DK, seq0 + q0, smem_u32(bar_q));
        load_k(0);
        if (nkv > 1) load_k(1);
        ok = mbar_wait(smem_u32(bar_q), 0, abort_flag, &g_attn_tc_status);
        issue_s(0);
    }

    for (int j = 0; j < nkv; ++j) {
        const int kv0 = j * AT_BN;
        PK_TF(0);
        if (tid == 0) {
            // V_j: the single V buffer is free, P.V of the previous tile was waited for below
            mbar_expect_tx(smem_u32(bar_v), L::TILE);
            load_tile_tma<DK>(sV, &map_v, hk * DK, seq0 + kv0, smem_u32(bar_v));
            PK_TF(1);
        }
        if (!mbar_wait(smem_u32(bar_s), j & 1, abort_flag, &g_attn_tc_status)) ok = false;
        PK_TF(2);
        fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld32(t_s, r0);
        tmem_ld32(t_s + 32, r1);
        tmem_wait_ld();
        PK_TF(3);
        const bool need_mask = (p.causal && kv0 + AT_BN - 1 > q0) || (kv0 + AT_BN > p.S);
        if (need_mask) {
            const int key0 = kv0 + hf * 64;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                if (key0 + e >= p.S || (p.causal && key0 + e > qi)) r0[e] = 0xff800000u;            // -inf
                if (key0 + 32 + e >= p.S || (p.causal && key0 + 32 + e > qi)) r1[e] = 0xff800000u;
            }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, fmaxf(__uint_as_float(r0[e]), __uint_as_float(r1[e])));
        xch[hf * 128 + row] = mx;
        pair_sync(quad);
        PK_TF(4);
        mx = fmaxf(mx, xch[(hf ^ 1) * 128 + row]);
        const float m_new = fmaxf(m, mx * p.scale_log2);
        const float corr = m == -INFINITY ? 0.0f : exp2f(m - m_new);
        // m_new is finite for every tile a row takes part in (its diagonal key is visible)
        float sum = 0.0f;
        const float neg_m = -m_new;
#pragma unroll
        for (int g = 0; g < 8; ++g) {  // 8 keys -> one 16-byte unit of the P operand tile
            float pe[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t raw = g < 4 ? r0[g * 8 + e] : r1[(g - 4) * 8 + e];
                pe[e] = ex2_approx(fmaf(__uint_as_float(raw), p.scale_log2, neg_m));  // FFMA + MUFU
                sum += pe[e];
            }
            uint4 w;
            w.x = pack_bf16(pe[0], pe[1]);
            w.y = pack_bf16(pe[2], pe[3]);
            w.z = pack_bf16(pe[4], pe[5]);
            w.w = pack_bf16(pe[6], pe[7]);
            st_swizzled(pP, row, g, w);
        }
        l = l * corr + sum;
        PK_TF(5);
        fence_async_smem();
        fence_before();
        if (__syncthreads_or(!ok)) {  // CTA-uniform exit as soon as any thread's wait gave up
            ok = false;
            break;
        }
        if (tid == 0) {
            ok = mbar_wait(smem_u32(bar_v), j & 1, abort_flag, &g_attn_tc_status);
            if (ok) {
                fence_after();
#pragma unroll
                for (int k = 0; k < AT_BN / 16; ++k)
                    mma_bf16(tmem + 128, desc_kmajor(sP, k), desc_mnmajor(sV, k), idesc_o, k > 0 ? 1u : 0u);
                commit(smem_u32(bar_o));
                if (j + 1 < nkv) {
                    issue_s(j + 1);                   // S of tile j was consumed before the barrier above
                    if (ok && j + 2 < nkv) load_k(j + 2);  // its buffer held K_j, read by S_j (complete)
                }
                PK_TF(6);
            }
        }
        if (!mbar_wait(smem_u32(bar_o), j & 1, abort_flag, &g_attn_tc_status)) ok = false;
        PK_TF(7);
        fence_after();
#pragma unroll
        for (int ch = 0; ch < OH / 32; ++ch) {
            uint32_t r[32];
            tmem_ld32(t_o + ch * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[ch * 32 + e] = o[ch * 32 + e] * corr + __uint_as_float(r[e]);
        }
        m = m_new;
        PK_TF(8);
    }

    // total row sum = the two halves' partial sums
    __syncthreads();
    xch[hf * 128 + row] = l;
    pair_sync(quad);
    l += xch[(hf ^ 1) * 128 + row];
    if (ok && qi < p.S) {
        const float inv = 1.0f / l;
        bf16* dst = p.out + (seq0 + qi) * p.ldo + h * DK + hf * OH;
#pragma unroll
        for (int g = 0; g < OH / 8; ++g) {
            uint4 v;
            v.x = pack_bf16(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv);
            v.y = pack_bf16(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
            v.z = pack_bf16(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv);
            v.w = pack_bf16(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + g * 8) = v;
        }
        if (hf == 0) p.lse[(seq0 + qi) * p.Hq + h] = (m + log2f(l)) * LN2;
    }
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

template <int DK>
static int launch_fwd(cudaStream_t st, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                      const FwdParams& p, int64_t B) {
    using L = FwdSmem<DK>;
    auto kern = attn_fwd_tc_kernel<DK>;
    static bool attr = false;
    if (!attr) {
        PK_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES));
        attr = true;
    }
    dim3 grid(static_cast<unsigned>((p.S + AT_BM - 1) / AT_BM), p.Hq, static_cast<unsigned>(B));
    kern<<<grid, AT_THREADS_TC, L::BYTES, st>>>(mq, mk, mv, p);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

// ---- entry points used by the dispatcher in pk_attn_simt.cu ------------------------------
int attn_tc_supported(int dtype, int dk, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                      int64_t ldv, const void* out, int64_t ldo, int64_t B, int64_t S) {
    if (dtype != PK_BF16 || (dk != 64 && dk != 128)) return 0;
    if (ldq % 8 || ldk % 8 || ldv % 8 || ldo % 8) return 0;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return 0;
    if (B * S >= (int64_t(1) << 31) || S >= (int64_t(1) << 30)) return 0;
    return 1;
}

int attn_tc_fwd(cudaStream_t st, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                void* out, int64_t ldo, float* lse, int64_t B, int64_t S, int Hq, int Hkv, int dk, float scale,
                int causal) {
    CUtensorMap mq, mk, mv;
    const int64_t R = B * S;
    int rc = make_tensor_map(&mq, q, static_cast<int64_t>(Hq) * dk, R, ldq, 64, AT_BM);
    if (rc != PK_OK) return rc;
    rc = make_tensor_map(&mk, k, static_cast<int64_t>(Hkv) * dk, R, ldk, 64, AT_BN);
    if (rc != PK_OK) return rc;
    rc = make_tensor_map(&mv, v, static_cast<int64_t>(Hkv) * dk, R, ldv, 64, AT_BN);
    if (rc != PK_OK) return rc;
    FwdParams p;
    p.out = static_cast<bf16*>(out);
    p.ldo = ldo;
    p.lse = lse;
    p.S = static_cast<int>(S);
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale_log2 = scale * LOG2E;
    p.causal = causal;
    return dk == 64 ? launch_fwd<64>(st, mq, mk, mv, p, B) : launch_fwd<128>(st, mq, mk, mv, p, B);
}

}  // namespace pk

extern "C" {

int pk_attn_tc_status(int* status_h, int clear) {
    PK_REQUIRE(status_h != nullptr, "null output");
    PK_CHECK_CUDA(cudaDeviceSynchronize());
    PK_CHECK_CUDA(cudaMemcpyFromSymbol(status_h, pk::g_attn_tc_status, sizeof(int)));
    if (clear) {
        const int zero = 0;
        PK_CHECK_CUDA(cudaMemcpyToSymbol(pk::g_attn_tc_status, &zero, sizeof(int)));
    }
    int bwd = 0;  // the backward kernels (pk_attn_bwd_tc.cu) keep their own word
    const int rc = pk::attn_bwd_tc_status(&bwd, clear);
    if (rc != PK_OK) return rc;
    *status_h |= bwd;
    int ws = 0;
    const int rc2 = pk::attn_fwd_ws_status(&ws, clear);
    if (rc2 != PK_OK) return rc2;
    *status_h |= ws;
    int row = 0;
    const int rc4 = pk::attn_fwd_row_status(&row, clear);
    if (rc4 != PK_OK) return rc4;
    *status_h |= row;
    int wsb = 0;
    const int rc3 = pk::attn_bwd_ws_status(&wsb, clear);
    if (rc3 != PK_OK) return rc3;
    *status_h |= wsb;
    return PK_OK;
}

}  // extern "C"
