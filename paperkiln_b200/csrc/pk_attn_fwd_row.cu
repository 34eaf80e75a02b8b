// Flash attention forward, warp-specialised, one thread per query row (bf16 operands, fp32
// accumulation in tensor memory), head_dim 64 or 128, causal or full, grouped-query head mapping,
// B stacked sequences. Same schedule as pk_attn_fwd_ws.cu -- one CTA per SM works on 256
// consecutive queries of one head as two 128-row slots that take turns on the tensor pipe -- but
// with four softmax warps per slot instead of eight:
//   warps 0-3    softmax of slot 0     warp w reads tensor-memory lanes 32 (w & 3) ..; a thread
//   warps 4-7    softmax of slot 1     owns ONE row and all 128 score columns of a key tile
//   warp 8       issues every tcgen05.mma (one thread)
//   warp 9       issues every TMA load (one thread); warps 10-11 idle. This warpgroup hands most
//                of its registers to the softmax warps (setmaxnreg: 232 registers each, enough
//                to hold a whole score row).
// A row's maximum and sum therefore need no exchange between threads: no named barriers, no
// shared-memory hand-over, half as many warps competing for issue slots, and the per-tile
// bookkeeping is paid once per 128 scores instead of once per 64.
// Per slot and 128-key tile (as in pk_attn_fwd_ws.cu):
//   S = Q K^T            smem operands (128B swizzle), fp32 result in tensor memory
//   p = exp2(S c - m)    in registers; P goes back to TENSOR MEMORY as packed bf16 (32 scores at
//                        a time) and is the A operand of the next MMA
//   O += P V             V read MN-major; O stays in tensor memory for the whole key loop and is
//                        rescaled in place only when a row maximum grew by more than 2^8
// Everything a thread does depends only on the data, so results are reproducible bit for bit.
// Every mbarrier wait is bounded (status word, no trap).
//
// Semantics: ops::fused_attention of the reference (src/ops.cpp:863-934) applied per head.
#include "pk_tc.cuh"

namespace pk {

PK_DEFINE_WAITCTL(attn_fwd_row)

using namespace tc;

namespace {

constexpr int WS_BM = 128;                   // rows per slot
constexpr int WS_BN = 128;                   // keys per tile
constexpr int WS_SOFT_WARPS = 8;
constexpr int WS_THREADS = (WS_SOFT_WARPS + 4) * 32;   // + one control warpgroup: MMA warp, TMA warp, 2 idle
constexpr float WS_LOG2E = 1.4426950408889634f;
constexpr float WS_LN2 = 0.6931471805599453f;
constexpr float WS_RESCALE_GAP = 8.0f;       // log2 units
constexpr int WS_REGS_SOFT = 232;            // registers per softmax thread after setmaxnreg (literal in the asm below)
constexpr int WS_REGS_CTRL = 40;             // registers per control thread

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
// 128 rows of one sequence starting at position `pos`: the tensor maps are three-dimensional
// (feature, position, sequence), so a tile that runs past the end of its sequence is filled with
// zeros there instead of reading the next sequence's rows (0 x Inf from a neighbour would
// otherwise reach this sequence's output through P.V).
template <int DK>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, int col0, int pos, int seq, uint32_t bar) {
#pragma unroll
    for (int c = 0; c < DK / 64; ++c) tma_load_3d(dst + c * CHUNK_BYTES, map, col0 + c * 64, pos, seq, bar);
}

struct RowParams {
    bf16* out;
    int64_t ldo;
    float* lse;
    int S;
    int Hq, Hkv;
    float scale_log2;  // scale * log2(e)
    int causal;
};

template <int DK>
struct RowLayout {
    static constexpr int NCH = DK / 64;
    static constexpr int TILE = NCH * (int)CHUNK_BYTES;   // 128 rows x DK bf16
    static constexpr int NS = DK == 64 ? 3 : 2;           // K and V stages
    static constexpr int OFF_Q = 0;                       // 2 slots
    static constexpr int OFF_K = 2 * TILE;
    static constexpr int OFF_V = OFF_K + NS * TILE;
    static constexpr int OFF_BAR = OFF_V + NS * TILE;
    static constexpr int BYTES = OFF_BAR + 256 + 1024;
    // tensor memory columns
    static constexpr int T_S = 0;                          // + slot * 128
    static constexpr int T_O = 256;                        // + slot * DK
    static constexpr int T_P = DK == 64 ? 384 : 0;         // + slot * (DK == 64 ? 64 : 128); aliases S when DK = 128
    static constexpr int P_PITCH = DK == 64 ? 64 : 128;
};

// Which of the 16 score pairs of every 32-score group take their exponential on the FMA pipe
// (ex2_fma_pair) instead of the special-function unit: bit i of the mask = second pair of
// iteration i. 0x55 moves 4 of 16 pairs (25 %), 0xDB 6 (37.5 %), 0xFF 8 (50 %).
template <int DK, int POLY_MASK>
__global__ void __launch_bounds__(WS_THREADS, 1)
attn_fwd_row_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const RowParams p) {
    using L = RowLayout<DK>;
    constexpr int NS = L::NS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* q_full = bars;            // [2]
    uint64_t* k_full = bars + 2;        // [NS]
    uint64_t* k_empty = bars + 5;       // [NS]
    uint64_t* v_full = bars + 8;        // [NS]
    uint64_t* v_empty = bars + 11;      // [NS]
    uint64_t* s_full = bars + 14;       // [2]
    uint64_t* p_full = bars + 16;       // [2]
    uint64_t* o_done = bars + 18;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int64_t seq0 = static_cast<int64_t>(b) * p.S;
    const int nkv_tot = (p.S + WS_BN - 1) / WS_BN;
    int nkv[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) nkv[s] = p.causal ? min(2 * qt + s + 1, nkv_tot) : nkv_tot;
    const int nkv_max = nkv[1];

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&q_full[i]), 1);
            mbar_init(smem_u32(&s_full[i]), 1);
            mbar_init(smem_u32(&p_full[i]), WS_SOFT_WARPS / 2);
            mbar_init(smem_u32(&o_done[i]), 1);
        }
        for (int i = 0; i < NS; ++i) {
            mbar_init(smem_u32(&k_full[i]), 1);
            mbar_init(smem_u32(&k_empty[i]), 1);
            mbar_init(smem_u32(&v_full[i]), 1);
            mbar_init(smem_u32(&v_empty[i]), 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sQ = smem_u32(smem + L::OFF_Q), sK = smem_u32(smem + L::OFF_K), sV = smem_u32(smem + L::OFF_V);

    // Register budget: setmaxnreg moves registers inside the pool the CTA was LAUNCHED with
    // (threads x registers per thread of the compiled kernel), not the SM's whole file; an
    // increase that the pool cannot cover would wait forever. The control warpgroup shrinks to
    // WS_REGS_CTRL and the softmax warps grow to WS_REGS_SOFT; launch_row() refuses to launch
    // unless 256 * WS_REGS_SOFT + 128 * WS_REGS_CTRL fits the launch allocation (384 threads x 168).
    // setmaxnreg is a warpgroup-wide aligned instruction: all four warps of the control
    // warpgroup execute the one instance below before they part ways.
    if (warp >= WS_SOFT_WARPS) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
      if (warp == WS_SOFT_WARPS + 1) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            for (int s = 0; s < 2; ++s) {
                mbar_expect_tx(smem_u32(&q_full[s]), L::TILE);
                load_tile<DK>(sQ + s * L::TILE, &map_q, h * DK, (2 * qt + s) * WS_BM, b, smem_u32(&q_full[s]));
            }
            for (int j = 0; j < nkv_max && ok; ++j) {
                const int st = j % NS, n = j / NS;
                const int pos = j * WS_BN;
                if (n > 0) ok = mbar_wait(smem_u32(&k_empty[st]), (n - 1) & 1, abort_flag, &g_attn_fwd_row_ctl);
                if (!ok) break;
                mbar_expect_tx(smem_u32(&k_full[st]), L::TILE);
                load_tile<DK>(sK + st * L::TILE, &map_k, hk * DK, pos, b, smem_u32(&k_full[st]));
                if (n > 0) ok = mbar_wait(smem_u32(&v_empty[st]), (n - 1) & 1, abort_flag, &g_attn_fwd_row_ctl);
                if (!ok) break;
                mbar_expect_tx(smem_u32(&v_full[st]), L::TILE);
                load_tile<DK>(sV + st * L::TILE, &map_v, hk * DK, pos, b, smem_u32(&v_full[st]));
            }
        }
        __syncwarp();
      } else if (warp == WS_SOFT_WARPS) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = idesc_bf16(WS_BN, 0, 0);
            const uint32_t idesc_o = idesc_bf16(DK, 0, 1);
            bool ok = true;
            const uint32_t q_lo0 = desc_lo_kmajor(sQ), k_lo0 = desc_lo_kmajor(sK), v_lo0 = desc_lo_mnmajor(sV);
            auto issue_s = [&](int s, int j) {  // S_s(j) = Q_s K_j^T
                const uint32_t q_lo = q_lo0 + s * (L::TILE >> 4), k_lo = k_lo0 + (j % NS) * (L::TILE >> 4);
                const uint32_t d = tmem + L::T_S + s * 128;
#pragma unroll
                for (int k = 0; k < DK / 16; ++k) mma_ss(d, q_lo + kstep_kmajor(k), k_lo + kstep_kmajor(k), idesc_s, k > 0 ? 1u : 0u);
                commit(smem_u32(&s_full[s]));
            };
            ok = mbar_wait(smem_u32(&q_full[0]), 0, abort_flag, &g_attn_fwd_row_ctl);
            if (ok) ok = mbar_wait(smem_u32(&q_full[1]), 0, abort_flag, &g_attn_fwd_row_ctl);
            if (ok) ok = mbar_wait(smem_u32(&k_full[0]), 0, abort_flag, &g_attn_fwd_row_ctl);
            if (ok) {
                fence_after();
                issue_s(0, 0);
                issue_s(1, 0);
                commit(smem_u32(&k_empty[0]));
            }
            for (int j = 0; j < nkv_max && ok; ++j) {
                const int st = j % NS;
                bool v_ready = false, k_ready = false;
#pragma unroll 1
                for (int s = 0; s < 2; ++s) {
                    if (j >= nkv[s] || !ok) continue;
                    ok = mbar_wait(smem_u32(&p_full[s]), j & 1, abort_flag, &g_attn_fwd_row_ctl);
                    if (ok && !v_ready) {
                        ok = mbar_wait(smem_u32(&v_full[st]), (j / NS) & 1, abort_flag, &g_attn_fwd_row_ctl);
                        v_ready = true;
                    }
                    if (!ok) break;
                    fence_after();
                    const uint32_t v_lo = v_lo0 + st * (L::TILE >> 4);
                    const uint32_t d = tmem + L::T_O + s * DK, a = tmem + L::T_P + s * L::P_PITCH;
#pragma unroll
                    for (int k = 0; k < WS_BN / 16; ++k)
                        mma_ts(d, a + k * 8, v_lo + kstep_mnmajor(k), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                    if (j + 1 < nkv[s]) {
                        if (!k_ready) {
                            ok = mbar_wait(smem_u32(&k_full[(j + 1) % NS]), ((j + 1) / NS) & 1, abort_flag, &g_attn_fwd_row_ctl);
                            k_ready = true;
                            if (!ok) break;
                            fence_after();
                        }
                        issue_s(s, j + 1);
                    } else {
                        commit(smem_u32(&o_done[s]));
                    }
                }
                if (!ok) break;
                commit(smem_u32(&v_empty[st]));                              // V_j free once P.V of both slots is done
                if (j + 1 < nkv_max) commit(smem_u32(&k_empty[(j + 1) % NS]));  // K_{j+1}: after its last S
            }
        }
        __syncwarp();
      }
    } else {
        // ------------------------------------------------------------------ softmax warps
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int s = warp >> 2;              // slot
        const int quad = warp & 3;            // tensor-memory lane quadrant = warp index mod 4
        const int row = quad * 32 + lane;     // this thread owns one query row, all 128 score columns
        const int q0 = (2 * qt + s) * WS_BM;
        const int qi = q0 + row;
        const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_s = tmem + lane_off + L::T_S + s * 128;
        const uint32_t t_p = tmem + lane_off + L::T_P + s * L::P_PITCH;   // 128 keys as 64 packed columns
        const uint32_t t_o = tmem + lane_off + L::T_O + s * DK;
        const int my_nkv = nkv[s];

        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < my_nkv; ++j) {
            const int kv0 = j * WS_BN;
            ok = mbar_wait(smem_u32(&s_full[s]), j & 1, abort_flag, &g_attn_fwd_row_ctl);
            ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the tensor-memory accesses below are warp-wide
            if (!ok) break;                    // nobody waits for this warp at a meeting point
            fence_after();
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, r[c]);
            tmem_wait_ld();
            const bool need_mask = (p.causal && kv0 + WS_BN - 1 > q0) || (kv0 + WS_BN > p.S);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int key = kv0 + c * 32 + e;
                        if (key >= p.S || (p.causal && key > qi)) r[c][e] = 0xff800000u;  // -inf
                    }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                mx0 = fmax3(mx0, __uint_as_float(r[0][e]), __uint_as_float(r[0][e + 1]));
                mx1 = fmax3(mx1, __uint_as_float(r[1][e]), __uint_as_float(r[1][e + 1]));
                mx2 = fmax3(mx2, __uint_as_float(r[2][e]), __uint_as_float(r[2][e + 1]));
                mx3 = fmax3(mx3, __uint_as_float(r[3][e]), __uint_as_float(r[3][e + 1]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            // Row maximum in log2 units. Every row sees at least one key in its first tile
            // (key 0), so cand is finite from j = 0 on.
            const float cand = fmaxf(m, mx * p.scale_log2);
            if (j == 0) {
                m = cand;
            } else {
                const bool grow = cand > m + WS_RESCALE_GAP;
                if (__any_sync(0xffffffffu, grow)) {
                    // s_full(j) also covers P.V of tile j-1 (issued before S(j)): O is quiescent
                    const float f = grow ? ex2_approx(m - cand) : 1.0f;
                    if (grow) m = cand;
                    l *= f;
#pragma unroll 1
                    for (int ch = 0; ch < DK / 16; ++ch) {
                        uint32_t o[16];
                        tmem_ld16(t_o + ch * 16, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                        tmem_st16(t_o + ch * 16, o);
                    }
                }
            }
            const float neg_m = -m;
            const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), nm2 = f2_pack(neg_m, neg_m);
            uint64_t sum_a = f2_pack(0.0f, 0.0f), sum_b = sum_a;
            // 32 scores -> 16 packed columns at a time; each quarter is stored as soon as it is ready
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 16; e += 2) {
                    float xa0, xa1, xb0, xb1;
                    f2_unpack(f2_fma(f2_pack_bits(r[c][2 * e], r[c][2 * e + 1]), sc2, nm2), xa0, xa1);
                    f2_unpack(f2_fma(f2_pack_bits(r[c][2 * e + 2], r[c][2 * e + 3]), sc2, nm2), xb0, xb1);
                    const float a0 = ex2_approx(xa0), a1 = ex2_approx(xa1);
                    float b0, b1;
                    if ((POLY_MASK >> (e >> 1)) & 1) {
                        ex2_fma_pair(f2_pack(xb0, xb1), b0, b1);
                    } else {
                        b0 = ex2_approx(xb0);
                        b1 = ex2_approx(xb1);
                    }
                    sum_a = f2_add(sum_a, f2_pack(a0, a1));
                    sum_b = f2_add(sum_b, f2_pack(b0, b1));
                    pk[e] = pack2(a0, a1);
                    pk[e + 1] = pack2(b0, b1);
                }
                tmem_st16(t_p + c * 16, pk);
            }
            {
                float s0, s1, s2, s3;
                f2_unpack(sum_a, s0, s1);
                f2_unpack(sum_b, s2, s3);
                l += (s0 + s1) + (s2 + s3);
            }
            tmem_wait_st();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[s]));
        }

        if (ok) ok = mbar_wait(smem_u32(&o_done[s]), 0, abort_flag, &g_attn_fwd_row_ctl);
        ok = __all_sync(0xffffffffu, ok);
        fence_after();
        if (ok) {
            const float inv = 1.0f / l;
            bf16* dst = p.out + (seq0 + qi) * p.ldo + h * DK;
#pragma unroll 1
            for (int ch = 0; ch < DK / 32; ++ch) {
                uint32_t o[32];
                tmem_ld32(t_o + ch * 32, o);
                tmem_wait_ld();
                if (qi < p.S) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 v;
                        v.x = pack2(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
                        v.y = pack2(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
                        v.z = pack2(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
                        v.w = pack2(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + ch * 32 + g * 8) = v;
                    }
                }
            }
            if (qi < p.S) p.lse[(seq0 + qi) * p.Hq + h] = (m + log2f(l)) * WS_LN2;
        }
    }

    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem, 512);
    }
}

template <int DK, int POLY_MASK>
int launch_row(cudaStream_t st, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const RowParams& p,
              int64_t B) {
    using L = RowLayout<DK>;
    auto kern = attn_fwd_row_kernel<DK, POLY_MASK>;
    static bool attr = false;
    if (!attr) {
        cudaFuncAttributes fa;
        PK_CHECK_CUDA(cudaFuncGetAttributes(&fa, kern));
        PK_REQUIRE(fa.numRegs * WS_THREADS >= WS_SOFT_WARPS * 32 * WS_REGS_SOFT + 4 * 32 * WS_REGS_CTRL,
                   "attention forward: the kernel's launch register allocation cannot cover its setmaxnreg plan");
        PK_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES));
        attr = true;
    }
    dim3 grid(static_cast<unsigned>((p.S + 2 * WS_BM - 1) / (2 * WS_BM)), p.Hq, static_cast<unsigned>(B));
    kern<<<grid, WS_THREADS, L::BYTES, st>>>(mq, mk, mv, p);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

// Measured at head_dim 64, B 8, S 4096 (TFLOP/s): no pair on the FMA pipe 515, 4 of 16 pairs 526,
// 6 of 16 520, 8 of 16 516; at head_dim 128 it is 802 / 793 / 775 / 748. The softmax warps are
// bound by their own instruction stream about as much as by the special-function unit, so only
// the smallest share pays, and only at head_dim 64.
constexpr int POLY_MASK_64 = 0x55, POLY_MASK_128 = 0;
}  // namespace

int attn_fwd_row(cudaStream_t st, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                void* out, int64_t ldo, float* lse, int64_t B, int64_t S, int Hq, int Hkv, int dk, float scale,
                int causal) {
    CUtensorMap mq, mk, mv;
    int rc = make_tensor_map_3d(&mq, q, static_cast<int64_t>(Hq) * dk, S, B, ldq, 64, WS_BM);
    if (rc != PK_OK) return rc;
    rc = make_tensor_map_3d(&mk, k, static_cast<int64_t>(Hkv) * dk, S, B, ldk, 64, WS_BN);
    if (rc != PK_OK) return rc;
    rc = make_tensor_map_3d(&mv, v, static_cast<int64_t>(Hkv) * dk, S, B, ldv, 64, WS_BN);
    if (rc != PK_OK) return rc;
    RowParams p;
    p.out = static_cast<bf16*>(out);
    p.ldo = ldo;
    p.lse = lse;
    p.S = static_cast<int>(S);
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale_log2 = scale * WS_LOG2E;
    p.causal = causal;
    return dk == 64 ? launch_row<64, POLY_MASK_64>(st, mq, mk, mv, p, B) : launch_row<128, POLY_MASK_128>(st, mq, mk, mv, p, B);
}


}  // namespace pk
