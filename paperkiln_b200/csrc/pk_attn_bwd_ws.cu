// Flash-attention backward, warp-specialised (bf16 operands, fp32 accumulation in tensor
// memory), head_dim 64 or 128, causal or full, grouped-query head mapping.
//
// Two kernels, no atomics: every gradient element is owned by one CTA and summed in a fixed
// order, so the result is reproducible bit for bit.
//
//   dQ kernel     CTA = (128-query tile, head, sequence); streams key tiles of 64:
//                   S = Q K^T, dP = dO V^T          [128 q x 64 keys], tensor memory, 3 buffers
//                   dS = P (dP - delta) scale        packed bf16 over the thread's own S columns
//                   dQ += dS K                        A operand from tensor memory, K MN-major
//   dK/dV kernel  CTA = (128-key tile, kv head, sequence); streams 64-query tiles of every
//                 query head of the group, in the transposed form (rows are keys):
//                   S^T = K Q^T, dP^T = V dO^T       [128 keys x 64 q], tensor memory, 3 buffers
//                                                     (2 at head_dim 128, where dV and dK need 256 columns)
//                   P^T, dS^T                         packed bf16 over the thread's own columns
//                   dV += P^T dO,  dK += dS^T Q      A from tensor memory, dO / Q MN-major
//   P is recomputed from the saved log-sum-exp: p = exp2(s c - lse log2 e).
//
// Roles in a CTA of 640 threads (one CTA per SM):
//   warps 0-7    element-wise work on the even streamed tiles
//   warps 8-15   the same on the odd tiles; warps w and w+4 of a group share lane quadrant
//                w & 3 and split the 64 columns. Tile t lives in score buffer t mod 3: the
//                scores of tile t+3 are issued as soon as tile t is finished, so in steady state
//                a group finds its next tile's scores already computed
//   warps 16, 18, 19  issue the tcgen05.mma instructions, one kind each (gradient products /
//                S / dP): the scores of tile t+2 are computed while the other group still
//                works on tile t+1. An issuing thread cannot run ahead of the tensor pipe, so
//                its barrier waits and address arithmetic would leave the pipe idle; with three
//                issuers the gaps of one are filled by the others' MMAs. Every accumulator
//                has one owner and a fixed order.
//   warp 17      issues every TMA / bulk load
// Nothing passes through shared memory on the way from the scores to the gradient MMAs.
// Per-query statistics (-lse log2 e and -delta scale) are kept head-major and padded to a
// multiple of 64 queries, so that the dK/dV kernel fetches the 64 values of a streamed tile
// with one bulk copy each and padding queries contribute p = 0 without a bounds test.
// Every mbarrier wait is bounded (status word, no trap).
//
// Formulas: backward of ops::fused_attention in the reference (src/ops.cpp:903-933).
#include "pk_tc.cuh"

namespace pk {

PK_DEFINE_WAITCTL(attn_bwd_ws)

using namespace tc;

namespace {

constexpr int BW_ROWS = 128;   // rows of the owning tile
constexpr int BW_COLS = 64;    // rows of the streamed tile = columns of a score tile
constexpr int BW_SOFT_WARPS = 16;
constexpr int BW_THREADS = (BW_SOFT_WARPS + 4) * 32;
constexpr int BW_REGS_SOFT = 112;  // literals in the setmaxnreg instructions below
constexpr int BW_REGS_CTRL = 32;
constexpr float BW_LOG2E = 1.4426950408889634f;
constexpr uint32_t CH128 = 16384;  // chunk pitch of a 128-row tile
constexpr uint32_t CH64 = 8192;    // chunk pitch of a 64-row tile

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
// Rows pos.. of sequence `seq` (three-dimensional tensor maps: feature, position, sequence). Rows
// past the end of the sequence read as zero, never as the next sequence's rows: P = 0 or dS = 0
// times an Inf of a neighbour would otherwise leak NaN into this sequence's gradients.
template <int DK>
__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* map, int col0, int pos, int seq, uint32_t bar,
                                         uint32_t chunk_pitch) {
#pragma unroll
    for (int c = 0; c < DK / 64; ++c) tma_load_3d(dst + c * chunk_pitch, map, col0 + c * 64, pos, seq, bar);
}
__device__ __forceinline__ void st16_global(bf16* dst, const uint32_t (&r)[16]) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        uint4 w;
        w.x = pack2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
        w.y = pack2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
        w.z = pack2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
        w.w = pack2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
        *reinterpret_cast<uint4*>(dst + g * 8) = w;
    }
}

// stats[0][bh][s] = -lse log2 e (-inf for padding), stats[1][bh][s] = -delta scale (0 for padding);
// delta[row, h] = sum_c dout[row, h, c] out[row, h, c]. dk / 8 lanes per (position, head), 16 bytes
// of out and of dout per lane; a warp covers consecutive heads of one position, i.e. contiguous memory.
template <int DK>
__global__ void __launch_bounds__(256)
attn_bwd_stats_kernel(const bf16* __restrict__ out, int64_t ldo, const bf16* __restrict__ dout, int64_t lddo,
                      const float* __restrict__ lse, float* __restrict__ lneg, float* __restrict__ dneg, int64_t B,
                      int64_t S, int64_t S_pad, int Hq, float scale) {
    constexpr int LPH = DK / 8;              // lanes per (position, head): 8 or 16
    constexpr int HPW = 32 / LPH;            // heads per warp and iteration
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPH, li = lane % LPH;
    const int groups = (Hq + HPW - 1) / HPW;  // warp iterations per position
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (w >= B * S_pad * groups) return;
    const int g = static_cast<int>(w % groups);
    const int64_t s = (w / groups) % S_pad, b = w / groups / S_pad;
    const int h = g * HPW + sub;
    const bool live = h < Hq;
    float acc = 0.0f;
    if (live && s < S) {
        const int64_t row = b * S + s;
        float a[8], d[8];
        Vec<bf16>::load(out + row * ldo + h * DK + li * 8, a);
        Vec<bf16>::load(dout + row * lddo + h * DK + li * 8, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += a[e] * d[e];
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (live && li == 0) {
        const int64_t o = (b * Hq + h) * S_pad + s;
        if (s < S) {
            lneg[o] = -lse[(b * S + s) * Hq + h] * BW_LOG2E;
            dneg[o] = -acc * scale;
        } else {
            lneg[o] = -INFINITY;
            dneg[o] = 0.0f;
        }
    }
}

struct WsBwdParams {
    bf16* dq;
    int64_t lddq;
    bf16* dk;
    int64_t lddk;
    bf16* dv;
    int64_t lddv;
    const float* lneg;  // [B*Hq][S_pad]
    const float* dneg;
    int S, S_pad;
    int Hq, Hkv;
    float scale, scale_log2;
    int causal;
};

// ------------------------------------------------------------------------------ dQ
template <int DK>
struct DqLayout {
    static constexpr int TILEQ = (DK / 64) * (int)CH128;  // Q, dO: 128 rows
    static constexpr int TILEK = (DK / 64) * (int)CH64;   // K_j, V_j: 64 rows
    // K/V stages. A stage is held from the scores of tile j (issued two tiles ahead) until dQ of
    // tile j is done, i.e. for three tiles; the rest is how far the TMA producer runs ahead, and
    // one tile of lead is not enough to cover the latency of a load.
    static constexpr int NS = DK == 64 ? 8 : 5;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_DO = TILEQ;
    static constexpr int OFF_K = 2 * TILEQ;
    static constexpr int OFF_V = OFF_K + NS * TILEK;
    static constexpr int OFF_BAR = OFF_V + NS * TILEK;
    static constexpr int BYTES = OFF_BAR + 256 + 1024;
    // Score buffers in tensor memory: buffer b holds S at b*128 and dP at b*128 + 64. With three of
    // them the scores of tile j+3 are issued as soon as tile j is finished, so an element-wise group
    // never waits for the tensor pipe in steady state. dS is packed over the first 16 of each
    // thread's own 32 S columns.
    static constexpr int NB = 3;
    static constexpr int T_DQ = NB * 128;
};

template <int DK>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_ws_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                      const WsBwdParams p) {
    using L = DqLayout<DK>;
    constexpr int NS = L::NS;
    constexpr int NB = L::NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* qdo_full = bars;            // Q and dO
    uint64_t* kv_full = bars + 1;         // [NS]
    uint64_t* kv_empty = kv_full + NS;    // [NS]
    uint64_t* s_full = kv_empty + NS;     // [NB]
    uint64_t* ds_full = s_full + NB;      // [NB]
    uint64_t* dq_done = ds_full + NB;     // [NB]  dQ of a buffer's tile complete: the buffer may be overwritten
    uint64_t* done = dq_done + NB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int64_t seq0 = static_cast<int64_t>(b) * p.S;
    const int q0 = qt * BW_ROWS;
    int nkv = (p.S + BW_COLS - 1) / BW_COLS;
    if (p.causal && 2 * (qt + 1) < nkv) nkv = 2 * (qt + 1);

    if (tid == 0) {
        mbar_init(smem_u32(qdo_full), 1);
        for (int i = 0; i < NS; ++i) {
            mbar_init(smem_u32(&kv_full[i]), 1);
            mbar_init(smem_u32(&kv_empty[i]), 1);
        }
        for (int i = 0; i < NB; ++i) {
            mbar_init(smem_u32(&s_full[i]), 2);   // S issuer + dP issuer
            mbar_init(smem_u32(&ds_full[i]), BW_SOFT_WARPS / 2);
            mbar_init(smem_u32(&dq_done[i]), 1);
        }
        mbar_init(smem_u32(done), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sQ = smem_u32(smem + L::OFF_Q), sDO = smem_u32(smem + L::OFF_DO);
    const uint32_t sK = smem_u32(smem + L::OFF_K), sV = smem_u32(smem + L::OFF_V);

    // setmaxnreg moves registers inside the pool the CTA was launched with; the launcher checks
    // that 512 * BW_REGS_SOFT + 128 * BW_REGS_CTRL fits it. One instance per warpgroup.
    if (warp >= BW_SOFT_WARPS) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
      if (warp == BW_SOFT_WARPS + 1) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(smem_u32(qdo_full), 2 * L::TILEQ);
            tma_tile<DK>(sQ, &map_q, h * DK, q0, b, smem_u32(qdo_full), CH128);
            tma_tile<DK>(sDO, &map_do, h * DK, q0, b, smem_u32(qdo_full), CH128);
            for (int j = 0; j < nkv; ++j) {
                const int st = j % NS, n = j / NS;
                if (n > 0) ok = mbar_wait(smem_u32(&kv_empty[st]), (n - 1) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (!ok) break;
                const int pos = j * BW_COLS;
                mbar_expect_tx(smem_u32(&kv_full[st]), 2 * L::TILEK);
                tma_tile<DK>(sK + st * L::TILEK, &map_k, hk * DK, pos, b, smem_u32(&kv_full[st]), CH64);
                tma_tile<DK>(sV + st * L::TILEK, &map_v, hk * DK, pos, b, smem_u32(&kv_full[st]), CH64);
            }
        }
        __syncwarp();
      } else if (warp == BW_SOFT_WARPS) {
        // ------------------------------------------------------------------ issuer X: dQ += dS K
        if (lane == 0) {
            const uint32_t idesc_q = idesc_bf16(DK, 0, 1);
            const uint32_t kmn_lo0 = desc_lo_mnmajor(sK, CH64);
            bool ok = true;
            for (int j = 0; j < nkv && ok; ++j) {
                const int bsel = j % NB;
                // K_j landed long ago (S(j) used it); this thread observes its barrier too before reading it --
                // first, so that only the wait on the critical path follows the group's arrival
                ok = mbar_wait(smem_u32(&kv_full[j % NS]), (j / NS) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (ok) ok = mbar_wait(smem_u32(&ds_full[bsel]), (j / NB) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (!ok) break;
                fence_after();
                const uint32_t kmn = kmn_lo0 + (j % NS) * (L::TILEK >> 4);
                const uint32_t a = tmem + bsel * 128;   // packed dS: 16 columns at the start of each half's 32
#pragma unroll
                for (int k = 0; k < BW_COLS / 16; ++k)   // contraction over the 64 keys
                    mma_ts(tmem + L::T_DQ, a + (k >> 1) * 32 + (k & 1) * 8, kmn + kstep_mnmajor(k), idesc_q,
                           (j > 0 || k > 0) ? 1u : 0u);
                commit(smem_u32(&kv_empty[j % NS]));  // last use of K_j; V_j was last read by dP(j), complete long before
                commit(smem_u32(&dq_done[bsel]));
            }
            if (ok) commit(smem_u32(done));
        }
        __syncwarp();
      } else {
        // ------------------------------------------------------------------ issuers Y: S = Q K^T (warp 18), Z: dP = dO V^T (warp 19)
        // An issuing thread cannot run ahead of the tensor pipe: its barrier waits and address
        // arithmetic would leave the pipe idle. With three issuers the gaps of one are filled by
        // the MMAs of the others; every accumulator still has one owner and a fixed order.
        if (lane == 0) {
            const bool is_s = warp == BW_SOFT_WARPS + 2;
            const uint32_t idesc_s = idesc_bf16(BW_COLS, 0, 0);
            const uint32_t a_lo = desc_lo_kmajor(is_s ? sQ : sDO);
            const uint32_t b_lo0 = desc_lo_kmajor(is_s ? sK : sV);
            const uint32_t t_off = is_s ? 0u : 64u;
            bool ok = true;
            auto issue = [&](int j) {  // S(j) or dP(j) into buffer j % NB
                const uint32_t b_lo = b_lo0 + (j % NS) * (L::TILEK >> 4);
                const uint32_t t = tmem + (j % NB) * 128 + t_off;
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)
                    mma_ss(t, a_lo + kstep_kmajor(k, CH128), b_lo + kstep_kmajor(k, CH64), idesc_s, k > 0 ? 1u : 0u);
                commit(smem_u32(&s_full[j % NB]));
            };
            ok = mbar_wait(smem_u32(qdo_full), 0, abort_flag, &g_attn_bwd_ws_ctl);
            for (int j = 0; j < NB && j < nkv && ok; ++j) {
                ok = mbar_wait(smem_u32(&kv_full[j % NS]), 0, abort_flag, &g_attn_bwd_ws_ctl);
                if (ok) {
                    fence_after();
                    issue(j);
                }
            }
            for (int j = 0; j + NB < nkv && ok; ++j) {
                // buffer j % NB is free once dQ of tile j has consumed the dS packed into it (which also
                // means that the element-wise group has read S(j) and dP(j))
                ok = mbar_wait(smem_u32(&kv_full[(j + NB) % NS]), ((j + NB) / NS) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (ok) ok = mbar_wait(smem_u32(&dq_done[j % NB]), (j / NB) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (!ok) break;
                fence_after();
                issue(j + NB);
            }
        }
        __syncwarp();
      }
    } else {
        // ------------------------------------------------------------------ element-wise warps
        asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
        const int grp = warp >> 3;
        const int wl = warp & 7;
        const int quad = wl & 3, hf = wl >> 2;
        const int row = quad * 32 + lane;
        const int qi = q0 + row;
        const bool row_ok = qi < p.S;
        const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_col = tmem + lane_off + hf * 32;   // + buffer * 128: this thread's 32 score columns
        const int64_t srow = (static_cast<int64_t>(b) * p.Hq + h) * p.S_pad + (row_ok ? qi : 0);
        // rows past the end of the sequence: p = 0 everywhere
        const float neg_lse2 = row_ok ? p.lneg[srow] : -INFINITY;
        const float neg_delta_s = row_ok ? p.dneg[srow] : 0.0f;
        bool ok = true;
        for (int j = grp; j < nkv; j += 2) {
            const int kv0 = j * BW_COLS;
            const int bsel = j % NB;
            const uint32_t t_s = t_col + bsel * 128, t_dp = t_s + 64;
            ok = mbar_wait(smem_u32(&s_full[bsel]), (j / NB) & 1, abort_flag, &g_attn_bwd_ws_ctl);
            ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the tensor-memory accesses are warp-wide
            if (!ok) break;
            fence_after();
            uint32_t rs[32], rd[32];
            tmem_ld32(t_s, rs);
            tmem_ld32(t_dp, rd);
            tmem_wait_ld();
            const bool need_mask = (p.causal && kv0 + BW_COLS - 1 > q0) || (kv0 + BW_COLS > p.S);
            const int key0 = kv0 + hf * 32;
            uint32_t pk[16];
            // two elements per instruction (packed fp32 pairs):
            // p = 2^(s c - lse2) (FFMA2 + 2 MUFU), ds = p (dp scale - delta scale) (FFMA2 + FMUL2)
            const uint64_t sl2 = f2_pack(p.scale_log2, p.scale_log2), nl2 = f2_pack(neg_lse2, neg_lse2);
            const uint64_t sc2 = f2_pack(p.scale, p.scale), nd2 = f2_pack(neg_delta_s, neg_delta_s);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                float x0, x1;
                f2_unpack(f2_fma(f2_pack_bits(rs[2 * e], rs[2 * e + 1]), sl2, nl2), x0, x1);
                float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                if (need_mask) {
                    const int ka = key0 + 2 * e;
                    if (ka >= p.S || (p.causal && ka > qi)) p0 = 0.0f;
                    if (ka + 1 >= p.S || (p.causal && ka + 1 > qi)) p1 = 0.0f;
                }
                float d0, d1;
                f2_unpack(f2_mul(f2_pack(p0, p1), f2_fma(f2_pack_bits(rd[2 * e], rd[2 * e + 1]), sc2, nd2)), d0, d1);
                pk[e] = pack2(d0, d1);
            }
            tmem_st16(t_s, pk);   // over this thread's own (already read) S columns
            tmem_wait_st();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ds_full[bsel]));
        }
        if (ok) ok = mbar_wait(smem_u32(done), 0, abort_flag, &g_attn_bwd_ws_ctl);
        ok = __all_sync(0xffffffffu, ok);
        fence_after();
        if (ok) {
            // dQ [128 x DK]: group, half -> a quarter of the columns each
            constexpr int W = DK / 4;
            const int c0 = grp * (DK / 2) + hf * W;
            bf16* dst = p.dq + (seq0 + qi) * p.lddq + h * DK + c0;
#pragma unroll
            for (int ch = 0; ch < W / 16; ++ch) {
                uint32_t r[16];
                tmem_ld16(tmem + lane_off + L::T_DQ + c0 + ch * 16, r);
                tmem_wait_ld();
                if (row_ok) st16_global(dst + ch * 16, r);
            }
        }
    }

    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ------------------------------------------------------------------------------ dK / dV
template <int DK>
struct DkvLayout {
    static constexpr int TILEK = (DK / 64) * (int)CH128;  // K, V: 128 rows, resident
    static constexpr int TILEQ = (DK / 64) * (int)CH64;   // Q_i, dO_i: 64 rows
    static constexpr int NS = DK == 64 ? 8 : 4;           // Q/dO stages: three tiles in use + TMA lead
    static constexpr int OFF_K = 0;
    static constexpr int OFF_V = TILEK;
    static constexpr int OFF_Q = 2 * TILEK;
    static constexpr int OFF_DO = OFF_Q + NS * TILEQ;
    static constexpr int OFF_X = OFF_DO + NS * TILEQ;     // per stage: [-lse2 | -delta scale] x 64 floats
    static constexpr int OFF_BAR = OFF_X + NS * 512;
    static constexpr int BYTES = OFF_BAR + 256 + 1024;
    // tensor memory columns: buffer b holds S^T at b*128 and dP^T at b*128 + 64; P^T / dS^T are
    // packed over the first 16 of each thread's own 32 columns. Three buffers where they fit
    // (head_dim 64), so that the scores of tile t+3 are issued as soon as tile t is finished.
    static constexpr int NB = DK == 64 ? 3 : 2;
    static constexpr int T_DV = NB * 128;
    static constexpr int T_DK = NB * 128 + DK;
};

template <int DK>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_ws_dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                       const WsBwdParams p) {
    using L = DkvLayout<DK>;
    constexpr int NS = L::NS;
    constexpr int NB = L::NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* kv_full = bars;
    uint64_t* q_full = bars + 1;          // [NS]  Q_i, dO_i and the statistics of tile i
    uint64_t* q_empty = q_full + NS;      // [NS]
    uint64_t* s_full = q_empty + NS;      // [NB]
    uint64_t* p_full = s_full + NB;       // [NB]
    uint64_t* g_done = p_full + NB;       // [NB]  dV / dK of a buffer's tile issued and complete
    uint64_t* done = g_done + NB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const float* xs_base = reinterpret_cast<const float*>(smem + L::OFF_X);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kt = blockIdx.x;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int group = p.Hq / p.Hkv;
    const int64_t seq0 = static_cast<int64_t>(b) * p.S;
    const int k0 = kt * BW_ROWS;
    const int nq_all = (p.S + BW_COLS - 1) / BW_COLS;
    const int i_begin = p.causal ? 2 * kt : 0;
    const int per_head = nq_all - i_begin;
    const int nit = per_head > 0 ? per_head * group : 0;

    if (tid == 0) {
        mbar_init(smem_u32(kv_full), 1);
        for (int i = 0; i < NS; ++i) {
            mbar_init(smem_u32(&q_full[i]), 1);
            mbar_init(smem_u32(&q_empty[i]), 1);
        }
        for (int i = 0; i < NB; ++i) {
            mbar_init(smem_u32(&s_full[i]), 2);   // S^T issuer + dP^T issuer
            mbar_init(smem_u32(&p_full[i]), BW_SOFT_WARPS / 2);
            mbar_init(smem_u32(&g_done[i]), 1);
        }
        mbar_init(smem_u32(done), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sK = smem_u32(smem + L::OFF_K), sV = smem_u32(smem + L::OFF_V);
    const uint32_t sQ = smem_u32(smem + L::OFF_Q), sDO = smem_u32(smem + L::OFF_DO);
    const uint32_t sX = smem_u32(smem + L::OFF_X);

    if (warp >= BW_SOFT_WARPS) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
      if (warp == BW_SOFT_WARPS + 1) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(smem_u32(kv_full), 2 * L::TILEK);
            tma_tile<DK>(sK, &map_k, hk * DK, k0, b, smem_u32(kv_full), CH128);
            tma_tile<DK>(sV, &map_v, hk * DK, k0, b, smem_u32(kv_full), CH128);
            for (int it = 0; it < nit; ++it) {
                const int st = it % NS, n = it / NS;
                const int h = hk * group + it / per_head;
                const int q0 = (i_begin + it % per_head) * BW_COLS;
                if (n > 0) ok = mbar_wait(smem_u32(&q_empty[st]), (n - 1) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (!ok) break;
                const uint32_t bar = smem_u32(&q_full[st]);
                mbar_expect_tx(bar, 2 * L::TILEQ + 512);
                tma_tile<DK>(sQ + st * L::TILEQ, &map_q, h * DK, q0, b, bar, CH64);
                tma_tile<DK>(sDO + st * L::TILEQ, &map_do, h * DK, q0, b, bar, CH64);
                const int64_t so = (static_cast<int64_t>(b) * p.Hq + h) * p.S_pad + q0;
                bulk_load(sX + st * 512, p.lneg + so, 256, bar);
                bulk_load(sX + st * 512 + 256, p.dneg + so, 256, bar);
            }
        }
        __syncwarp();
      } else if (warp == BW_SOFT_WARPS) {
        // ------------------------------------------------------------------ issuer X: dV += P^T dO, dK += dS^T Q
        if (lane == 0) {
            const uint32_t idesc_g = idesc_bf16(DK, 0, 1);
            const uint32_t qmn_lo0 = desc_lo_mnmajor(sQ, CH64), domn_lo0 = desc_lo_mnmajor(sDO, CH64);
            bool ok = true;
            for (int it = 0; it < nit && ok; ++it) {
                const int bsel = it % NB;
                // Q_i / dO_i landed long ago (the scores used them); observe their barrier too, first
                ok = mbar_wait(smem_u32(&q_full[it % NS]), (it / NS) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (ok) ok = mbar_wait(smem_u32(&p_full[bsel]), (it / NB) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (!ok) break;
                fence_after();
                const uint32_t st_off = (it % NS) * (L::TILEQ >> 4);
                const uint32_t a_p = tmem + bsel * 128, a_ds = a_p + 64;
                const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
                for (int k = 0; k < BW_COLS / 16; ++k)   // contraction over the 64 queries
                    mma_ts(tmem + L::T_DV, a_p + (k >> 1) * 32 + (k & 1) * 8, domn_lo0 + st_off + kstep_mnmajor(k), idesc_g,
                           k > 0 ? 1u : acc);
#pragma unroll
                for (int k = 0; k < BW_COLS / 16; ++k)
                    mma_ts(tmem + L::T_DK, a_ds + (k >> 1) * 32 + (k & 1) * 8, qmn_lo0 + st_off + kstep_mnmajor(k), idesc_g,
                           k > 0 ? 1u : acc);
                commit(smem_u32(&q_empty[it % NS]));
                commit(smem_u32(&g_done[bsel]));   // P^T / dS^T of this buffer consumed: the score issuers may overwrite it
            }
            if (ok) commit(smem_u32(done));
        }
        __syncwarp();
      } else {
        // ------------------------------------------------------------------ issuers Y: S^T = K Q^T (warp 18), Z: dP^T = V dO^T (warp 19)
        if (lane == 0) {
            const bool is_s = warp == BW_SOFT_WARPS + 2;
            const uint32_t idesc_s = idesc_bf16(BW_COLS, 0, 0);
            const uint32_t a_lo = desc_lo_kmajor(is_s ? sK : sV);
            const uint32_t b_lo0 = desc_lo_kmajor(is_s ? sQ : sDO);
            const uint32_t t_off = is_s ? 0u : 64u;
            bool ok = true;
            auto issue = [&](int it) {  // S^T or dP^T of tile `it` into buffer it % NB
                const uint32_t b_lo = b_lo0 + (it % NS) * (L::TILEQ >> 4);
                const uint32_t t = tmem + (it % NB) * 128 + t_off;
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)
                    mma_ss(t, a_lo + kstep_kmajor(k, CH128), b_lo + kstep_kmajor(k, CH64), idesc_s, k > 0 ? 1u : 0u);
                commit(smem_u32(&s_full[it % NB]));
            };
            ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, &g_attn_bwd_ws_ctl);
            for (int it = 0; it < NB && it < nit && ok; ++it) {
                ok = mbar_wait(smem_u32(&q_full[it % NS]), 0, abort_flag, &g_attn_bwd_ws_ctl);
                if (ok) {
                    fence_after();
                    issue(it);
                }
            }
            for (int it = 0; it + NB < nit && ok; ++it) {
                // the packed P^T / dS^T of tile `it` live in this buffer until dV / dK of that tile are done
                ok = mbar_wait(smem_u32(&q_full[(it + NB) % NS]), ((it + NB) / NS) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (ok) ok = mbar_wait(smem_u32(&g_done[it % NB]), (it / NB) & 1, abort_flag, &g_attn_bwd_ws_ctl);
                if (!ok) break;
                fence_after();
                issue(it + NB);
            }
        }
        __syncwarp();
      }
    } else {
        // ------------------------------------------------------------------ element-wise warps
        asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
        const int grp = warp >> 3;
        const int wl = warp & 7;
        const int quad = wl & 3, hf = wl >> 2;
        const int row = quad * 32 + lane;
        const int kj = k0 + row;  // this thread's key
        const bool key_ok = kj < p.S;
        const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_col = tmem + lane_off + hf * 32;   // + buffer * 128: this thread's 32 columns of S^T
        bool ok = true;
        for (int it = grp; it < nit; it += 2) {
            const int st = it % NS;
            const int q0 = (i_begin + it % per_head) * BW_COLS;
            const int bsel = it % NB;
            const uint32_t t_s = t_col + bsel * 128, t_dp = t_s + 64;
            ok = mbar_wait(smem_u32(&s_full[bsel]), (it / NB) & 1, abort_flag, &g_attn_bwd_ws_ctl);
            // the statistics arrived with Q_i / dO_i: observe that barrier too before reading them
            if (ok) ok = mbar_wait(smem_u32(&q_full[st]), (it / NS) & 1, abort_flag, &g_attn_bwd_ws_ctl);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after();
            uint32_t rs[32], rd[32];
            tmem_ld32(t_s, rs);
            tmem_ld32(t_dp, rd);
            tmem_wait_ld();
            const bool need_mask = (p.causal && k0 + BW_ROWS - 1 > q0) || (k0 + BW_ROWS > p.S);
            const float* xs = xs_base + st * 128 + hf * 32;   // [-lse2 x 64 | -delta scale x 64]
            const int qc0 = q0 + hf * 32;
            uint32_t pp[16], pd[16];
            // two elements per instruction (packed fp32 pairs); the statistics come as pairs too
            const uint64_t sl2 = f2_pack(p.scale_log2, p.scale_log2), sc2 = f2_pack(p.scale, p.scale);
            const uint64_t* xs2 = reinterpret_cast<const uint64_t*>(xs);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                float x0, x1;
                f2_unpack(f2_fma(f2_pack_bits(rs[2 * e], rs[2 * e + 1]), sl2, xs2[e]), x0, x1);
                float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                if (need_mask) {  // queries past the end already have -lse2 = -inf
                    if (!key_ok || (p.causal && kj > qc0 + 2 * e)) p0 = 0.0f;
                    if (!key_ok || (p.causal && kj > qc0 + 2 * e + 1)) p1 = 0.0f;
                }
                pp[e] = pack2(p0, p1);
                float d0, d1;
                f2_unpack(f2_mul(f2_pack(p0, p1), f2_fma(f2_pack_bits(rd[2 * e], rd[2 * e + 1]), sc2, xs2[32 + e])), d0, d1);
                pd[e] = pack2(d0, d1);
            }
            tmem_st16(t_s, pp);    // over this thread's own (already read) columns
            tmem_st16(t_dp, pd);
            tmem_wait_st();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[bsel]));
        }
        if (ok) ok = mbar_wait(smem_u32(done), 0, abort_flag, &g_attn_bwd_ws_ctl);
        ok = __all_sync(0xffffffffu, ok);
        fence_after();
        if (ok) {
            // group 0 writes dV, group 1 writes dK; the two halves split the columns
            constexpr int W = DK / 2;
            bf16* dst = (grp == 0 ? p.dv + (seq0 + kj) * p.lddv : p.dk + (seq0 + kj) * p.lddk) + hk * DK + hf * W;
            const uint32_t t_src = tmem + lane_off + (grp == 0 ? L::T_DV : L::T_DK) + hf * W;
#pragma unroll
            for (int ch = 0; ch < W / 16; ++ch) {
                uint32_t r[16];
                if (nit > 0) {
                    tmem_ld16(t_src + ch * 16, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) r[e] = 0u;
                }
                if (key_ok) st16_global(dst + ch * 16, r);
            }
        }
    }

    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem, 512);
    }
}

template <typename K>
int prepare_kernel(K kern, int smem_bytes) {
    cudaFuncAttributes fa;
    PK_CHECK_CUDA(cudaFuncGetAttributes(&fa, kern));
    PK_REQUIRE(fa.numRegs * BW_THREADS >= BW_SOFT_WARPS * 32 * BW_REGS_SOFT + 4 * 32 * BW_REGS_CTRL,
               "attention backward: the kernel's launch register allocation cannot cover its setmaxnreg plan");
    PK_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    return PK_OK;
}

template <int DK>
int launch_bwd_ws(cudaStream_t st, const CUtensorMap& mq128, const CUtensorMap& mdo128, const CUtensorMap& mk64,
                  const CUtensorMap& mv64, const CUtensorMap& mq64, const CUtensorMap& mdo64, const CUtensorMap& mk128,
                  const CUtensorMap& mv128, const WsBwdParams& p, int64_t B) {
    auto kq = attn_bwd_ws_dq_kernel<DK>;
    auto kkv = attn_bwd_ws_dkv_kernel<DK>;
    static bool ready = false;
    if (!ready) {
        int rc = prepare_kernel(kq, DqLayout<DK>::BYTES);
        if (rc != PK_OK) return rc;
        rc = prepare_kernel(kkv, DkvLayout<DK>::BYTES);
        if (rc != PK_OK) return rc;
        ready = true;
    }
    const unsigned tiles = static_cast<unsigned>((p.S + BW_ROWS - 1) / BW_ROWS);
    dim3 gq(tiles, p.Hq, static_cast<unsigned>(B));
    kq<<<gq, BW_THREADS, DqLayout<DK>::BYTES, st>>>(mq128, mk64, mv64, mdo128, p);
    PK_LAUNCH_CHECK();
    dim3 gkv(tiles, p.Hkv, static_cast<unsigned>(B));
    kkv<<<gkv, BW_THREADS, DkvLayout<DK>::BYTES, st>>>(mq64, mk128, mv128, mdo64, p);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

int64_t padded_len(int64_t S) { return (S + BW_COLS - 1) / BW_COLS * BW_COLS; }

}  // namespace

size_t attn_bwd_ws_scratch_bytes(int64_t B, int64_t S, int Hq) {
    return 2 * static_cast<size_t>(B) * static_cast<size_t>(Hq) * static_cast<size_t>(padded_len(S)) * sizeof(float);
}

int attn_bwd_ws(cudaStream_t st, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                const void* out, int64_t ldo, const float* lse, const void* dout, int64_t lddo, void* dq, int64_t lddq,
                void* dk_, int64_t lddk, void* dv, int64_t lddv, float* scratch, int64_t B, int64_t S, int Hq, int Hkv,
                int dk, float scale, int causal) {
    const int64_t S_pad = padded_len(S);
    float* lneg = scratch;
    float* dneg = scratch + B * Hq * S_pad;
    PK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "scratch must be 16-byte aligned");
    {
        const int hpw = 32 / (dk / 8);
        const int64_t nw = B * S_pad * ((Hq + hpw - 1) / hpw);
        const unsigned blocks = static_cast<unsigned>((nw + 7) / 8);
        if (dk == 64)
            attn_bwd_stats_kernel<64><<<blocks, 256, 0, st>>>(static_cast<const bf16*>(out), ldo, static_cast<const bf16*>(dout),
                                                              lddo, lse, lneg, dneg, B, S, S_pad, Hq, scale);
        else
            attn_bwd_stats_kernel<128><<<blocks, 256, 0, st>>>(static_cast<const bf16*>(out), ldo, static_cast<const bf16*>(dout),
                                                               lddo, lse, lneg, dneg, B, S, S_pad, Hq, scale);
        PK_LAUNCH_CHECK();
    }

    CUtensorMap mq128, mdo128, mk64, mv64, mq64, mdo64, mk128, mv128;
    const int64_t R = B * S;
    const int64_t wq = static_cast<int64_t>(Hq) * dk, wk = static_cast<int64_t>(Hkv) * dk;
    int rc;
    if ((rc = make_tensor_map_3d(&mq128, q, wq, S, B, ldq, 64, 128)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mdo128, dout, wq, S, B, lddo, 64, 128)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mk64, k, wk, S, B, ldk, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mv64, v, wk, S, B, ldv, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mq64, q, wq, S, B, ldq, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mdo64, dout, wq, S, B, lddo, 64, 64)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mk128, k, wk, S, B, ldk, 64, 128)) != PK_OK) return rc;
    if ((rc = make_tensor_map_3d(&mv128, v, wk, S, B, ldv, 64, 128)) != PK_OK) return rc;
    WsBwdParams p;
    p.dq = static_cast<bf16*>(dq);
    p.lddq = lddq;
    p.dk = static_cast<bf16*>(dk_);
    p.lddk = lddk;
    p.dv = static_cast<bf16*>(dv);
    p.lddv = lddv;
    p.lneg = lneg;
    p.dneg = dneg;
    p.S = static_cast<int>(S);
    p.S_pad = static_cast<int>(S_pad);
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale = scale;
    p.scale_log2 = scale * BW_LOG2E;
    p.causal = causal;
    return dk == 64 ? launch_bwd_ws<64>(st, mq128, mdo128, mk64, mv64, mq64, mdo64, mk128, mv128, p, B)
                    : launch_bwd_ws<128>(st, mq128, mdo128, mk64, mv64, mq64, mdo64, mk128, mv128, p, B);
}


}  // namespace pk
