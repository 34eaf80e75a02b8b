// bf16 GEMM on a pair of SMs per output tile (tcgen05 cta_group::2).
//
// A cluster of two CTAs computes one 256 x 256 tile: CTA r owns rows r*128 .. r*128+127 of the
// tile (its A slice and its half of the fp32 accumulator, 128 lanes x 256 columns of its own
// tensor memory) and loads only HALF of the B slice (128 of the 256 columns); one
// tcgen05.mma.cta_group::2 issued by the leader CTA (rank 0) drives both tensor cores and takes
// the two halves of B from the two CTAs' shared memories. Per 64-wide k slice a CTA therefore
// receives 32 KB instead of the 48 KB of the one-CTA kernel (pk_gemm_tc.cu) and its tensor core
// reads 8 KB instead of 12 KB of operands per MMA, which is what keeps that kernel's tensor pipe
// near 70 % busy.
//
// Roles in each CTA (192 threads):
//   warp 0      TMA producer: its A slice and its half of B into a 6-stage ring; the loads of
//               both CTAs complete on the LEADER's "full" barrier (cta_group::2 form of the load,
//               no multicast)
//   warp 1      allocates tensor memory (both CTAs); in the leader, one thread issues the MMAs
//               and signals "stage free" / "accumulator full" in both CTAs with multicast commits
//   warps 2..5  epilogue: tcgen05.ld of the CTA's own rows, bias / residual / accumulate, stores;
//               "accumulator free" arrives at the leader's barrier (8 warps of the pair)
// The k order is fixed and every accumulator column has one issuer: reproducible bit for bit,
// and identical to the one-CTA kernel's result (same products, same order).
// Every mbarrier wait is bounded (status word shared with pk_gemm_tc.cu's convention, no trap);
// both CTAs always reach the two cluster-wide barriers at the start and the end.
#include <cuda.h>

#include "pk_common.cuh"
#include "pk_tc.cuh"
#include "pk_gemm_epilogue.cuh"

namespace pk {

PK_DEFINE_WAITCTL(gemm_tc2)

namespace {

using namespace tc;

constexpr int T2_BM = 128;         // rows per CTA; the pair covers 256
constexpr int T2_BN = 256;
constexpr int T2_BK = 64;
constexpr int T2_THREADS = 192;          // producer warp, MMA warp, four epilogue warps
constexpr int T2_THREADS_SWIGLU = 320;   // SwiGLU mode: eight epilogue warps (two per tensor-memory lane quadrant, 64 of
                                         // the tile's 128 G / U columns each): its epilogue has an exponential and a
                                         // division per element and was the bound with four
constexpr int T2_STAGES = 6;
constexpr int T2_A_BYTES = T2_BM * T2_BK * 2;          // 16 KiB
constexpr int T2_B_BYTES = (T2_BN / 2) * T2_BK * 2;    // 16 KiB: this CTA's half of B
constexpr int T2_STAGE_BYTES = T2_A_BYTES + T2_B_BYTES;
constexpr int T2_EPI_BOXES = 4;              // per epilogue warp: boxes of 32 rows x 64 bytes for TMA loads / stores of the output
constexpr int T2_EPI_BYTES = 4 * T2_EPI_BOXES * 2048;
constexpr int T2_SMEM_BYTES = T2_STAGES * T2_STAGE_BYTES + T2_EPI_BYTES + 1024 + 512;

struct T2Params {
    int64_t M, N, K;
    void* C;
    int64_t ldc;
    const float* bias;
    const void* residual;
    int64_t ldr;
    int accumulate;
    int a_mn_major, b_mn_major;
    // split-K, as in the one-CTA kernel: work item w = (tile w % n_tiles, k part w / n_tiles),
    // fp32 partial tiles in partial + part * slab (row stride pstride); splits == 1: off
    int splits, kb_per_split;
    float* partial;
    int64_t slab, pstride;
    // SwiGLU pair mode (template parameter SWIGLU): the tile's 256 columns are 128 columns of
    // G = A Wg (loaded by CTA 0 of the pair) and the SAME 128 columns of U = A Wu (CTA 1, second
    // tensor map); the epilogue writes y = silu(G) * U [M, N] and, when C / U are given, G and U.
    void* U;        // nullable, row stride ldc like C
    void* Y;
    int64_t ldy;
    // 1: the output goes through shared-memory staging and TMA stores (map_c; map_u / map_y in
    // SwiGLU mode), 0: the threads store their rows themselves (unaligned C, ragged N with a
    // residual or accumulate read)
    int tma_out;
    // rotary embedding in the epilogue (StagedOut in pk_gemm_epilogue.cuh); rope_cs == nullptr: none
    const float* rope_cs;
    const int32_t* rope_pos;
    int rope_half;
    int64_t rope_cols, rope_npos;
    float rope_sign;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion is counted on a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void mma2_ss(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives (once all MMAs issued so far are complete) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(static_cast<uint16_t>(3))
        : "memory");
}
__host__ __device__ inline uint32_t idesc_pair(int n, int a_mn_major, int b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= 1u << 7;
    d |= 1u << 10;
    d |= static_cast<uint32_t>(a_mn_major & 1) << 15;
    d |= static_cast<uint32_t>(b_mn_major & 1) << 16;
    d |= static_cast<uint32_t>(n >> 3) << 17;
    d |= static_cast<uint32_t>(256 >> 4) << 24;  // M of the pair
    return d;
}
__device__ __forceinline__ bool wait2(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait(bar, parity, abort_flag, &g_gemm_tc2_ctl);
}

template <typename TC>
__device__ __forceinline__ void store8(TC* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<bf16>(bf16* p, const float (&v)[8]) {
    Vec<bf16>::store(p, v);
}
template <typename TC>
__device__ __forceinline__ void load8(const TC* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
    Vec<bf16>::load(p, v);
}

template <typename TC, bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SWIGLU ? T2_THREADS_SWIGLU : T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_c,
                const __grid_constant__ CUtensorMap map_u, const __grid_constant__ CUtensorMap map_y, const T2Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* epi_smem = smem + T2_STAGES * T2_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + T2_EPI_BYTES);
    uint64_t* full_bar = bars;                        // [STAGES]  used in the leader
    uint64_t* empty_bar = bars + T2_STAGES;           // [STAGES]  one per CTA, both signalled by the leader
    uint64_t* acc_full = bars + 2 * T2_STAGES;        // [2]       one per CTA, both signalled by the leader
    uint64_t* acc_empty = bars + 2 * T2_STAGES + 2;   // [2]       used in the leader: 8 epilogue warps of the pair
    uint64_t* in_bar = bars + 2 * T2_STAGES + 4;      // [4 warps][EPI_BOXES] per CTA: residual / C box has landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(in_bar + 4 * T2_EPI_BOXES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    // columns of the output a tile covers: 256, or 128 of G and of U each in SwiGLU pair mode
    constexpr int TILE_N = SWIGLU ? T2_BN / 2 : T2_BN;
    const int64_t tiles_m = (p.M + 2 * T2_BM - 1) / (2 * T2_BM), tiles_n = (p.N + TILE_N - 1) / TILE_N;
    const int64_t n_tiles = tiles_m * tiles_n;
    const int64_t n_work = n_tiles * p.splits;
    const int k_blocks = static_cast<int>((p.K + T2_BK - 1) / T2_BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < T2_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full[a]), 1);
            mbar_init(smem_u32(&acc_empty[a]), SWIGLU ? 16 : 8);   // epilogue warps of the pair
        }
        for (int b = 0; b < 4 * T2_EPI_BOXES; ++b) mbar_init(smem_u32(&in_bar[b]), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers are initialised before anything remote touches them
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t w = pair; w < n_work && ok; w += n_pairs) {
                const int64_t tile = w % n_tiles;
                const int kb0 = static_cast<int>(w / n_tiles) * p.kb_per_split;
                const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
                const int32_t m0 = static_cast<int32_t>((tile / tiles_n) * (2 * T2_BM) + rank * T2_BM);
                const int32_t n0 = SWIGLU ? static_cast<int32_t>((tile % tiles_n) * TILE_N)
                                          : static_cast<int32_t>((tile % tiles_n) * T2_BN + rank * (T2_BN / 2));
                const CUtensorMap* mb = (SWIGLU && rank == 1) ? &map_b2 : &map_b;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait2(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t fb_local = smem_u32(&full_bar[stage]);
                    const uint32_t fb = map_to_rank(fb_local, 0);   // the leader's barrier counts both CTAs' bytes
                    if (leader) mbar_expect_tx(fb_local, 2 * T2_STAGE_BYTES);
                    const uint32_t sa = smem_u32(smem + stage * T2_STAGE_BYTES);
                    const uint32_t sb = sa + T2_A_BYTES;
                    const int32_t k0 = kb * T2_BK;
                    if (!p.a_mn_major) {
                        tma_load_2d_pair(sa, &map_a, k0, m0, fb);                 // box 64(k) x 128(m)
                    } else {
#pragma unroll
                        for (int c = 0; c < T2_BM / 64; ++c)                      // boxes 64(m) x 64(k)
                            tma_load_2d_pair(sa + c * 8192, &map_a, m0 + c * 64, k0, fb);
                    }
                    if (!p.b_mn_major) {
                        tma_load_2d_pair(sb, mb, k0, n0, fb);                     // box 64(k) x 128(n)
                    } else {
#pragma unroll
                        for (int c = 0; c < (T2_BN / 2) / 64; ++c)                // boxes 64(n) x 64(k)
                            tma_load_2d_pair(sb + c * 8192, mb, n0 + c * 64, k0, fb);
                    }
                    if (++stage == T2_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            const uint32_t idesc = idesc_pair(T2_BN, p.a_mn_major, p.b_mn_major);
            const uint32_t a_flags = ((p.a_mn_major ? 8192u : 16u) >> 4) << 16, b_flags = ((p.b_mn_major ? 8192u : 16u) >> 4) << 16;
            const uint32_t a_step = (p.a_mn_major ? 2048u : 32u) >> 4, b_step = (p.b_mn_major ? 2048u : 32u) >> 4;
            const uint32_t a_lo0 = ((smem_u32(smem) & 0x3ffffu) >> 4) | a_flags;
            const uint32_t b_lo0 = (((smem_u32(smem) + T2_A_BYTES) & 0x3ffffu) >> 4) | b_flags;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int64_t w = pair; w < n_work && ok; w += n_pairs) {
                const int kb0 = static_cast<int>(w / n_tiles) * p.kb_per_split;
                const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
                if (!wait2(smem_u32(&acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * T2_BN);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait2(smem_u32(&full_bar[stage]), phase, abort_flag)) { ok = false; break; }
                    fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (T2_STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (T2_STAGE_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < T2_BK / 16; ++k)
                        mma2_ss(d_tmem, a_lo + k * a_step, b_lo + k * b_step, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    commit_pair(smem_u32(&empty_bar[stage]));   // frees the stage in both CTAs
                    if (++stage == T2_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                commit_pair(smem_u32(&acc_full[acc]));          // accumulator complete, both CTAs
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        TC* C = static_cast<TC*>(p.C);
        const TC* Rsd = static_cast<const TC*>(p.residual);
        StagedOut out;   // staged form of the output (p.tma_out): boxes, barriers and maps of this warp
        // boxes per warp: four, or two in SwiGLU mode (eight warps, stores only)
        constexpr int WARP_BOXES = SWIGLU ? T2_EPI_BOXES / 2 : T2_EPI_BOXES;
        out.boxes = epi_smem + (warp - 2) * (WARP_BOXES * EPI_BOX_BYTES);
        out.in_bar = in_bar + ((warp - 2) & 3) * T2_EPI_BOXES;
        out.out = &map_c;
        out.in = p.splits > 1 ? nullptr : (Rsd != nullptr ? &map_u : (p.accumulate ? &map_c : nullptr));
        out.bias = p.splits > 1 ? nullptr : p.bias;
        out.N = p.splits > 1 ? p.pstride : p.N;
        out.slab = -1;
        out.uc = 0;
        out.rope_cs = p.rope_cs;
        out.rope_pos = p.rope_pos;
        out.rope_half = p.rope_half;
        out.rope_cols = p.rope_cols;
        out.rope_npos = p.rope_npos;
        out.rope_sign = p.rope_sign;
        out.M = p.M;
        bool ok = true;
        for (int64_t w = pair; w < n_work && ok; w += n_pairs) {
            const int64_t tile = w % n_tiles;
            const int64_t m0 = (tile / tiles_n) * (2 * T2_BM) + rank * T2_BM, n0 = (tile % tiles_n) * TILE_N;
            const int64_t m = m0 + quad * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * T2_BN);
            float* part = p.splits > 1 ? p.partial + (w / n_tiles) * p.slab + m * p.pstride : nullptr;
            const bool staged = !SWIGLU && p.tma_out;   // waits for the accumulator after it has requested its inputs
            if (!staged) {
                ok = wait2(smem_u32(&acc_full[acc]), acc_phase, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fence_after();
            }
            if (SWIGLU) {
                // columns 0..127 of the accumulator are G, 128..255 the same columns of U. G and U are
                // rounded to the storage type first and y is formed from the rounded values with the
                // arithmetic of the stand-alone SwiGLU kernel, so y has the bits the separate
                // GEMM + GEMM + SwiGLU sequence produces, whether or not G and U are also stored.
                TC* Gout = static_cast<TC*>(p.C);
                TC* Uout = static_cast<TC*>(p.U);
                TC* Yout = static_cast<TC*>(p.Y);
                // warps 2..5 take the tile's first 64 columns of G / U, warps 6..9 the other 64
                const int ch0 = ((warp - 2) >> 2) * (TILE_N / 64), ch1 = ch0 + TILE_N / 64;
#pragma unroll 1
                for (int ch = ch0; ch < ch1; ++ch) {
                    const int64_t c0 = n0 + ch * 32;
                    if (c0 >= p.N) break;  // uniform across the warp
                    uint32_t rg[32], ru[32];
                    tmem_ld32(t_row + static_cast<uint32_t>(ch * 32), rg);
                    tmem_ld32(t_row + static_cast<uint32_t>(TILE_N + ch * 32), ru);
                    tmem_wait_ld();
                    if (p.tma_out) {
                        // staged form: up to three boxes per 32 columns (G, U, y), each handed to a TMA store
                        float gv[32], uv[32], yv[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            gv[e] = to_f32(from_f32<TC>(__uint_as_float(rg[e])));
                            uv[e] = to_f32(from_f32<TC>(__uint_as_float(ru[e])));
                            yv[e] = (gv[e] / (1.0f + expf(-gv[e]))) * uv[e];
                        }
                        const int32_t x = static_cast<int32_t>(c0), y0 = static_cast<int32_t>(m0 + quad * 32);
                        auto emit = [&](const float* vals, const CUtensorMap* map) {
                            uint8_t* box = out.boxes + (out.uc & (WARP_BOXES - 1)) * EPI_BOX_BYTES;
                            if (lane == 0) bulk_wait_read<WARP_BOXES - 1>();
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(box + box_offset(lane, j)) = pack_out<TC>(vals + j * 8);
                            fence_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                tma_store_2d(map, smem_u32(box), x, y0);
                                bulk_commit();
                            }
                            ++out.uc;
                        };
                        if (Gout) emit(gv, &map_c);
                        if (Uout) emit(uv, &map_u);
                        emit(yv, &map_y);
                    } else if (m < p.M) {
#pragma unroll
                        for (int g8 = 0; g8 < 4; ++g8) {
                            const int64_t c = c0 + g8 * 8;
                            if (c >= p.N) break;   // N is a multiple of 8 in this mode
                            float gv[8], uv[8], yv[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                gv[e] = to_f32(from_f32<TC>(__uint_as_float(rg[g8 * 8 + e])));
                                uv[e] = to_f32(from_f32<TC>(__uint_as_float(ru[g8 * 8 + e])));
                                yv[e] = (gv[e] / (1.0f + expf(-gv[e]))) * uv[e];
                            }
                            if (Gout) store8<TC>(Gout + m * p.ldc + c, gv);
                            if (Uout) store8<TC>(Uout + m * p.ldc + c, uv);
                            store8<TC>(Yout + m * p.ldy + c, yv);
                        }
                    }
                }
            } else if (p.tma_out) {
                // staged form (pk_gemm_epilogue.cuh); with k parts the fp32 partial tile goes to its slab
                const int32_t y0 = static_cast<int32_t>(m0 + quad * 32);
                const uint32_t acc_bar = smem_u32(&acc_full[acc]);
                if (p.splits > 1) {
                    out.slab = static_cast<int32_t>(w / n_tiles);
                    ok = staged_epilogue<float, T2_BN, T2_EPI_BOXES>(out, n0, y0, t_row, acc_bar, acc_phase, abort_flag, &g_gemm_tc2_ctl, lane);
                } else if (sizeof(TC) == 2 && p.rope_cs != nullptr) {
                    ok = staged_epilogue<TC, T2_BN, T2_EPI_BOXES, true>(out, n0, y0, t_row, acc_bar, acc_phase, abort_flag, &g_gemm_tc2_ctl, lane);
                } else {
                    ok = staged_epilogue<TC, T2_BN, T2_EPI_BOXES>(out, n0, y0, t_row, acc_bar, acc_phase, abort_flag, &g_gemm_tc2_ctl, lane);
                }
                if (!ok) break;
            } else
#pragma unroll 1
            for (int ch = 0; ch < T2_BN / 32; ++ch) {
                const int64_t c0 = n0 + ch * 32;
                if (c0 >= p.N) break;  // uniform across the warp
                uint32_t r[32];
                tmem_ld32(t_row + static_cast<uint32_t>(ch * 32), r);
                tmem_wait_ld();
                if (part != nullptr) {
                    // raw fp32 partial; pstride is a multiple of 256 columns, so whole chunks fit
                    if (m < p.M) {
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            *reinterpret_cast<uint4*>(part + c0 + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
                    }
                } else if (m < p.M) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int64_t c = c0 + g * 8;
                        if (c < p.N && c + 8 > p.N) {
                            for (int e = 0; e < 8 && c + e < p.N; ++e) {   // ragged last group
                                float x = __uint_as_float(r[g * 8 + e]);
                                if (p.bias) x += p.bias[c + e];
                                if (Rsd) x += to_f32(Rsd[m * p.ldr + c + e]);
                                if (p.accumulate) x += to_f32(C[m * p.ldc + c + e]);
                                C[m * p.ldc + c + e] = from_f32<TC>(x);
                            }
                        } else if (c < p.N) {
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g * 8 + e]);
                            if (p.bias) {
                                float b[8];
                                load8<float>(p.bias + c, b);
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] += b[e];
                            }
                            if (Rsd) {
                                float q[8];
                                load8<TC>(Rsd + m * p.ldr + c, q);
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] += q[e];
                            }
                            if (p.accumulate) {
                                float q[8];
                                load8<TC>(C + m * p.ldc + c, q);
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] += q[e];
                            }
                            store8<TC>(C + m * p.ldc + c, v);
                        }
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) remote_arrive(map_to_rank(smem_u32(&acc_empty[acc]), 0));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }
    if (warp >= 2 && lane == 0) bulk_wait_all();   // this thread's TMA stores are complete before the CTA's shared memory goes away
    fence_before();
    __syncthreads();
    cluster_sync_all();   // no CTA leaves while the other may still signal its barriers or read its shared memory
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);


template <typename TC, bool SWIGLU>
int launch2(cudaStream_t st, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, T2Params p, int c_dtype) {
    auto kern = gemm_tc2_kernel<TC, SWIGLU>;
    static bool attr_set = false;
    if (!attr_set) {
        PK_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES));
        attr_set = true;
    }
    // how many CTA pairs the GPU can hold at once (SM pairs are formed inside GPCs, so this may be
    // fewer than half the SM count)
    static int max_pairs = 0;
    if (max_pairs == 0) {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2));
        probe.blockDim = dim3(SWIGLU ? T2_THREADS_SWIGLU : T2_THREADS);
        probe.dynamicSmemBytes = T2_SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        probe.attrs = &attr;
        probe.numAttrs = 1;
        int n = 0;
        PK_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &probe));
        PK_REQUIRE(n > 0, "no CTA pair fits on this GPU");
        max_pairs = n;
    }
    const int64_t tile_n = SWIGLU ? T2_BN / 2 : T2_BN;
    const int64_t tiles = ((p.M + 2 * T2_BM - 1) / (2 * T2_BM)) * ((p.N + tile_n - 1) / tile_n);
    // Split-K when the last wave of tiles would leave many SM pairs idle and the k loop is long
    // (weight gradients: a few hundred tiles, tens of thousands of rows): the smallest number of
    // k parts whose work items fill the waves to 95 %, if the caller's workspace holds them.
    const int64_t k_blocks = (p.K + T2_BK - 1) / T2_BK;
    p.splits = 1;
    p.pstride = (p.N + T2_BN - 1) / T2_BN * T2_BN;
    p.slab = p.M * p.pstride;
    size_t ws_bytes = 0;
    p.partial = gemm_splitk_workspace(&ws_bytes);
    auto fill = [&](int64_t items) {
        return static_cast<double>(items) / static_cast<double>((items + max_pairs - 1) / max_pairs * max_pairs);
    };
    if (!SWIGLU && p.rope_cs == nullptr && p.partial != nullptr && k_blocks >= 256 && fill(tiles) < 0.9) {
        for (int sp = 2; sp <= 4; ++sp) {
            if (static_cast<size_t>(sp) * p.slab * sizeof(float) > ws_bytes) break;
            if (fill(tiles * sp) >= 0.95) {
                p.splits = sp;
                break;
            }
        }
    }
    p.kb_per_split = static_cast<int>((k_blocks + p.splits - 1) / p.splits);
    if (p.splits > 1 && static_cast<int64_t>(p.kb_per_split) * (p.splits - 1) >= k_blocks)
        p.splits = static_cast<int>((k_blocks + p.kb_per_split - 1) / p.kb_per_split);
    gemm_note_splits(p.splits);
    // Output through shared-memory staging and TMA stores (pk_gemm_epilogue.cuh) when the outputs can
    // be described by tensor maps (16-byte aligned base and row stride) and every 16-byte group
    // the epilogue reads (bias, residual or C) lies inside a row.
    constexpr int64_t PER16 = 16 / static_cast<int64_t>(sizeof(TC));
    CUtensorMap mc = ma, mu = ma, my = ma;
    if (SWIGLU) {
        const bool keep = p.C != nullptr;
        p.tma_out = aligned16(p.Y) && (p.ldy % 8) == 0 && (p.N % 8) == 0 &&
                    (!keep || (aligned16(p.C) && aligned16(p.U) && (p.ldc % 8) == 0));
        if (p.tma_out) {
            int rc = make_tensor_map_out(&my, p.Y, 2, p.N, p.M, p.ldy, 32);
            if (rc == PK_OK && keep) rc = make_tensor_map_out(&mc, p.C, 2, p.N, p.M, p.ldc, 32);
            if (rc == PK_OK && keep) rc = make_tensor_map_out(&mu, p.U, 2, p.N, p.M, p.ldc, 32);
            if (rc != PK_OK) return rc;
        }
    } else if (p.splits > 1) {
        p.tma_out = aligned16(p.partial);
        if (p.tma_out) {   // fp32 partial tiles: columns, rows, k part
            const int rc = make_tensor_map_out_3d(&mc, p.partial, 4, p.pstride, p.M, p.splits, p.pstride, p.slab, 32);
            if (rc != PK_OK) return rc;
        }
    } else {
        const bool reads = p.bias != nullptr || p.residual != nullptr || p.accumulate != 0;
        p.tma_out = aligned16(p.C) && (p.ldc % PER16) == 0 && !(p.residual != nullptr && p.accumulate != 0) &&
                    (p.residual == nullptr || (aligned16(p.residual) && (p.ldr % PER16) == 0)) &&
                    (p.bias == nullptr || aligned16(p.bias)) && (p.N % PER16 == 0 || !reads);
        if (p.tma_out) {
            int rc = make_tensor_map_out(&mc, p.C, static_cast<int>(sizeof(TC)), p.N, p.M, p.ldc, 32);
            if (rc != PK_OK) return rc;
            if (p.residual != nullptr) {   // the kernel's map_u slot: U in SwiGLU mode, else the residual
                rc = make_tensor_map_out(&mu, p.residual, static_cast<int>(sizeof(TC)), p.N, p.M, p.ldr, 32);
                if (rc != PK_OK) return rc;
            }
        }
    }
    if (p.rope_cs != nullptr && !p.tma_out) {
        set_error("pk_gemm_rope: the output cannot go through the staged epilogue");
        return PK_ERR_UNSUPPORTED;
    }
    int64_t pairs = max_pairs;
    if (pairs > tiles * p.splits) pairs = tiles * p.splits;
    kern<<<static_cast<unsigned>(2 * pairs), SWIGLU ? T2_THREADS_SWIGLU : T2_THREADS, T2_SMEM_BYTES, st>>>(ma, mb, mb2, mc, mu, my, p);
    PK_LAUNCH_CHECK();
    if (p.splits > 1)
        return gemm_splitk_reduce(st, c_dtype, p.partial, p.splits, p.slab, p.pstride, p.M, p.N, p.C, p.ldc, p.accumulate,
                                  p.bias, p.residual, p.ldr);
    return PK_OK;
}

}  // namespace

int gemm_tc2_launch(cudaStream_t st, int c_dtype, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                    const void* B, int64_t ldb, void* C, int64_t ldc, int accumulate, const float* bias, const void* residual,
                    int64_t ldr, const RopeEpilogue* rope) {
    const int a_mn = ta ? 1 : 0, b_mn = tb ? 0 : 1;
    CUtensorMap ma, mb;
    int rc;
    // same boxes as the one-CTA kernel, except that a CTA takes 128 of the tile's 256 B columns
    if (!a_mn) rc = make_tensor_map(&ma, A, K, M, lda, T2_BK, T2_BM);
    else rc = make_tensor_map(&ma, A, M, K, lda, 64, T2_BK);
    if (rc != PK_OK) return rc;
    if (!b_mn) rc = make_tensor_map(&mb, B, K, N, ldb, T2_BK, T2_BN / 2);
    else rc = make_tensor_map(&mb, B, N, K, ldb, 64, T2_BK);
    if (rc != PK_OK) return rc;
    T2Params p;
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.bias = bias; p.residual = residual; p.ldr = ldr;
    p.accumulate = accumulate;
    p.a_mn_major = a_mn; p.b_mn_major = b_mn;
    p.U = nullptr; p.Y = nullptr; p.ldy = 0;
    p.rope_cs = nullptr; p.rope_pos = nullptr; p.rope_half = 0; p.rope_cols = 0; p.rope_npos = 0; p.rope_sign = 1.0f;
    if (rope != nullptr) {
        p.rope_cs = rope->cos_sin; p.rope_pos = rope->pos; p.rope_half = rope->half;
        p.rope_cols = rope->cols; p.rope_npos = rope->n_pos; p.rope_sign = rope->sign;
    }
    if (c_dtype == PK_F32) return launch2<float, false>(st, ma, mb, mb, p, c_dtype);
    return launch2<bf16, false>(st, ma, mb, mb, p, c_dtype);
}

// y = silu(A Wg) * (A Wu) in one pass over A (SwiGLU pair mode of the kernel above). Wg, Wu are
// [K, N] row-major (MN-major operands); G / U (nullable, both or neither) receive the two products.
int gemm_tc2_swiglu_launch(cudaStream_t st, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* Wg,
                           int64_t ldg, const void* Wu, int64_t ldu, void* G, void* U, int64_t ldgu, void* Y, int64_t ldy) {
    CUtensorMap ma, mg, mu;
    int rc = make_tensor_map(&ma, A, K, M, lda, T2_BK, T2_BM);
    if (rc != PK_OK) return rc;
    if ((rc = make_tensor_map(&mg, Wg, N, K, ldg, 64, T2_BK)) != PK_OK) return rc;
    if ((rc = make_tensor_map(&mu, Wu, N, K, ldu, 64, T2_BK)) != PK_OK) return rc;
    T2Params p;
    p.M = M; p.N = N; p.K = K;
    p.C = G; p.ldc = ldgu;
    p.bias = nullptr; p.residual = nullptr; p.ldr = 0;
    p.accumulate = 0;
    p.a_mn_major = 0; p.b_mn_major = 1;
    p.U = U; p.Y = Y; p.ldy = ldy;
    p.rope_cs = nullptr; p.rope_pos = nullptr; p.rope_half = 0; p.rope_cols = 0; p.rope_npos = 0; p.rope_sign = 1.0f;
    return launch2<bf16, true>(st, ma, mg, mu, p, PK_BF16);
}


}  // namespace pk

