// Fused Q8_0 dequantise-GEMM with a LoRA side path on CTA pairs (tcgen05 cta_group::2).
//
//     C[M,N] (+)= A[M,K] . deq(W) + XA[M,r] . L (+ bias) (+ residual)
//
// W is a frozen weight stored as int8 with one fp16 scale per 32 values along a row. It is never
// expanded in global memory: TMA brings a 64-deep k slice of int8 into shared memory, four
// converter warps turn it into bf16 -- float(q) * float(scale), one fp32 multiply and one rounding,
// the bits pk_q8_dequantize produces -- and write it in the 128-byte-swizzled layout that
// tcgen05.mma reads as its B operand. The LoRA term is one more k slice of the same accumulator:
// after the last slice of W the producer loads XA as the A operand and L as the B operand (both
// bf16, by TMA, zero-filled beyond the rank) and the issuer adds ceil(r / 16) MMAs.
//
// Tile schedule, pairing and epilogue are those of pk_gemm_tc2.cu: a cluster of two CTAs owns a
// 256 x 256 output tile, CTA r holds rows r*128.. of A and of the accumulator and columns r*128..
// of B; the leader issues tcgen05.mma.cta_group::2. Roles in each CTA (448 threads):
//   warp 0       producer: lane 0 issues the TMA loads -- the A slice (completes on the leader's
//                "full" barrier) and the raw int8 half slice of W (this CTA's "raw" barrier); all 32
//                lanes copy the slice's fp16 scales into shared memory with cp.async, whose
//                completion is counted on the same "raw" barrier
//   warp 1       tensor-memory allocation; in the leader one thread issues the MMAs
//   warps 2..5   epilogue: rows leave through shared-memory boxes and TMA stores, what is added to
//                them (residual, C) arrives by TMA (pk_gemm_epilogue.cuh); direct stores otherwise
//   warps 6..13  converters: int8 + scale -> swizzled bf16, fence.proxy.async, then one arrival per
//                warp on the LEADER's "full" barrier, which therefore completes when the A bytes of
//                both CTAs have landed and all 16 converter warps of the pair are done: the issuer
//                waits once per k slice
// Measured (16384 x 4864 x 896, TFLOP/s): with row-per-thread stores in the epilogue 836, with
// the staged epilogue 952 (the bf16 pair kernel on an already expanded weight: 1201 -> 1413); the
// k loop of this shape is only 14 slices, so a tile's epilogue is as long as its MMAs. With the
// converters idle (arrivals only) the old form reached 1005, so converting costs about a sixth.
// Three ring stages cost 6 %, five give nothing over four; half the conversion work per slice
// changes nothing either, so neither the ring's depth nor the converters' throughput is the
// bound: what remains against the bf16 kernel is the extra hop of every slice (raw bytes land ->
// converter warps wake, convert, arrive on the leader's barrier -> the issuer wakes). Sixteen
// converter warps (two groups on alternate k slices) need more registers than 704 threads
// leave the epilogue (517); eight epilogue warps were slower (781). Not kept earlier:
// converters loading the int8 slice from global memory into registers instead of staging it by
// TMA 723; a cluster-scope release on every converter arrival 495; a second barrier for the
// issuer to wait on 340.
// Both layouts of W are served: trans_w = 0 (W is [K, N], the operand is MN-major; forward) and
// trans_w = 1 (W is [N, K], K-major; input gradient). The k order is fixed and the products are
// the ones a bf16 GEMM over the expanded weight would form, so the result equals
// pk_q8_dequantize + pk_gemm bit for bit.
// Every mbarrier wait is bounded (status word, no trap); both CTAs always reach the two
// cluster-wide barriers at the start and the end.
#include <cuda.h>
#include <cuda_fp16.h>

#include "pk_common.cuh"
#include "pk_tc.cuh"
#include "pk_gemm_epilogue.cuh"

namespace pk {

PK_DEFINE_WAITCTL(gemm_q8)

namespace {

using namespace tc;

constexpr int Q8_BM = 128;          // rows per CTA; the pair covers 256
constexpr int Q8_BN = 256;
constexpr int Q8_BK = 64;
constexpr int Q8_CONV_WARP0 = 6;    // first converter warp
constexpr int Q8_CONV_WARPS = 8;    // converter warps that work on one k slice
constexpr int Q8_THREADS = (Q8_CONV_WARP0 + Q8_CONV_WARPS) * 32;
constexpr int Q8_CONV_ITERS = 1024 / (Q8_CONV_WARPS * 32);   // 16-byte operand units per thread and k slice (4)
constexpr int Q8_STAGES = 4;
constexpr int Q8_A_BYTES = Q8_BM * Q8_BK * 2;          // 16 KiB
constexpr int Q8_B_BYTES = (Q8_BN / 2) * Q8_BK * 2;    // 16 KiB: this CTA's half of B in bf16
constexpr int Q8_RAW_BYTES = (Q8_BN / 2) * Q8_BK;      // 8 KiB: the same half as int8
constexpr int Q8_STAGE_BYTES = Q8_A_BYTES + Q8_B_BYTES + Q8_RAW_BYTES;
constexpr int Q8_SCALE_BYTES = 512;                    // fp16 scales of one half slice: 64 x 4 or 128 x 2
constexpr int Q8_EPI_BOXES = 4;                        // per epilogue warp: boxes of 32 rows x 64 bytes (pk_gemm_epilogue.cuh)
constexpr int Q8_EPI_BYTES = 4 * Q8_EPI_BOXES * EPI_BOX_BYTES;
constexpr int Q8_SMEM_BYTES = Q8_STAGES * (Q8_STAGE_BYTES + Q8_SCALE_BYTES) + Q8_EPI_BYTES + 1024 + 512;

struct Q8Params {
    int64_t M, N, K;
    void* C;
    int64_t ldc;
    const float* bias;
    const void* residual;
    int64_t ldr;
    int accumulate;
    const __half* scales;   // [rows of W, cols of W / 32]
    int64_t scale_ld;       // cols of W / 32
    int lora_ksteps;        // ceil(r / 16); 0: no LoRA slice
    int tma_out;            // 1: output through shared-memory staging and TMA stores (map_c, map_r)
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The converters' arrival on the leader's barrier. Their shared-memory writes are read by the
// tensor core (async proxy) of their own SM and have been ordered for it by fence.proxy.async;
// the arrival itself needs no cluster-wide release of generic writes, which costs about a
// thousand cycles per arrival and would sit on the critical path of every k slice.
__device__ __forceinline__ void remote_arrive_cta_release(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
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
__device__ __forceinline__ void commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(static_cast<uint16_t>(3))
        : "memory");
}
__host__ __device__ inline uint32_t idesc_pair(int n, int b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;                                     // fp32 accumulator
    d |= 1u << 7;                                     // A bf16
    d |= 1u << 10;                                    // B bf16
    d |= static_cast<uint32_t>(b_mn_major & 1) << 16;
    d |= static_cast<uint32_t>(n >> 3) << 17;
    d |= static_cast<uint32_t>(256 >> 4) << 24;       // M of the pair
    return d;
}
__device__ __forceinline__ bool waitq(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait(bar, parity, abort_flag, &g_gemm_q8_ctl);
}
// 4- or 8-byte asynchronous copy global -> shared; src_bytes == 0 writes zeros instead.
template <int BYTES>
__device__ __forceinline__ void cp_async_small(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(dst), "l"(src), "n"(BYTES), "r"(src_bytes) : "memory");
}
// One arrival on the barrier once all earlier cp.async of this thread have landed (the arrival is
// part of the barrier's expected count).
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
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

// Eight int8 (two 32-bit words) times one scale -> eight bf16 (one 16-byte operand unit).
// A byte b = q + 128 placed in the low mantissa bits of 2^23 reads as the float 8388608 + b;
// subtracting 8388736 gives float(q) exactly. Then one fp32 multiply and one rounding to bf16.
__device__ __forceinline__ uint4 dequant8(uint32_t w0, uint32_t w1, float s) {
    const uint64_t bias = f2_pack(-8388736.0f, -8388736.0f);
    const uint64_t ss = f2_pack(s, s);
    uint32_t out[4];
    const uint32_t w[2] = {w0 ^ 0x80808080u, w1 ^ 0x80808080u};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t lo = __byte_perm(w[h], 0x4B000000u, 0x7650 + 2 * e);
            const uint32_t hi = __byte_perm(w[h], 0x4B000000u, 0x7651 + 2 * e);
            const uint64_t v = f2_mul(f2_add(f2_pack_bits(lo, hi), bias), ss);
            float a, b;
            f2_unpack(v, a, b);
            const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
            out[h * 2 + e] = *reinterpret_cast<const uint32_t*>(&p);
        }
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

template <typename TC, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Q8_THREADS, 1)
gemm_q8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_xa, const __grid_constant__ CUtensorMap map_l,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_r, const Q8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* scale_smem = smem + Q8_STAGES * Q8_STAGE_BYTES;   // [STAGES][Q8_SCALE_BYTES]
    uint8_t* epi_smem = scale_smem + Q8_STAGES * Q8_SCALE_BYTES;   // [4 warps][EPI_BOXES][2048]
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Q8_EPI_BYTES);
    uint64_t* full_bar = bars;                        // [STAGES]  leader: TMA bytes of A (and of the LoRA slice) of both
                                                      //           CTAs + the 16 converter warps of the pair
    uint64_t* empty_bar = bars + Q8_STAGES;           // [STAGES]  per CTA, both signalled by the leader's commits
    uint64_t* raw_full = bars + 2 * Q8_STAGES;        // [STAGES]  per CTA: its int8 half slice and its scales have landed
    uint64_t* acc_full = bars + 3 * Q8_STAGES;        // [2]       per CTA, both signalled by the leader
    uint64_t* acc_empty = bars + 3 * Q8_STAGES + 2;   // [2]       leader: 8 epilogue warps of the pair
    uint64_t* in_bar = bars + 3 * Q8_STAGES + 4;      // [4 warps][EPI_BOXES] per CTA: residual / C box has landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(in_bar + 4 * Q8_EPI_BOXES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int64_t tiles_m = (p.M + 2 * Q8_BM - 1) / (2 * Q8_BM), tiles_n = (p.N + Q8_BN - 1) / Q8_BN;
    const int64_t n_tiles = tiles_m * tiles_n;
    const int k_blocks = static_cast<int>((p.K + Q8_BK - 1) / Q8_BK);
    const bool lora = p.lora_ksteps > 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Q8_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1 + 2 * Q8_CONV_WARPS);   // producer's expect_tx + converter warps
            mbar_init(smem_u32(&empty_bar[s]), 1);
            mbar_init(smem_u32(&raw_full[s]), 1 + 32);                   // lane 0's expect_tx + one per producer lane
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full[a]), 1);
            mbar_init(smem_u32(&acc_empty[a]), 8);
        }
        for (int b = 0; b < 4 * Q8_EPI_BOXES; ++b) mbar_init(smem_u32(&in_bar[b]), 1);
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
        // ------------------------------------------------ producer (both CTAs): TMA by lane 0, scales by all lanes
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const unsigned short* sp = reinterpret_cast<const unsigned short*>(p.scales);
        for (int64_t w = pair; w < n_tiles && ok; w += n_pairs) {
            const int32_t m0 = static_cast<int32_t>((w / tiles_n) * (2 * Q8_BM) + rank * Q8_BM);
            const int32_t n0 = static_cast<int32_t>((w % tiles_n) * Q8_BN + rank * (Q8_BN / 2));
            const int nb = k_blocks + (lora ? 1 : 0);
            for (int kb = 0; kb < nb; ++kb) {
                if (lane == 0) ok = waitq(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t rb = smem_u32(&raw_full[stage]);
                if (lane == 0) {
                    const uint32_t fb_local = smem_u32(&full_bar[stage]);
                    const uint32_t fb = map_to_rank(fb_local, 0);   // the leader's barrier counts both CTAs' bytes
                    const uint32_t sa = smem_u32(smem + stage * Q8_STAGE_BYTES);
                    const uint32_t sb = sa + Q8_A_BYTES;
                    const uint32_t sr = sb + Q8_B_BYTES;
                    if (kb < k_blocks) {
                        const int32_t k0 = kb * Q8_BK;
                        if (leader) mbar_expect_tx(fb_local, 2 * Q8_A_BYTES);
                        tma_load_2d_pair(sa, &map_a, k0, m0, fb);                 // box 64(k) x 128(m)
                        mbar_expect_tx(rb, Q8_RAW_BYTES);
                        if (B_MN) tma_load_2d(sr, &map_w, n0, k0, rb);            // box 128(n) x 64(k) bytes
                        else tma_load_2d(sr, &map_w, k0, n0, rb);                 // box 64(k) x 128(n) bytes
                    } else {
                        // LoRA slice: XA as the A operand, L as the B operand, both already bf16
                        if (leader) mbar_expect_tx(fb_local, 2 * (Q8_A_BYTES + Q8_B_BYTES));
                        tma_load_2d_pair(sa, &map_xa, 0, m0, fb);                 // box 64(r) x 128(m), zero beyond r
                        if (B_MN) {
#pragma unroll
                            for (int c = 0; c < (Q8_BN / 2) / 64; ++c)            // boxes 64(n) x 64(r)
                                tma_load_2d_pair(sb + c * 8192, &map_l, n0 + c * 64, 0, fb);
                        } else {
                            tma_load_2d_pair(sb, &map_l, 0, n0, fb);              // box 64(r) x 128(n)
                        }
                        mbar_arrive(rb);   // stands for the expect_tx arrival: nothing to convert in this slice
                    }
                }
                if (kb < k_blocks) {
                    // fp16 scales of this half slice, laid out [row of the slice][scale column]
                    const uint32_t ss = smem_u32(scale_smem + stage * Q8_SCALE_BYTES);
                    const int64_t k0 = static_cast<int64_t>(kb) * Q8_BK;
                    if (B_MN) {   // 64 k rows x 4 scales (8 bytes) each
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const int row = lane + 32 * i;
                            const bool in = k0 + row < p.K && n0 < p.N;
                            const unsigned short* src = in ? sp + (k0 + row) * p.scale_ld + (n0 >> 5) : sp;
                            cp_async_small<8>(ss + row * 8, src, in ? 8u : 0u);
                        }
                    } else {      // 128 n rows x 2 scales (4 bytes) each
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int row = lane + 32 * i;
                            const bool in = n0 + row < p.N && k0 < p.K;
                            const unsigned short* src = in ? sp + static_cast<int64_t>(n0 + row) * p.scale_ld + (k0 >> 5) : sp;
                            cp_async_small<4>(ss + row * 4, src, in ? 4u : 0u);
                        }
                    }
                    cp_async_arrive(rb);
                } else {
                    mbar_arrive(rb);
                }
                if (++stage == Q8_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            const uint32_t idesc = idesc_pair(Q8_BN, B_MN ? 1 : 0);
            const uint32_t b_flags = ((B_MN ? 8192u : 16u) >> 4) << 16;
            const uint32_t b_step = (B_MN ? 2048u : 32u) >> 4;
            const uint32_t a_lo0 = ((smem_u32(smem) & 0x3ffffu) >> 4) | ((16u >> 4) << 16);
            const uint32_t b_lo0 = (((smem_u32(smem) + Q8_A_BYTES) & 0x3ffffu) >> 4) | b_flags;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int64_t w = pair; w < n_tiles && ok; w += n_pairs) {
                if (!waitq(smem_u32(&acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * Q8_BN);
                const int nb = k_blocks + (lora ? 1 : 0);
                for (int kb = 0; kb < nb; ++kb) {
                    if (!waitq(smem_u32(&full_bar[stage]), phase, abort_flag)) { ok = false; break; }
                    fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (Q8_STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (Q8_STAGE_BYTES >> 4);
                    if (kb < k_blocks) {
#pragma unroll
                        for (int k = 0; k < Q8_BK / 16; ++k)
                            mma2_ss(d_tmem, a_lo + k * 2u, b_lo + k * b_step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    } else {
                        for (int k = 0; k < p.lora_ksteps; ++k)
                            mma2_ss(d_tmem, a_lo + k * 2u, b_lo + k * b_step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    commit_pair(smem_u32(&empty_bar[stage]));   // frees the stage in both CTAs
                    if (++stage == Q8_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                commit_pair(smem_u32(&acc_full[acc]));          // accumulator complete, both CTAs
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else if (warp >= Q8_CONV_WARP0) {
        // ------------------------------------------------ converters (both CTAs)
        const int c = threadIdx.x - Q8_CONV_WARP0 * 32;   // 0..255
        // MN-major (W is [K, N]): thread = (k row r0 + 16 i, 8 columns starting at 8 j), j < 16
        // K-major  (W is [N, K]): thread = (row r0 + 32 i, 8 k values starting at 8 j), j < 8
        const int j = B_MN ? (c & 15) : (c & 7);
        const int r0 = B_MN ? (c >> 4) : (c >> 3);
        constexpr int raw_pitch = B_MN ? 128 : 64;
        constexpr int row_step = B_MN ? 16 : 32;
        constexpr int scale_pitch = B_MN ? 8 : 4;   // bytes of scales per row of the slice
        const int raw_off = r0 * raw_pitch + 8 * j;
        // destination of iteration 0; iteration i adds row_step rows (the swizzle term (row & 7) does not change)
        const int dst_off = B_MN ? ((j >> 3) * 8192 + r0 * 128 + (((j & 7) ^ (r0 & 7)) << 4))
                                 : (r0 * 128 + ((j ^ (r0 & 7)) << 4));
        const int scale_off = r0 * scale_pitch + (j >> 2) * 2;
        const uint32_t leader_full0 = map_to_rank(smem_u32(&full_bar[0]), 0);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int64_t w = pair; w < n_tiles && ok; w += n_pairs) {
            const int nb = k_blocks + (lora ? 1 : 0);
            for (int kb = 0; kb < nb; ++kb) {
                if (!waitq(smem_u32(&raw_full[stage]), phase, abort_flag)) { ok = false; break; }
                if (kb < k_blocks) {
                    const uint8_t* raw = smem + stage * Q8_STAGE_BYTES + Q8_A_BYTES + Q8_B_BYTES + raw_off;
                    uint8_t* dst = smem + stage * Q8_STAGE_BYTES + Q8_A_BYTES + dst_off;
                    const uint8_t* scl = scale_smem + stage * Q8_SCALE_BYTES + scale_off;
#pragma unroll
                    for (int i = 0; i < Q8_CONV_ITERS; ++i) {
                        const uint2 q = *reinterpret_cast<const uint2*>(raw + i * row_step * raw_pitch);
                        const float sc = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(scl + i * row_step * scale_pitch)));
                        *reinterpret_cast<uint4*>(dst + i * row_step * 128) = dequant8(q.x, q.y, sc);
                    }
                    fence_async_smem();   // generic-proxy writes -> visible to the tensor core's reads
                }
                // (the LoRA slice has nothing to convert: the arrival only keeps the barrier's count)
                __syncwarp();
                if (lane == 0) remote_arrive_cta_release(leader_full0 + stage * 8);
                if (++stage == Q8_STAGES) { stage = 0; phase ^= 1u; }
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
        out.boxes = epi_smem + (warp - 2) * (Q8_EPI_BOXES * EPI_BOX_BYTES);
        out.in_bar = in_bar + (warp - 2) * Q8_EPI_BOXES;
        out.out = &map_c;
        out.in = Rsd != nullptr ? &map_r : (p.accumulate ? &map_c : nullptr);
        out.bias = p.bias;
        out.N = p.N;
        out.slab = -1;
        out.uc = 0;
        bool ok = true;
        for (int64_t w = pair; w < n_tiles && ok; w += n_pairs) {
            const int64_t m0 = (w / tiles_n) * (2 * Q8_BM) + rank * Q8_BM, n0 = (w % tiles_n) * Q8_BN;
            const int64_t m = m0 + quad * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * Q8_BN);
            if (p.tma_out) {
                ok = staged_epilogue<TC, Q8_BN, Q8_EPI_BOXES>(out, n0, static_cast<int32_t>(m0 + quad * 32), t_row,
                                                              smem_u32(&acc_full[acc]), acc_phase, abort_flag, &g_gemm_q8_ctl, lane);
                if (!ok) break;
            } else {
                ok = waitq(smem_u32(&acc_full[acc]), acc_phase, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fence_after();
            }
#pragma unroll 1
            for (int ch = 0; ch < (p.tma_out ? 0 : Q8_BN / 32); ++ch) {
                const int64_t c0 = n0 + ch * 32;
                if (c0 >= p.N) break;  // uniform across the warp
                uint32_t r[32];
                tmem_ld32(t_row + static_cast<uint32_t>(ch * 32), r);
                tmem_wait_ld();
                if (m < p.M) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int64_t cc = c0 + g * 8;
                        if (cc >= p.N) break;   // N is a multiple of 8
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g * 8 + e]);
                        if (p.bias) {
                            float b[8];
                            load8<float>(p.bias + cc, b);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] += b[e];
                        }
                        if (Rsd) {
                            float q[8];
                            load8<TC>(Rsd + m * p.ldr + cc, q);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] += q[e];
                        }
                        if (p.accumulate) {
                            float q[8];
                            load8<TC>(C + m * p.ldc + cc, q);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] += q[e];
                        }
                        store8<TC>(C + m * p.ldc + cc, v);
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
    if (warp >= 2 && warp < Q8_CONV_WARP0 && lane == 0) bulk_wait_all();   // this thread's TMA stores are complete
    fence_before();
    __syncthreads();
    cluster_sync_all();   // no CTA leaves while the other may still signal its barriers or read its shared memory
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// Prepares one instantiation of the kernel on the current device (shared-memory opt-in) and tells
// how many CTA pairs of it the device holds at once; cached per device and per instantiation
// (the template parameters keep the caches of the four kernels apart).
template <typename TC, bool B_MN>
int max_pairs_of(int* out) {
    auto kern = gemm_q8_kernel<TC, B_MN>;
    static int cache[64] = {0};
    static bool attr_done[64] = {false};
    int dev = 0;
    PK_CHECK_CUDA(cudaGetDevice(&dev));
    PK_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    if (!attr_done[dev]) {
        PK_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Q8_SMEM_BYTES));
        attr_done[dev] = true;
    }
    if (cache[dev] == 0) {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2));
        probe.blockDim = dim3(Q8_THREADS);
        probe.dynamicSmemBytes = Q8_SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        probe.attrs = &attr;
        probe.numAttrs = 1;
        int n = 0;
        PK_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &probe));
        PK_REQUIRE(n > 0, "no CTA pair of the Q8_0 GEMM fits on this GPU");
        cache[dev] = n;
    }
    *out = cache[dev];
    return PK_OK;
}


template <typename TC, bool B_MN>
int launch_q8(cudaStream_t st, const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mxa, const CUtensorMap& ml,
              Q8Params p) {
    auto kern = gemm_q8_kernel<TC, B_MN>;
    // staged output (pk_gemm_epilogue.cuh) when C, the residual and the bias can be reached in 16-byte groups
    constexpr int64_t PER16 = 16 / static_cast<int64_t>(sizeof(TC));
    const bool reads = p.bias != nullptr || p.residual != nullptr || p.accumulate != 0;
    p.tma_out = aligned16(p.C) && (p.ldc % PER16) == 0 && !(p.residual != nullptr && p.accumulate != 0) &&
                (p.residual == nullptr || (aligned16(p.residual) && (p.ldr % PER16) == 0)) &&
                (p.bias == nullptr || aligned16(p.bias)) && (p.N % PER16 == 0 || !reads);
    CUtensorMap mc = ma, mr = ma;
    if (p.tma_out) {
        int rc = make_tensor_map_out(&mc, p.C, static_cast<int>(sizeof(TC)), p.N, p.M, p.ldc, 32);
        if (rc == PK_OK && p.residual != nullptr)
            rc = make_tensor_map_out(&mr, p.residual, static_cast<int>(sizeof(TC)), p.N, p.M, p.ldr, 32);
        if (rc != PK_OK) return rc;
    }
    int max_pairs = 0;
    const int rc = max_pairs_of<TC, B_MN>(&max_pairs);
    if (rc != PK_OK) return rc;
    const int64_t tiles = ((p.M + 2 * Q8_BM - 1) / (2 * Q8_BM)) * ((p.N + Q8_BN - 1) / Q8_BN);
    int64_t pairs = max_pairs;
    if (pairs > tiles) pairs = tiles;
    kern<<<static_cast<unsigned>(2 * pairs), Q8_THREADS, Q8_SMEM_BYTES, st>>>(ma, mw, mxa, ml, mc, mr, p);
    PK_LAUNCH_CHECK();
    return PK_OK;
}

}  // namespace

void gemm_note_path(int path);  // pk_gemm_simt.cu

}  // namespace pk

using namespace pk;

extern "C" int pk_gemm_q8_lora(void* stream, int c_dtype, int trans_w, int64_t M, int64_t N, int64_t K, const void* A,
                               int64_t lda, const int8_t* Wq, const uint16_t* scales, const void* XA, int64_t ldxa,
                               const void* L, int64_t ldl, int r, void* C, int64_t ldc, int accumulate, const float* bias,
                               const void* residual, int64_t ldr) {
    PK_REQUIRE(valid_dtype(c_dtype), "bad dtype");
    PK_REQUIRE(M >= 0 && N >= 0 && K >= 0 && r >= 0, "negative shape");
    if (M == 0 || N == 0) return PK_OK;
    PK_REQUIRE(K > 0, "empty contraction");
    PK_REQUIRE(A && Wq && scales && C, "null pointer");
    PK_REQUIRE(lda >= K && ldc >= N, "leading dimension too small");
    PK_REQUIRE(residual == nullptr || ldr >= N, "residual leading dimension too small");
    const bool lora = XA != nullptr && r > 0;
    PK_REQUIRE(!lora || (L != nullptr && ldxa >= r && ldl >= (trans_w ? r : N)), "bad LoRA operands");
    const int64_t w_cols = trans_w ? K : N;
    // the scales of a half slice are copied as 8-byte (W is [K, N]) or 4-byte (W is [N, K]) pieces
    bool ok = (trans_w ? w_cols % 64 == 0 : w_cols % 128 == 0) && aligned16(scales) && lda % 8 == 0 && ldc % 8 == 0 && N % 8 == 0 && aligned16(A) && aligned16(Wq) && aligned16(C) &&
              (residual == nullptr || (aligned16(residual) && ldr % 8 == 0)) &&
              (bias == nullptr || aligned16(bias)) && M < (int64_t(1) << 31) && N < (int64_t(1) << 31) && K < (int64_t(1) << 31);
    if (lora) ok = ok && r % 8 == 0 && r <= 64 && ldxa % 8 == 0 && ldl % 8 == 0 && aligned16(XA) && aligned16(L);
    if (!ok) {
        set_error("pk_gemm_q8_lora: shape or alignment outside what the kernel takes (M %lld N %lld K %lld r %d)",
                  static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K), r);
        return PK_ERR_UNSUPPORTED;
    }
    cudaStream_t st = as_stream(stream);
    CUtensorMap ma, mw, mxa, ml;
    int rc = tc::make_tensor_map(&ma, A, K, M, lda, Q8_BK, Q8_BM);
    if (rc != PK_OK) return rc;
    // the int8 matrix as bytes: [K, N] (box 128 n x 64 k) or [N, K] (box 64 k x 128 n)
    if (!trans_w) rc = tc::make_tensor_map_u8(&mw, Wq, N, K, N, Q8_BN / 2, Q8_BK);
    else rc = tc::make_tensor_map_u8(&mw, Wq, K, N, K, Q8_BK, Q8_BN / 2);
    if (rc != PK_OK) return rc;
    if (lora) {
        rc = tc::make_tensor_map(&mxa, XA, r, M, ldxa, Q8_BK, Q8_BM);
        if (rc != PK_OK) return rc;
        if (!trans_w) rc = tc::make_tensor_map(&ml, L, N, r, ldl, 64, Q8_BK);   // L [r, N]: boxes 64(n) x 64(r)
        else rc = tc::make_tensor_map(&ml, L, r, N, ldl, Q8_BK, Q8_BN / 2);     // L [N, r]: box 64(r) x 128(n)
        if (rc != PK_OK) return rc;
    } else {
        mxa = ma;   // never dereferenced
        ml = ma;
    }
    Q8Params p;
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.bias = bias; p.residual = residual; p.ldr = ldr;
    p.accumulate = accumulate;
    p.scales = reinterpret_cast<const __half*>(scales);
    p.scale_ld = w_cols / 32;
    p.lora_ksteps = lora ? (r + 15) / 16 : 0;
    ProfScope prof(PROF_GEMM_TC, 2.0 * M * N * (K + (lora ? r : 0)), st);
    gemm_note_path(4);
    note_launch(PATH_GEMM_Q8);
    if (!trans_w) {
        if (c_dtype == PK_F32) return launch_q8<float, true>(st, ma, mw, mxa, ml, p);
        return launch_q8<bf16, true>(st, ma, mw, mxa, ml, p);
    }
    if (c_dtype == PK_F32) return launch_q8<float, false>(st, ma, mw, mxa, ml, p);
    return launch_q8<bf16, false>(st, ma, mw, mxa, ml, p);
}
