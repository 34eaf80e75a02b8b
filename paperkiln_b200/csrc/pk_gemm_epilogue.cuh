// Epilogue of the tcgen05 GEMM kernels: accumulator rows leave through shared memory and TMA.
//
// A thread of an epilogue warp owns one accumulator row (tensor-memory lane). Storing that row
// from registers makes every warp-level store touch 32 different lines, and reading what is to be
// added (a residual, or C itself when accumulating) the same way costs a round trip per 16
// bytes; both made the epilogue, not the MMAs, the bound of every GEMM with a short k loop
// (16384 x 4864 x 896 with a residual: 548 -> 1040 TFLOP/s with this form; 2048 x 2048 weights
// with a residual 971 -> 1114). Here each warp has BOXES boxes of 32 rows x 64 bytes in shared
// memory (64-byte swizzle, so the 16-byte accesses of a warp spread over the banks) that take
// turns: what is to be added arrives in the box by TMA, BOXES - 1 units ahead -- the first
// ones before the accumulator is even complete --, each thread adds its 64 bytes in place, and
// lane 0 hands the box to a TMA store, which writes whole lines and clips at the edges of C.
// The arithmetic and its order (accumulator + bias, + residual or + C, one rounding) are those of
// the direct form, so the results are bit-identical.
#pragma once

#include "pk_common.cuh"
#include "pk_tc.cuh"

namespace pk {
namespace tc {

constexpr int EPI_BOX_BYTES = 2048;   // 32 rows x 64 bytes

template <int COLS>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[COLS]);
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }

// v[0 .. 16 / sizeof(TC)) += the elements packed in 16 bytes
template <typename TC>
__device__ __forceinline__ void add_packed(float* v, uint4 q);
template <>
__device__ __forceinline__ void add_packed<float>(float* v, uint4 q) {
    v[0] += __uint_as_float(q.x); v[1] += __uint_as_float(q.y); v[2] += __uint_as_float(q.z); v[3] += __uint_as_float(q.w);
}
template <>
__device__ __forceinline__ void add_packed<bf16>(float* v, uint4 q) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] += __uint_as_float(w[i] << 16);
        v[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
    }
}
// 16 bytes of output from 16 / sizeof(TC) values
template <typename TC>
__device__ __forceinline__ uint4 pack_out(const float* v);
template <>
__device__ __forceinline__ uint4 pack_out<float>(const float* v) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
template <>
__device__ __forceinline__ uint4 pack_out<bf16>(const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
// byte offset of 16-byte unit j of row `lane` inside a box (64-byte swizzle: bits 4-5 ^= bits 7-8)
__device__ __forceinline__ int box_offset(int lane, int j) { return lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4); }

struct StagedOut {
    uint8_t* boxes;            // this warp's BOXES boxes (512-byte aligned)
    uint64_t* in_bar;          // this warp's BOXES barriers (count 1): "the box's input has landed"
    const CUtensorMap* out;    // C (2-D: columns, rows) or the split-K partial slabs (3-D: columns, rows, slab)
    const CUtensorMap* in;     // what is added to the accumulator (residual, or C when accumulating); null: nothing
    const float* bias;         // nullable; N is then a multiple of 4
    int64_t N;                 // columns of C
    int32_t slab;              // >= 0: `out` is 3-D and this is the slab
    uint32_t uc;               // units staged so far by this warp: box index and barrier phase rotate with it
    // Rotary embedding on the way out (bf16 outputs; q and k projections): columns [0, rope_cols)
    // are heads of 2 * rope_half columns whose adjacent pairs are turned by the angle of the row's
    // position, after the value has been rounded to bf16 as a separate GEMM would have stored it.
    const float* rope_cs = nullptr;    // (cos, sin) per [position, pair]; null: no rotation
    const int32_t* rope_pos = nullptr; // position of every row of C
    int rope_half = 0;                 // 32 or 64: a 32-column unit lies inside one head
    int64_t rope_cols = 0;
    int64_t rope_npos = 0;
    float rope_sign = 1.0f;            // -1: inverse rotation
    int64_t M = 0;                     // rows of C (only read when rotating)
};

// Writes the 32 x BN block of one warp: accumulator columns [0, BN) at tensor-memory address
// t_row -> C columns n0.., rows y0 .. y0 + 31. Waits for the accumulator (acc_bar / acc_parity)
// after it has requested the first inputs. Returns false when a bounded wait gave up.
template <typename TC, int BN, int BOXES, bool ROPE = false>
__device__ __forceinline__ bool staged_epilogue(StagedOut& s, int64_t n0, int32_t y0, uint32_t t_row, uint32_t acc_bar,
                                                uint32_t acc_parity, volatile int* abort_flag, WaitCtl* ctl, int lane) {
    constexpr int UC = 64 / static_cast<int>(sizeof(TC));   // output columns in 64 bytes
    constexpr int UNITS = BN / UC;
    const int64_t units_left = (s.N - n0 + UC - 1) / UC;
    const int n_units = units_left < UNITS ? static_cast<int>(units_left) : UNITS;
    const bool reads = s.in != nullptr;
    if (reads && lane == 0) {
        bulk_wait_read<0>();   // the stores of the previous block have read their boxes
        for (int u = 0; u < BOXES - 1 && u < n_units; ++u) {
            const uint32_t bx = (s.uc + u) & (BOXES - 1);
            const uint32_t bar = smem_u32(&s.in_bar[bx]);
            mbar_expect_tx(bar, EPI_BOX_BYTES);
            tma_load_2d(smem_u32(s.boxes + bx * EPI_BOX_BYTES), s.in, static_cast<int32_t>(n0 + u * UC), y0, bar);
        }
    }
    // rotary embedding: this row's (cos, sin) table row; the 16 pairs of a unit are fetched one unit
    // ahead (the first before the accumulator is complete) so that their latency is not in the loop
    const bool rot = ROPE && sizeof(TC) == 2 && s.rope_cs != nullptr && y0 + lane < s.M;
    const float4* cs_row = nullptr;
    float4 cs_cur[UC / 4], cs_nxt[UC / 4];
#pragma unroll
    for (int g = 0; g < UC / 4; ++g) cs_cur[g] = cs_nxt[g] = make_float4(1.0f, 0.0f, 1.0f, 0.0f);
    auto rope_fetch = [&](int u, float4 (&dst)[UC / 4]) {
        // float4 index of the unit's first pair inside the table row: pair j0 -> floats 2 j0
        const int f4 = static_cast<int>((n0 + static_cast<int64_t>(u) * UC) % (2 * s.rope_half)) / 4;
#pragma unroll
        for (int g = 0; g < UC / 4; ++g) dst[g] = __ldg(cs_row + f4 + g);
    };
    if (rot) {
        int64_t pp = s.rope_pos[y0 + lane];
        pp = pp < 0 ? 0 : (pp >= s.rope_npos ? s.rope_npos - 1 : pp);
        cs_row = reinterpret_cast<const float4*>(s.rope_cs + pp * s.rope_half * 2);
        if (n0 < s.rope_cols) rope_fetch(0, cs_cur);
    }
    bool ok = mbar_wait(acc_bar, acc_parity, abort_flag, ctl);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;
    fence_after();
    uint32_t r[2][UC];
    tmem_ld_cols<UC>(t_row, r[0]);
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        if (u < n_units && ok) {
            if (rot && u + 1 < n_units && n0 + (u + 1) * UC < s.rope_cols) rope_fetch(u + 1, cs_nxt);
            tmem_wait_ld();
            if (u + 1 < n_units) tmem_ld_cols<UC>(t_row + static_cast<uint32_t>((u + 1) * UC), r[(u + 1) & 1]);
            float v[UC];
#pragma unroll
            for (int e = 0; e < UC; ++e) v[e] = __uint_as_float(r[u & 1][e]);
            if (s.bias) {
#pragma unroll
                for (int g = 0; g < UC / 4; ++g) {
                    const int64_t c = n0 + u * UC + g * 4;
                    if (c < s.N) {
                        const float4 b = *reinterpret_cast<const float4*>(s.bias + c);
                        v[g * 4] += b.x; v[g * 4 + 1] += b.y; v[g * 4 + 2] += b.z; v[g * 4 + 3] += b.w;
                    }
                }
            }
            if (rot && n0 + u * UC < s.rope_cols) {
#pragma unroll
                for (int g = 0; g < UC / 4; ++g) {
                    const float4 c2 = cs_cur[g];   // (cos, sin) of two pairs
                    float a[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) a[e] = to_f32(from_f32<bf16>(v[g * 4 + e]));
                    rope_rotate(a[0], a[1], c2.x, c2.y * s.rope_sign, v[g * 4], v[g * 4 + 1]);
                    rope_rotate(a[2], a[3], c2.z, c2.w * s.rope_sign, v[g * 4 + 2], v[g * 4 + 3]);
                }
            }
#pragma unroll
            for (int g = 0; g < UC / 4; ++g) cs_cur[g] = cs_nxt[g];
            const uint32_t bx = s.uc & (BOXES - 1);
            uint8_t* box = s.boxes + bx * EPI_BOX_BYTES;
            if (reads) {
                ok = mbar_wait(smem_u32(&s.in_bar[bx]), (s.uc / BOXES) & 1u, abort_flag, ctl);
                ok = __all_sync(0xffffffffu, ok);
                if (ok) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) add_packed<TC>(v + j * (UC / 4), *reinterpret_cast<const uint4*>(box + box_offset(lane, j)));
                }
            } else {
                if (lane == 0) bulk_wait_read<BOXES - 1>();   // the store that last used this box has read it
                __syncwarp();
            }
            if (ok) {
#pragma unroll
                for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(box + box_offset(lane, j)) = pack_out<TC>(v + j * (UC / 4));
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (s.slab >= 0) tma_store_3d(s.out, smem_u32(box), static_cast<int32_t>(n0 + u * UC), y0, s.slab);
                    else tma_store_2d(s.out, smem_u32(box), static_cast<int32_t>(n0 + u * UC), y0);
                    bulk_commit();
                    if (reads && u + BOXES - 1 < n_units) {
                        bulk_wait_read<1>();   // the box of the unit before this one is free once its store has read it
                        const uint32_t nb = (s.uc + BOXES - 1) & (BOXES - 1);
                        const uint32_t bar = smem_u32(&s.in_bar[nb]);
                        mbar_expect_tx(bar, EPI_BOX_BYTES);
                        tma_load_2d(smem_u32(s.boxes + nb * EPI_BOX_BYTES), s.in, static_cast<int32_t>(n0 + (u + BOXES - 1) * UC), y0, bar);
                    }
                }
            }
            ++s.uc;
        }
    }
    return ok;
}

}  // namespace tc
}  // namespace pk
