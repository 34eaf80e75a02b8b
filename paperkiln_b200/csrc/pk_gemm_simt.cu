// SIMT GEMM (fp32 FMA, fp32 accumulation) for fp32 operands -- the precision the
// reference's CPU path computes in -- and for bf16 operands whose shapes the
// tensor-core kernel does not take. Also hosts the pk_gemm dispatcher.
//
// C[M,N] (+)= op(A).op(B) (+ bias) (+ residual); any M, N, K >= 0, any leading
// dimensions; transposes are index arithmetic (never materialised), as in the
// reference's gemm_tiled_ops (src/cuda_resident.cu:141-171). The k loop runs in
// ascending order inside one thread, so results are reproducible.
#include "pk_common.cuh"

namespace pk {

int gemm_tc_supported(int c_dtype, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A,
                      int64_t lda, const void* B, int64_t ldb, const void* C, int64_t ldc,
                      const void* residual, int64_t ldr, const float* bias);
int gemm_tc_launch(cudaStream_t st, int c_dtype, int ta, int tb, int64_t M, int64_t N, int64_t K,
                   const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
                   int accumulate, const float* bias, const void* residual, int64_t ldr);

float* gemm_splitk_workspace(size_t* bytes);   // pk_gemm_tc.cu

// CTA-pair kernel (pk_gemm_tc2.cu)
int gemm_tc2_launch(cudaStream_t st, int c_dtype, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                    const void* B, int64_t ldb, void* C, int64_t ldc, int accumulate, const float* bias, const void* residual,
                    int64_t ldr, const RopeEpilogue* rope);

static thread_local int g_last_path = -1;
static int g_force_simt = 0;
int gemm_tc2_swiglu_launch(cudaStream_t st, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* Wg,
                           int64_t ldg, const void* Wu, int64_t ldu, void* G, void* U, int64_t ldgu, void* Y, int64_t ldy);
static int g_pair_mode = 1;  // 1: 256 x 256 tiles on CTA pairs where the shape has enough of them

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TAB, typename TC, bool TRA, bool TRB>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TAB* __restrict__ A, int64_t lda, const TAB* __restrict__ B, int64_t ldb,
                 TC* __restrict__ C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                 const float* __restrict__ bias, const TC* __restrict__ residual, int64_t ldr) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int t = threadIdx.x;
    const int tx = t & 15, ty = t >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < K; k0 += BK) {
        // ---- stage A tile [BM x BK] as As[k][m]
        if (!TRA) {
            const int kk = t & 15;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int i = (t >> 4) + it * 16;
                const int64_t m = m0 + i, k = k0 + kk;
                As[kk][i] = (m < M && k < K) ? to_f32(A[m * lda + k]) : 0.0f;
            }
        } else {
            const int i = t & 63;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int kk = (t >> 6) + it * 4;
                const int64_t m = m0 + i, k = k0 + kk;
                As[kk][i] = (m < M && k < K) ? to_f32(A[k * lda + m]) : 0.0f;
            }
        }
        // ---- stage B tile [BK x BN] as Bs[k][n]
        if (!TRB) {
            const int j = t & 63;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int kk = (t >> 6) + it * 4;
                const int64_t n = n0 + j, k = k0 + kk;
                Bs[kk][j] = (n < N && k < K) ? to_f32(B[k * ldb + n]) : 0.0f;
            }
        } else {
            const int kk = t & 15;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int j = (t >> 4) + it * 16;
                const int64_t n = n0 + j, k = k0 + kk;
                Bs[kk][j] = (n < N && k < K) ? to_f32(B[n * ldb + k]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (residual) v += to_f32(residual[m * ldr + n]);
            if (accumulate) v += to_f32(C[m * ldc + n]);
            C[m * ldc + n] = from_f32<TC>(v);
        }
    }
}

template <typename TAB, typename TC>
int launch_simt(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A,
                int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, int accumulate,
                const float* bias, const void* residual, int64_t ldr) {
    dim3 grid(static_cast<unsigned>((N + BN - 1) / BN), static_cast<unsigned>((M + BM - 1) / BM));
    if (grid.y > 65535u) {
        set_error("pk_gemm: M too large for the SIMT kernel grid");
        return PK_ERR_UNSUPPORTED;
    }
    const TAB* a = static_cast<const TAB*>(A);
    const TAB* b = static_cast<const TAB*>(B);
    TC* c = static_cast<TC*>(C);
    const TC* r = static_cast<const TC*>(residual);
#define PK_SIMT(TRA_, TRB_) \
    gemm_simt_kernel<TAB, TC, TRA_, TRB_><<<grid, 256, 0, st>>>(a, lda, b, ldb, c, ldc, M, N, K, accumulate, bias, r, ldr)
    if (!ta && !tb) PK_SIMT(false, false);
    else if (!ta && tb) PK_SIMT(false, true);
    else if (ta && !tb) PK_SIMT(true, false);
    else PK_SIMT(true, true);
#undef PK_SIMT
    PK_LAUNCH_CHECK();
    return PK_OK;
}

void gemm_note_path(int path) { g_last_path = path; }  // for the kernels with an entry point of their own

}  // namespace pk

using namespace pk;

extern "C" {

int pk_gemm(void* stream, int ab_dtype, int c_dtype, int trans_a, int trans_b, int64_t M, int64_t N,
            int64_t K, const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
            int accumulate, const float* bias, const void* residual, int64_t ldr) {
    PK_REQUIRE(valid_dtype(ab_dtype) && valid_dtype(c_dtype), "bad dtype");
    PK_REQUIRE(M >= 0 && N >= 0 && K >= 0, "negative shape");
    if (M == 0 || N == 0) return PK_OK;
    PK_REQUIRE(C != nullptr, "null C");
    PK_REQUIRE(K == 0 || (A && B), "null operand");
    PK_REQUIRE(lda >= (trans_a ? M : K) && ldb >= (trans_b ? K : N) && ldc >= N, "leading dimension too small");
    PK_REQUIRE(residual == nullptr || ldr >= N, "residual leading dimension too small");
    PK_REQUIRE(!(ab_dtype == PK_F32 && c_dtype == PK_BF16), "fp32 operands with bf16 output are not provided");
    cudaStream_t st = as_stream(stream);
    if (ab_dtype == PK_BF16 && !g_force_simt &&
        gemm_tc_supported(c_dtype, trans_a, trans_b, M, N, K, A, lda, B, ldb, C, ldc, residual, ldr, bias)) {
        ProfScope prof(PROF_GEMM_TC, 2.0 * M * N * K, st);
        if (g_pair_mode) {
            // worth it only when the 256 x 256 tiles keep the SM pairs busy (same fill rule as the tile width)
            const int64_t pairs = sm_count() / 2;
            const int64_t t2 = ((M + 255) / 256) * ((N + 255) / 256);
            const double fill = static_cast<double>(t2) / static_cast<double>((t2 + pairs - 1) / pairs * pairs);
            // ... or when cutting a long k loop into 2-4 parts does (the pair kernel's own split-K rule;
            // input gradient of a wide vocabulary projection: 48 tiles, k = 151 936)
            bool split_fills = false;
            size_t ws_bytes = 0;
            if (fill < 0.8 && K >= 256 * 64 && gemm_splitk_workspace(&ws_bytes) != nullptr) {
                const size_t part_bytes = static_cast<size_t>(M) * static_cast<size_t>((N + 255) / 256 * 256) * sizeof(float);
                for (int sp = 2; sp <= 4 && !split_fills; ++sp) {
                    const int64_t items = t2 * sp;
                    const double f = static_cast<double>(items) / static_cast<double>((items + pairs - 1) / pairs * pairs);
                    split_fills = f >= 0.95 && sp * part_bytes <= ws_bytes;
                }
            }
            if (N >= 256 && M >= 256 && (fill >= 0.8 || split_fills)) {
                g_last_path = 3;
                note_launch(PATH_GEMM_TC_PAIR);
                return gemm_tc2_launch(st, c_dtype, trans_a, trans_b, M, N, K, A, lda, B, ldb, C, ldc, accumulate, bias,
                                       residual, ldr, nullptr);
            }
        }
        g_last_path = 2;
        note_launch(PATH_GEMM_TC);
        return gemm_tc_launch(st, c_dtype, trans_a, trans_b, M, N, K, A, lda, B, ldb, C, ldc, accumulate,
                              bias, residual, ldr);
    }
    ProfScope prof(PROF_GEMM_SIMT, 2.0 * M * N * K, st);
    if (ab_dtype == PK_F32) {
        g_last_path = 0;
        note_launch(PATH_GEMM_SIMT_F32);
        return launch_simt<float, float>(st, trans_a, trans_b, M, N, K, A, lda, B, ldb, C, ldc, accumulate,
                                         bias, residual, ldr);
    }
    g_last_path = 1;
    note_launch(PATH_GEMM_SIMT_BF16);
    if (c_dtype == PK_F32)
        return launch_simt<bf16, float>(st, trans_a, trans_b, M, N, K, A, lda, B, ldb, C, ldc, accumulate,
                                        bias, residual, ldr);
    return launch_simt<bf16, bf16>(st, trans_a, trans_b, M, N, K, A, lda, B, ldb, C, ldc, accumulate, bias,
                                   residual, ldr);
}

int pk_gemm_swiglu(void* stream, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* Wg, int64_t ldg,
                   const void* Wu, int64_t ldu, void* G, void* U, int64_t ldgu, void* Y, int64_t ldy) {
    PK_REQUIRE(M >= 0 && N >= 0 && K > 0, "bad shape");
    if (M == 0 || N == 0) return PK_OK;
    PK_REQUIRE(A && Wg && Wu && Y, "null pointer");
    PK_REQUIRE((G == nullptr) == (U == nullptr), "G and U are stored together or not at all");
    PK_REQUIRE(lda >= K && ldg >= N && ldu >= N && ldy >= N && (G == nullptr || ldgu >= N), "leading dimension too small");
    const bool ok = !g_force_simt && N % 8 == 0 && M >= 256 && N >= 128 && lda % 8 == 0 && ldg % 8 == 0 && ldu % 8 == 0 &&
                    ldy % 8 == 0 && (G == nullptr || ldgu % 8 == 0) && aligned16(A) && aligned16(Wg) && aligned16(Wu) &&
                    aligned16(Y) && (G == nullptr || (aligned16(G) && aligned16(U))) && M < (int64_t(1) << 31) &&
                    N < (int64_t(1) << 31) && K < (int64_t(1) << 31);
    if (!ok) {
        set_error("pk_gemm_swiglu: shape or alignment outside what the kernel takes (M %lld N %lld K %lld)",
                  static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K));
        return PK_ERR_UNSUPPORTED;
    }
    cudaStream_t st = as_stream(stream);
    ProfScope prof(PROF_GEMM_TC, 4.0 * M * N * K, st);
    g_last_path = 3;
    note_launch(PATH_GEMM_TC_PAIR);
    return gemm_tc2_swiglu_launch(st, M, N, K, A, lda, Wg, ldg, Wu, ldu, G, U, ldgu, Y, ldy);
}

int pk_gemm_rope(void* stream, int trans_b, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B,
                 int64_t ldb, void* C, int64_t ldc, const float* bias, const int32_t* pos, const float* cos_sin, int64_t n_pos,
                 int n_heads, int head_dim, int inverse) {
    PK_REQUIRE(M >= 0 && N >= 0 && K > 0 && n_heads >= 0 && n_pos > 0, "bad shape");
    if (M == 0 || N == 0) return PK_OK;
    PK_REQUIRE(A && B && C && pos && cos_sin, "null pointer");
    PK_REQUIRE(lda >= K && ldb >= (trans_b ? K : N) && ldc >= N, "leading dimension too small");
    PK_REQUIRE(static_cast<int64_t>(n_heads) * head_dim <= N, "more rotated columns than C has");
    // the pair kernel's staged epilogue, a 32-column unit inside one head, the same fill rule as pk_gemm
    const int64_t pairs = sm_count() / 2;
    const int64_t t2 = ((M + 255) / 256) * ((N + 255) / 256);
    const double fill = static_cast<double>(t2) / static_cast<double>((t2 + pairs - 1) / pairs * pairs);
    const bool ok = !g_force_simt && g_pair_mode && (head_dim == 64 || head_dim == 128) && M >= 256 && N >= 256 && fill >= 0.8 &&
                    N % 8 == 0 && aligned16(cos_sin) && (bias == nullptr || aligned16(bias)) &&
                    gemm_tc_supported(PK_BF16, 0, trans_b, M, N, K, A, lda, B, ldb, C, ldc, nullptr, 0, bias);
    if (!ok) {
        set_error("pk_gemm_rope: shape or alignment outside what the kernel takes (M %lld N %lld K %lld head_dim %d)",
                  static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K), head_dim);
        return PK_ERR_UNSUPPORTED;
    }
    RopeEpilogue rope;
    rope.cos_sin = cos_sin;
    rope.pos = pos;
    rope.n_pos = n_pos;
    rope.half = head_dim / 2;
    rope.cols = static_cast<int64_t>(n_heads) * head_dim;
    rope.sign = inverse ? -1.0f : 1.0f;
    cudaStream_t st = as_stream(stream);
    ProfScope prof(PROF_GEMM_TC, 2.0 * M * N * K, st);
    g_last_path = 3;
    note_launch(PATH_GEMM_TC_PAIR);
    return gemm_tc2_launch(st, PK_BF16, 0, trans_b, M, N, K, A, lda, B, ldb, C, ldc, 0, bias, nullptr, 0, &rope);
}

int pk_gemm_last_path(void) { return g_last_path; }
int pk_gemm_force_simt(int on) {
    g_force_simt = on ? 1 : 0;
    return PK_OK;
}
int pk_gemm_pair_mode(int on) {
    g_pair_mode = on ? 1 : 0;
    return PK_OK;
}

}  // extern "C"
