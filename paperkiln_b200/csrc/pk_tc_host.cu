// Host-side pieces shared by the tensor-core kernels: tensor-map construction, the
// collected status words of the attention kernels, the settable limit of the bounded
// device-side waits, and a self-test of such a wait.
#include <cuda.h>

#include <mutex>

#include "pk_common.cuh"
#include "pk_tc.cuh"

namespace pk {

int gemm_tc_set_wait_limit(long long cycles);       // pk_gemm_tc.cu
int gemm_tc2_set_wait_limit(long long cycles);      // pk_gemm_tc2.cu
int gemm_q8_set_wait_limit(long long cycles);       // pk_gemm_q8.cu
int attn_fwd_row_set_wait_limit(long long cycles);  // pk_attn_fwd_row.cu
int attn_bwd_ws_set_wait_limit(long long cycles);   // pk_attn_bwd_ws.cu
int attn_fwd_row_status(int* status_h, int clear);
int attn_bwd_ws_status(int* status_h, int clear);
int gemm_tc_status(int* status_h, int clear);
int gemm_tc2_status(int* status_h, int clear);
int gemm_q8_status(int* status_h, int clear);

PK_DEFINE_WAITCTL(wait_selftest)

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

static int encode(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
                  const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return PK_ERR_CUDA;
    }
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (rank %d, dims %llu x %llu, box %u x %u)", static_cast<int>(r),
                  rank, static_cast<unsigned long long>(dims[0]), static_cast<unsigned long long>(dims[1]), box[0], box[1]);
        return PK_ERR_CUDA;
    }
    return PK_OK;
}

int make_tensor_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_inner,
                    int box_outer) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

int make_tensor_map_3d(CUtensorMap* map, const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t ld,
                       int box_inner, int box_rows) {
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(ld) * 2 * static_cast<cuuint64_t>(rows)};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows), 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

int make_tensor_map_out(CUtensorMap* map, const void* base, int elem_bytes, int64_t inner, int64_t outer, int64_t ld,
                        int box_outer) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * static_cast<cuuint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(64 / elem_bytes), static_cast<cuuint32_t>(box_outer)};
    return encode(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims,
                  strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

int make_tensor_map_out_3d(CUtensorMap* map, const void* base, int elem_bytes, int64_t inner, int64_t rows, int64_t slabs,
                           int64_t ld, int64_t slab_elems, int box_outer) {
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(slabs)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * static_cast<cuuint64_t>(elem_bytes),
                                   static_cast<cuuint64_t>(slab_elems) * static_cast<cuuint64_t>(elem_bytes)};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(64 / elem_bytes), static_cast<cuuint32_t>(box_outer), 1};
    return encode(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims,
                  strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

int make_tensor_map_u8(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_inner,
                       int box_outer) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace tc

// Shapes and pointers the tcgen05 attention kernels take (used by the dispatcher in pk_attn_simt.cu).
int attn_tc_supported(int dtype, int dk, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                      int64_t ldv, const void* out, int64_t ldo, int64_t B, int64_t S) {
    if (dtype != PK_BF16 || (dk != 64 && dk != 128)) return 0;
    if (ldq % 8 || ldk % 8 || ldv % 8 || ldo % 8) return 0;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return 0;
    if (B * S >= (int64_t(1) << 31) || S >= (int64_t(1) << 30)) return 0;
    return 1;
}

namespace {
// One warp waits, with the family's bounded wait, on an mbarrier that nobody ever arrives at.
// The wait runs into its limit, records PK_ERR_TIMEOUT in the control block and returns: the
// path every tensor-core kernel takes when a producer never shows up, exercised on its own.
__global__ void wait_selftest_kernel(long long* waited_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tc::mbar_init(tc::smem_u32(&bar), 1);
        abort_flag = 0;
        tc::mbar_fence_init();
    }
    __syncwarp();
    const long long t0 = clock64();
    const bool ok = tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_flag, &g_wait_selftest_ctl);
    if (threadIdx.x == 0) waited_cycles[0] = ok ? -1 : clock64() - t0;
}
}  // namespace

}  // namespace pk

extern "C" {

int pk_attn_tc_status(int* status_h, int clear) {
    PK_REQUIRE(status_h != nullptr, "null output");
    PK_CHECK_CUDA(cudaDeviceSynchronize());
    int fwd = 0, bwd = 0;
    int rc = pk::attn_fwd_row_status(&fwd, clear);
    if (rc == PK_OK) rc = pk::attn_bwd_ws_status(&bwd, clear);
    if (rc != PK_OK) return rc;
    *status_h = fwd | bwd;
    return PK_OK;
}

int pk_kernel_status(int* status_h, int clear) {
    PK_REQUIRE(status_h != nullptr, "null output");
    int (*const readers[])(int*, int) = {pk::gemm_tc_status, pk::gemm_tc2_status, pk::gemm_q8_status,
                                         pk::attn_fwd_row_status, pk::attn_bwd_ws_status};
    int all = 0;
    for (auto rd : readers) {
        int one = 0;
        const int rc = rd(&one, clear);
        if (rc != PK_OK) return rc;
        all |= one;
    }
    *status_h = all;
    return PK_OK;
}

int pk_set_wait_limit_us(double microseconds) {
    PK_REQUIRE(microseconds > 0.0 && microseconds <= 60e6, "limit must be in (0, 60 s]");
    int dev = 0, khz = 0;
    PK_CHECK_CUDA(cudaGetDevice(&dev));
    PK_CHECK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    // cycles at the highest SM clock: at a lower clock the wait lasts longer, never shorter
    long long cycles = static_cast<long long>(microseconds * 1e-3 * static_cast<double>(khz));
    if (cycles < 1024) cycles = 1024;
    int rc = pk::gemm_tc_set_wait_limit(cycles);
    if (rc == PK_OK) rc = pk::gemm_tc2_set_wait_limit(cycles);
    if (rc == PK_OK) rc = pk::gemm_q8_set_wait_limit(cycles);
    if (rc == PK_OK) rc = pk::attn_fwd_row_set_wait_limit(cycles);
    if (rc == PK_OK) rc = pk::attn_bwd_ws_set_wait_limit(cycles);
    if (rc == PK_OK) rc = pk::wait_selftest_set_wait_limit(cycles);
    return rc;
}

int pk_wait_selftest(void* stream, int* status_h, double* waited_us_h) {
    PK_REQUIRE(status_h != nullptr && waited_us_h != nullptr, "null output");
    cudaStream_t st = pk::as_stream(stream);
    long long* d = nullptr;
    PK_CHECK_CUDA(cudaMalloc(&d, sizeof(long long)));
    pk::wait_selftest_kernel<<<1, 32, 0, st>>>(d);
    cudaError_t e = cudaGetLastError();
    long long cycles = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&cycles, d, sizeof(long long), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d);
    if (e != cudaSuccess) {
        pk::set_error("pk_wait_selftest: %s", cudaGetErrorString(e));
        return PK_ERR_CUDA;
    }
    int dev = 0, khz = 0;
    PK_CHECK_CUDA(cudaGetDevice(&dev));
    PK_CHECK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    *waited_us_h = cycles < 0 ? -1.0 : static_cast<double>(cycles) * 1e3 / static_cast<double>(khz);
    return pk::wait_selftest_status(status_h, 1);
}

}  // extern "C"
