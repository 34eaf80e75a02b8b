// Runtime entries of libpk: device selection, memory, copies, streams and the
// per-thread error message. See include/pk.h for the contract of each call.
#include <cstdarg>
#include <cstring>
#include <vector>

#include "pk_common.cuh"

namespace pk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cached;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
            cached = n;
            cached_dev = dev;
        }
    }
    return cached;
}

// ---- launch counters per kernel path ---------------------------------------------------
static int64_t g_path_counts[PATH_SLOTS] = {0};
void note_launch(int slot) {
    if (slot >= 0 && slot < PATH_SLOTS) ++g_path_counts[slot];
}

// ---- event-based profiling --------------------------------------------------------
namespace {
struct ProfRec {
    cudaEvent_t a, b;
    int kind;
    double work;
};
bool g_prof_on = false;
std::vector<ProfRec> g_prof;
size_t g_prof_used = 0;
}  // namespace

ProfScope::ProfScope(int kind, double work, cudaStream_t st_) : slot(-1), st(st_) {
    if (!g_prof_on) return;
    if (g_prof_used == g_prof.size()) {
        ProfRec r{};
        if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
        g_prof.push_back(r);
    }
    slot = static_cast<int>(g_prof_used++);
    g_prof[slot].kind = kind;
    g_prof[slot].work = work;
    cudaEventRecord(g_prof[slot].a, st);
}
ProfScope::~ProfScope() {
    if (slot >= 0) cudaEventRecord(g_prof[slot].b, st);
}

}  // namespace pk

extern "C" {

int pk_prof_enable(int on) {
    pk::g_prof_on = on != 0;
    return PK_OK;
}
int pk_prof_reset(void) {
    pk::g_prof_used = 0;
    return PK_OK;
}
int pk_prof_summary(int kind, double* ms_h, double* work_h, int64_t* launches_h) {
    PK_REQUIRE(kind >= 0 && kind < pk::PROF_KINDS && ms_h && work_h && launches_h, "bad argument");
    PK_CHECK_CUDA(cudaDeviceSynchronize());
    double ms = 0.0, work = 0.0;
    int64_t n = 0;
    for (size_t i = 0; i < pk::g_prof_used; ++i) {
        if (pk::g_prof[i].kind != kind) continue;
        float t = 0.0f;
        PK_CHECK_CUDA(cudaEventElapsedTime(&t, pk::g_prof[i].a, pk::g_prof[i].b));
        ms += t;
        work += pk::g_prof[i].work;
        ++n;
    }
    *ms_h = ms;
    *work_h = work;
    *launches_h = n;
    return PK_OK;
}

int pk_launch_counts(int64_t* counts_h, int n, int reset) {
    PK_REQUIRE(counts_h != nullptr && n >= 0, "bad argument");
    for (int i = 0; i < n; ++i) counts_h[i] = i < pk::PATH_SLOTS ? pk::g_path_counts[i] : 0;
    if (reset)
        for (int i = 0; i < pk::PATH_SLOTS; ++i) pk::g_path_counts[i] = 0;
    return PK_OK;
}

int pk_abi_version(void) { return PK_ABI_VERSION; }
const char* pk_last_error(void) { return pk::g_err; }

int pk_device_count(int* count_h) {
    PK_REQUIRE(count_h != nullptr, "null output");
    PK_CHECK_CUDA(cudaGetDeviceCount(count_h));
    return PK_OK;
}
int pk_set_device(int device) {
    PK_CHECK_CUDA(cudaSetDevice(device));
    return PK_OK;
}
int pk_device_name(int device, char* name_h, size_t cap) {
    PK_REQUIRE(name_h != nullptr && cap > 0, "null output");
    cudaDeviceProp p;
    PK_CHECK_CUDA(cudaGetDeviceProperties(&p, device));
    snprintf(name_h, cap, "%s sm_%d%d", p.name, p.major, p.minor);
    return PK_OK;
}
int pk_mem_info(size_t* free_h, size_t* total_h) {
    PK_REQUIRE(free_h && total_h, "null output");
    PK_CHECK_CUDA(cudaMemGetInfo(free_h, total_h));
    return PK_OK;
}
int pk_malloc(void** ptr_h, size_t bytes) {
    PK_REQUIRE(ptr_h != nullptr, "null output");
    *ptr_h = nullptr;
    if (bytes == 0) return PK_OK;
    PK_CHECK_CUDA(cudaMalloc(ptr_h, bytes));
    return PK_OK;
}
int pk_free(void* ptr) {
    if (ptr) PK_CHECK_CUDA(cudaFree(ptr));
    return PK_OK;
}
int pk_host_alloc(void** ptr_h, size_t bytes) {
    PK_REQUIRE(ptr_h != nullptr, "null output");
    PK_CHECK_CUDA(cudaMallocHost(ptr_h, bytes ? bytes : 1));
    return PK_OK;
}
int pk_host_free(void* ptr_h) {
    if (ptr_h) PK_CHECK_CUDA(cudaFreeHost(ptr_h));
    return PK_OK;
}
int pk_memcpy_h2d(void* dst, const void* src_h, size_t bytes, void* stream) {
    if (bytes == 0) return PK_OK;
    PK_CHECK_CUDA(cudaMemcpyAsync(dst, src_h, bytes, cudaMemcpyHostToDevice, pk::as_stream(stream)));
    return PK_OK;
}
int pk_memcpy_d2h(void* dst_h, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return PK_OK;
    PK_CHECK_CUDA(cudaMemcpyAsync(dst_h, src, bytes, cudaMemcpyDeviceToHost, pk::as_stream(stream)));
    return PK_OK;
}
int pk_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return PK_OK;
    PK_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, pk::as_stream(stream)));
    return PK_OK;
}
int pk_memset(void* dst, int value, size_t bytes, void* stream) {
    if (bytes == 0) return PK_OK;
    PK_CHECK_CUDA(cudaMemsetAsync(dst, value, bytes, pk::as_stream(stream)));
    return PK_OK;
}
int pk_stream_create(void** stream_h) {
    PK_REQUIRE(stream_h != nullptr, "null output");
    cudaStream_t s;
    PK_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream_h = s;
    return PK_OK;
}
int pk_stream_destroy(void* stream) {
    if (stream) PK_CHECK_CUDA(cudaStreamDestroy(pk::as_stream(stream)));
    return PK_OK;
}
int pk_stream_sync(void* stream) {
    PK_CHECK_CUDA(cudaStreamSynchronize(pk::as_stream(stream)));
    return PK_OK;
}
int pk_device_sync(void) {
    PK_CHECK_CUDA(cudaDeviceSynchronize());
    return PK_OK;
}

}  // extern "C"
