// Device residency layer: runtime switches, the caching allocator and Tensor.
// See microtorch/device.hpp for the contract. All GPU work goes through the C ABI
// of pk.h; nothing here includes a CUDA header.
#include "microtorch/device.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <unordered_map>
#include <vector>

#include "pk.h"

namespace microtorch {
namespace device {

namespace {

struct Runtime {
    Device dev = Device::CPU;
    bool inited = false;
    int ordinal = 0;
    void* own_stream = nullptr;
    void* ext_stream = nullptr;
    DType cdt = DType::F32;
    bool step_residency = true;
    bool device_ops = true;
    bool env_seen = false;  // the environment was consulted (explicitly or at first use)
};
Runtime& rt() {
    static Runtime r;
    return r;
}

// Size-bucketed caching allocator. Blocks are rounded up to 512 bytes (2 MiB above
// 1 MiB) and reused by exact rounded size; training steps repeat the same shapes,
// so after the first step no driver allocation happens. All work is ordered on one
// stream, which makes reuse immediately after release safe.
struct Allocator {
    std::mutex mu;
    std::unordered_map<size_t, std::vector<void*>> free_blocks;
    MemStats stats;
    // activation blocks in use by rounded size, and a copy taken whenever the activation
    // high-water mark rises: what was live at the peak, by size
    std::map<size_t, size_t> live_by_size, peak_by_size;

    static size_t round(size_t n) {
        if (n == 0) n = 1;
        const size_t q = n >= (size_t(1) << 20) ? (size_t(2) << 20) : 512;
        return (n + q - 1) / q * q;
    }
    void* get(size_t rounded, Pool pool) {
        std::lock_guard<std::mutex> lk(mu);
        void* p = nullptr;
        auto it = free_blocks.find(rounded);
        if (it != free_blocks.end() && !it->second.empty()) {
            p = it->second.back();
            it->second.pop_back();
        } else {
            int rc = pk_malloc(&p, rounded);
            if (rc != PK_OK) {
                release_cached_locked();
                rc = pk_malloc(&p, rounded);
            }
            if (rc != PK_OK)
                throw std::runtime_error(std::string("device allocation of ") + std::to_string(rounded) +
                                         " bytes failed: " + pk_last_error());
            stats.reserved += rounded;
            ++stats.driver_allocs;
        }
        const int k = static_cast<int>(pool);
        stats.in_use[k] += rounded;
        if (pool == Pool::Activation) {
            ++live_by_size[rounded];
            if (stats.in_use[k] > stats.peak[k]) peak_by_size = live_by_size;
        }
        stats.peak[k] = std::max(stats.peak[k], stats.in_use[k]);
        return p;
    }
    void put(void* p, size_t rounded, Pool pool) {
        std::lock_guard<std::mutex> lk(mu);
        stats.in_use[static_cast<int>(pool)] -= rounded;
        if (pool == Pool::Activation) {
            auto it = live_by_size.find(rounded);
            if (it != live_by_size.end() && --it->second == 0) live_by_size.erase(it);
        }
        free_blocks[rounded].push_back(p);
    }
    void release_cached_locked() {
        pk_device_sync();
        for (auto& [sz, v] : free_blocks) {
            for (void* p : v) {
                pk_free(p);
                stats.reserved -= sz;
            }
            v.clear();
        }
    }
};
Allocator& alloc() {
    static Allocator* a = new Allocator();  // never destroyed: Storages may outlive static teardown
    return *a;
}

}  // namespace

void check(int rc, const char* what) {
    if (rc != PK_OK)
        throw std::runtime_error(std::string(what) + " failed (status " + std::to_string(rc) + "): " + pk_last_error());
}

Device get() { return rt().dev; }
bool cuda_compiled() { return true; }
bool initialized() { return rt().inited; }

void init(int ordinal) {
    Runtime& r = rt();
    if (r.inited && r.ordinal == ordinal) return;
    // One GPU per process (the data-parallel layout is one process per GPU): the kernels cache
    // per-device set-up -- shared-memory opt-ins, occupancy figures, the split-K workspace -- once.
    if (r.inited)
        throw std::runtime_error("microtorch: GPU " + std::to_string(r.ordinal) + " is already selected; a process uses one "
                                 "GPU (start one process per GPU)");
    int n = 0;
    check(pk_device_count(&n), "pk_device_count");
    if (n <= 0) throw std::runtime_error("no CUDA device is visible; this library has no CPU execution path");
    if (ordinal < 0 || ordinal >= n) throw std::runtime_error("GPU ordinal out of range");
    check(pk_set_device(ordinal), "pk_set_device");
    if (!r.own_stream) check(pk_stream_create(&r.own_stream), "pk_stream_create");
    {
        // Workspace for the split-K partial tiles of weight-gradient GEMMs with few output tiles
        // (one per process: every GEMM of this library runs on the one compute stream).
        static void* gemm_ws = nullptr;
        constexpr size_t kGemmWsBytes = size_t(128) << 20;
        if (gemm_ws) pk_free(gemm_ws);
        gemm_ws = nullptr;
        check(pk_malloc(&gemm_ws, kGemmWsBytes), "pk_malloc");
        check(pk_gemm_set_workspace(gemm_ws, kGemmWsBytes), "pk_gemm_set_workspace");
    }
    r.ordinal = ordinal;
    r.inited = true;
    r.dev = Device::CUDA;
}

void set(Device d) {
    if (d == Device::CUDA) {
        init(rt().ordinal);
    } else {
        rt().dev = Device::CPU;
    }
}

void set_from_env() {
    rt().env_seen = true;
    if (const char* g = std::getenv("MICROTORCH_GPU")) rt().ordinal = std::atoi(g);
    if (const char* t = std::getenv("MICROTORCH_DTYPE")) {
        const std::string s(t);
        if (s == "bf16") rt().cdt = DType::BF16;
        else if (s == "fp32" || s == "f32") rt().cdt = DType::F32;
        else throw std::runtime_error("MICROTORCH_DTYPE must be fp32 or bf16");
    }
    if (const char* d = std::getenv("MICROTORCH_DEVICE")) {
        const std::string s(d);
        if (s == "cuda") set(Device::CUDA);
        else if (s == "cpu") set(Device::CPU);
        else throw std::runtime_error("MICROTORCH_DEVICE must be cuda or cpu");
    }
}

void set_stream(void* s) { rt().ext_stream = s; }
void* stream() {
    Runtime& r = rt();
    if (r.dev != Device::CUDA && !r.inited && !r.env_seen) {
        // A program written for the reference may never touch the device switch (its CPU path
        // needs none). The first op then honours MICROTORCH_DEVICE / _DTYPE / _GPU once, so
        // such a program runs on the GPU by setting the environment alone.
        r.env_seen = true;
        set_from_env();
    }
    if (r.dev != Device::CUDA)
        throw std::runtime_error("microtorch: the CUDA device is not selected and there is no CPU fallback "
                                 "(call device::init() or set MICROTORCH_DEVICE=cuda)");
    return r.ext_stream ? r.ext_stream : r.own_stream;
}
void synchronize() { check(pk_stream_sync(stream()), "pk_stream_sync"); }

void set_compute_dtype(DType t) { rt().cdt = t; }
DType compute_dtype() { return rt().cdt; }

void step_begin() {}
void step_end() {}
void set_step_residency(bool on) { rt().step_residency = on; }
bool step_residency_enabled() { return rt().step_residency; }
void set_device_ops(bool on) { rt().device_ops = on; }
bool device_ops_enabled() { return rt().device_ops; }

MemStats mem_stats() {
    std::lock_guard<std::mutex> lk(alloc().mu);
    return alloc().stats;
}
void reset_peak() {
    std::lock_guard<std::mutex> lk(alloc().mu);
    for (int k = 0; k < 2; ++k) alloc().stats.peak[k] = alloc().stats.in_use[k];
    alloc().peak_by_size = alloc().live_by_size;
}
std::vector<std::pair<size_t, size_t>> peak_activation_blocks() {
    std::lock_guard<std::mutex> lk(alloc().mu);
    return std::vector<std::pair<size_t, size_t>>(alloc().peak_by_size.begin(), alloc().peak_by_size.end());
}
void empty_cache() {
    std::lock_guard<std::mutex> lk(alloc().mu);
    alloc().release_cached_locked();
}

}  // namespace device

Storage::~Storage() {
    if (owned && ptr) device::alloc().put(ptr, bytes, pool);
}

Tensor Tensor::empty(size_t rows, size_t cols, DType dt, device::Pool pool) {
    (void)device::stream();  // throws when the device is not selected
    Tensor t;
    t.rows_ = rows;
    t.cols_ = cols;
    t.dt_ = dt;
    auto st = std::make_shared<Storage>();
    st->bytes = device::Allocator::round(rows * cols * dtype_bytes(dt));
    st->pool = pool;
    st->ptr = device::alloc().get(st->bytes, pool);
    t.st_ = std::move(st);
    return t;
}

Tensor Tensor::empty_strided(size_t rows, size_t cols, size_t ld, DType dt, device::Pool pool) {
    if (ld < cols) throw std::runtime_error("Tensor::empty_strided: ld < cols");
    Tensor t = empty(rows, ld, dt, pool);
    t.cols_ = cols;
    t.ld_ = ld == cols ? 0 : ld;
    return t;
}

Tensor Tensor::dense() const {
    if (is_dense()) return *this;
    Tensor t = empty(rows_, cols_, dt_);
    device::check(pk_copy_cols(device::stream(), dt(), ptr(), static_cast<int64_t>(ld()), 0, t.ptr(),
                               static_cast<int64_t>(cols_), 0, static_cast<int64_t>(rows_),
                               static_cast<int64_t>(cols_), 0), "pk_copy_cols");
    return t;
}

Tensor Tensor::zeros(size_t rows, size_t cols, DType dt, device::Pool pool) {
    Tensor t = empty(rows, cols, dt, pool);
    t.zero_();
    return t;
}

Tensor Tensor::bytes(size_t nbytes, device::Pool pool) { return empty(1, (nbytes + 3) / 4, DType::F32, pool); }

Tensor Tensor::from_host(const Matrix& m, DType dt, device::Pool pool) {
    Tensor t = empty(m.rows(), m.cols(), dt, pool);
    t.copy_from_host(m);
    return t;
}

Tensor Tensor::view(size_t elem_offset, size_t rows, size_t cols) const {
    if (!st_) throw std::runtime_error("Tensor::view on an undefined tensor");
    if (!is_dense()) throw std::runtime_error("Tensor::view on a strided tensor");
    const size_t end = off_ + (elem_offset + rows * cols) * dtype_bytes(dt_);
    if (end > st_->bytes) throw std::runtime_error("Tensor::view exceeds the storage");
    Tensor t = *this;
    t.off_ = off_ + elem_offset * dtype_bytes(dt_);
    t.rows_ = rows;
    t.cols_ = cols;
    return t;
}

Tensor Tensor::reshape(size_t rows, size_t cols) const {
    if (!is_dense()) throw std::runtime_error("Tensor::reshape on a strided tensor");
    if (rows * cols != numel()) throw std::runtime_error("Tensor::reshape changes the element count");
    Tensor t = *this;
    t.rows_ = rows;
    t.cols_ = cols;
    return t;
}

Tensor Tensor::clone() const {  // keeps the row stride
    Tensor t = empty_strided(rows_, cols_, ld(), dt_);
    device::check(pk_memcpy_d2d(t.ptr(), ptr(), nbytes(), device::stream()), "pk_memcpy_d2d");
    return t;
}

Tensor Tensor::cast(DType dt) const {
    if (dt == dt_) return *this;
    if (!is_dense()) return dense().cast(dt);
    Tensor t = empty(rows_, cols_, dt);
    device::check(pk_cast(device::stream(), this->dt(), ptr(), t.dt(), t.ptr(), static_cast<int64_t>(numel())), "pk_cast");
    return t;
}

void Tensor::zero_() {
    if (numel()) device::check(pk_memset(ptr(), 0, nbytes(), device::stream()), "pk_memset");
}

void Tensor::copy_from_host(const Matrix& m) {
    if (m.rows() != rows_ || m.cols() != cols_) throw std::runtime_error("Tensor::copy_from_host: shape mismatch");
    if (!is_dense()) throw std::runtime_error("Tensor::copy_from_host on a strided tensor");
    if (numel() == 0) return;
    void* s = device::stream();
    if (dt_ == DType::F32) {
        device::check(pk_memcpy_h2d(ptr(), m.data(), nbytes(), s), "pk_memcpy_h2d");
        device::check(pk_stream_sync(s), "pk_stream_sync");  // m is pageable and may die after return
    } else {
        Tensor tmp = empty(rows_, cols_, DType::F32);
        device::check(pk_memcpy_h2d(tmp.ptr(), m.data(), tmp.nbytes(), s), "pk_memcpy_h2d");
        device::check(pk_cast(s, PK_F32, tmp.ptr(), PK_BF16, ptr(), static_cast<int64_t>(numel())), "pk_cast");
        device::check(pk_stream_sync(s), "pk_stream_sync");
    }
}

Matrix Tensor::to_host() const {
    if (!is_dense()) return dense().to_host();
    Matrix m(rows_, cols_);
    if (numel() == 0) return m;
    void* s = device::stream();
    if (dt_ == DType::F32) {
        device::check(pk_memcpy_d2h(m.data(), ptr(), nbytes(), s), "pk_memcpy_d2h");
    } else {
        Tensor tmp = cast(DType::F32);
        device::check(pk_memcpy_d2h(m.data(), tmp.ptr(), tmp.nbytes(), s), "pk_memcpy_d2h");
        device::check(pk_stream_sync(s), "pk_stream_sync");
        return m;
    }
    device::check(pk_stream_sync(s), "pk_stream_sync");
    return m;
}

}  // namespace microtorch
