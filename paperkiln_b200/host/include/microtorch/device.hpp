#pragma once
// Device residency layer.
//
// The reference keeps every tensor in host memory and round-trips each op
// through the GPU (include/microtorch/device.hpp:20-33 and the DevState /
// step window machinery of include/microtorch/device_cache.hpp:44-71). Here the
// roles are inverted: a tensor's home is device memory, the host copy is a
// lazily refreshed view, and every op of the tape calls a libpk kernel through
// the C ABI of pk.h. There is no CPU execution path: selecting the CUDA device
// without a usable GPU throws.
//
// Pieces
//   DType / Tensor   a 2-D row-major device array (fp32 or bf16) with shared
//                    ownership of its storage; views share storage
//   allocator        size-bucketed caching allocator over pk_malloc with
//                    separate accounting for activations and persistent state
//                    (the "peak activation bytes" metric comes from here)
//   runtime          stream, compute dtype (fp32 parity mode / bf16 mode), the
//                    reference's set/get/set_from_env switches
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "microtorch/matrix.hpp"

namespace microtorch {

enum class DType : int { F32 = 0, BF16 = 1 };
inline size_t dtype_bytes(DType t) { return t == DType::BF16 ? 2 : 4; }

namespace device {

enum class Device { CPU, CUDA };
// Device::CUDA is the only device that executes ops. get() reports CUDA once
// init() succeeded. set(Device::CPU) is accepted for source compatibility but
// any op executed afterwards throws: there is no CPU fallback.
Device get();
void set(Device d);
bool cuda_compiled();
// Honors MICROTORCH_DEVICE (cuda|cpu), MICROTORCH_DTYPE (fp32|bf16),
// MICROTORCH_GPU (ordinal). Reference: src/device.cpp:48-67.
void set_from_env();

// Selects the GPU, creates the compute stream. Idempotent for the same ordinal; a process uses
// one GPU, so another ordinal after the first throws (data parallelism is one process per GPU).
void init(int ordinal = 0);
bool initialized();
// Use an externally owned stream (e.g. the current stream of a framework the
// process shares the GPU with). Pass nullptr to return to the library's own.
void set_stream(void* cuda_stream);
void* stream();
void synchronize();

void set_compute_dtype(DType t);
DType compute_dtype();

// The reference's step window (device_cache.hpp:48-50) scoped which device
// copies could be trusted. Device memory is authoritative here, so these only
// mark step boundaries for the allocator statistics.
void step_begin();
void step_end();
void set_step_residency(bool on);
bool step_residency_enabled();
void set_device_ops(bool on);
bool device_ops_enabled();

enum class Pool : int { Activation = 0, Persistent = 1 };
struct MemStats {
    size_t in_use[2] = {0, 0};
    size_t peak[2] = {0, 0};
    size_t reserved = 0;     // bytes held from the driver (in use + cached)
    size_t driver_allocs = 0;  // number of pk_malloc calls so far
};
MemStats mem_stats();
void reset_peak();
void empty_cache();
// The activation blocks that were in use when the activation high-water mark was last raised
// (since reset_peak): (block size in bytes, number of blocks), ascending by size.
std::vector<std::pair<size_t, size_t>> peak_activation_blocks();

// Throws std::runtime_error carrying pk_last_error() when rc != 0.
void check(int rc, const char* what);

}  // namespace device

struct Storage {
    void* ptr = nullptr;
    size_t bytes = 0;    // rounded allocation size
    device::Pool pool = device::Pool::Activation;
    bool owned = true;   // false: wraps memory owned by someone else
    ~Storage();
};

class Tensor {
public:
    Tensor() = default;
    static Tensor empty(size_t rows, size_t cols, DType dt, device::Pool pool = device::Pool::Activation);
    // Rows `ld` elements apart (ld >= cols). Only GEMM outputs use a padded row stride (a
    // row stride that is a multiple of 16 bytes lets the tensor-core kernel write shapes
    // such as a 50257-wide vocabulary); every other consumer sees dense().
    static Tensor empty_strided(size_t rows, size_t cols, size_t ld, DType dt,
                                device::Pool pool = device::Pool::Activation);
    static Tensor zeros(size_t rows, size_t cols, DType dt, device::Pool pool = device::Pool::Activation);
    static Tensor from_host(const Matrix& m, DType dt = DType::F32, device::Pool pool = device::Pool::Activation);
    // Raw byte buffer (scratch, index arrays): rows = 1, cols = bytes, dtype tag F32 unused.
    static Tensor bytes(size_t nbytes, device::Pool pool = device::Pool::Activation);

    bool defined() const { return st_ != nullptr; }
    size_t rows() const { return rows_; }
    size_t cols() const { return cols_; }
    size_t numel() const { return rows_ * cols_; }
    size_t ld() const { return ld_ ? ld_ : cols_; }
    bool is_dense() const { return ld() == cols_; }
    // bytes spanned in memory (rows * ld)
    size_t nbytes() const { return rows_ * ld() * dtype_bytes(dt_); }
    Tensor dense() const;  // *this when dense, else a packed copy
    DType dtype() const { return dt_; }
    int dt() const { return static_cast<int>(dt_); }
    void* ptr() const { return st_ ? static_cast<char*>(st_->ptr) + off_ : nullptr; }
    float* f32() const { return static_cast<float*>(ptr()); }
    long use_count() const { return st_.use_count(); }

    // A [rows, cols] window starting `elem_offset` elements into this tensor's storage.
    Tensor view(size_t elem_offset, size_t rows, size_t cols) const;
    Tensor reshape(size_t rows, size_t cols) const;
    Tensor clone() const;
    Tensor cast(DType dt) const;  // returns *this when the dtype already matches
    void zero_();
    void copy_from_host(const Matrix& m);  // converts to this tensor's dtype
    Matrix to_host() const;                // synchronises

private:
    std::shared_ptr<Storage> st_;
    size_t off_ = 0;  // bytes
    size_t rows_ = 0, cols_ = 0, ld_ = 0;  // ld_ == 0: dense
    DType dt_ = DType::F32;
};

}  // namespace microtorch
