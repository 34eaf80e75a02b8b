#pragma once
// Reverse-mode tape with device-resident tensors and the activation-checkpoint
// scheduler.
//
// Public surface = the reference's include/microtorch/autograd.hpp:64-103
// (make_var, backward, zero_grad, checkpoint(fn, x), NoGrad, grad_enabled,
// live_variables; Variable{data, grad, requires_grad, parents, backward_fn}).
// What differs is where the numbers live: `data` and `grad` are Values -- 2-D
// arrays whose home is GPU memory and whose host Matrix is materialised only
// when somebody reads it (a test, a binding, state_dict).
//
// Checkpoint scheduling (reference semantics: src/autograd.cpp:68-102)
//   forward   fn(x) runs under NoGrad; every interior activation is returned
//             to the allocator as soon as its last consumer has run; only the
//             segment output survives
//   backward  the segment is re-run under grad on a leaf that ALIASES the
//             stored boundary (no copy); the upstream gradient is pushed
//             through the fresh sub-tape, whose nodes drop their saved
//             tensors, gradients and outputs as soon as their closure has
//             run; then the "segment done" hook fires (data-parallel runs use
//             it to start the gradient all-reduce of that block while the next
//             block recomputes)
// Every kernel is deterministic, so the recomputed activations are the bits the
// forward pass produced, and gradients with and without checkpointing are equal.
#include <atomic>
#include <functional>
#include <memory>
#include <vector>

#include "microtorch/device.hpp"

namespace microtorch {

// Device array with a lazily synchronised host mirror.
class Value {
public:
    Value() = default;
    Value(const Matrix& m) : host_(m), host_valid_(true) {}              // NOLINT: implicit by design
    Value(Matrix&& m) : host_(std::move(m)), host_valid_(true) {}       // NOLINT
    explicit Value(Tensor t) : dev_(std::move(t)), dev_valid_(true) {}
    // A [rows, cols] device value whose producer has not run yet: `produce` is called by the first
    // device() / host() that wants the contents, and never if nobody does. An op uses this for
    // an output that may turn out to be dead (the last projection of a recomputed segment: its
    // backward needs the inputs, not the value).
    static Value deferred(size_t rows, size_t cols, std::function<Tensor()> produce);
    bool pending() const { return static_cast<bool>(deferred_); }

    size_t rows() const { return deferred_ ? def_rows_ : dev_valid_ ? dev_.rows() : host_.rows(); }
    size_t cols() const { return deferred_ ? def_cols_ : dev_valid_ ? dev_.cols() : host_.cols(); }
    bool empty() const { return rows() == 0; }

    // Host view; downloads (and synchronises) when the device copy is newer.
    const Matrix& host() const;
    operator const Matrix&() const { return host(); }  // NOLINT
    float operator()(size_t i, size_t j) const { return host()(i, j); }
    // Element of the host view that can be assigned to (v->data(i, j) = x, as code written for
    // the reference does): like mutable_host(), so the device copy is refreshed on its next use.
    // Code that only reads should go through host().
    float& operator()(size_t i, size_t j) { return mutable_host()(i, j); }
    // Mutable host access: the device copy becomes stale and is re-uploaded on next use.
    Matrix& mutable_host();
    Value& operator=(const Matrix& m);
    Value& operator=(Matrix&& m);
    void fill(float v);

    // Device view; uploads when the host copy is newer. fp32 unless the value was
    // produced on the device in another dtype.
    const Tensor& device() const;
    // Replace / adopt a device tensor (host mirror becomes stale).
    void set_device(Tensor t);
    // Call after writing through device() pointers in place.
    void mark_device_modified() { host_valid_ = false; ++version_; }
    bool on_device() const { return dev_valid_ || deferred_; }
    uint64_t version() const { return version_; }
    void reset();

private:
    mutable Tensor dev_;
    mutable Matrix host_;
    mutable bool host_valid_ = false;
    mutable bool dev_valid_ = false;
    mutable std::function<Tensor()> deferred_;
    size_t def_rows_ = 0, def_cols_ = 0;
    uint64_t version_ = 0;
    void materialise() const;
};

class Variable;
using Var = std::shared_ptr<Variable>;

namespace detail {
extern std::atomic<size_t> g_live_vars;
}

class Variable {
public:
    Value data;
    Value grad;  // empty until the first accumulate()
    bool requires_grad = false;
    bool is_param = false;  // registered by a Module: gradient kept in fp32

    std::vector<Var> parents;
    std::function<void()> backward_fn;

    // While the private sub-tape of a checkpointed segment runs its backward pass: how many of this
    // node's consumers have not run their closure yet (-1 outside such a pass). When it reaches
    // zero the node's output is dead -- no closure reads its own node's output -- and is returned
    // to the allocator at once; a closure that finds 1 here (itself) on an interior input whose
    // buffer nobody else references may overwrite that input with the gradient it produces
    // (disposable_input()).
    int pending_consumers = -1;

    // Optional preallocated home of the gradient (a window of a flat buffer shared by
    // all parameters of a model); used on the first accumulate() instead of a fresh
    // allocation. Must be zero when adopted.
    Tensor grad_home;

    explicit Variable(Value d, bool rg = false) : data(std::move(d)), requires_grad(rg) { ++detail::g_live_vars; }
    ~Variable() { --detail::g_live_vars; }
    Variable(const Variable&) = delete;
    Variable& operator=(const Variable&) = delete;

    bool is_leaf() const { return parents.empty(); }
    DType grad_dtype() const;

    // grad += g. The first contribution adopts g's buffer when that is safe (no copy).
    void accumulate(const Tensor& g);
    void accumulate(const Matrix& g);
    // Gradient buffer to accumulate into in place (allocated and zeroed on first use).
    Tensor& grad_for_accumulate();

    // Tensor of `data` in the compute dtype (cached cast for fp32 leaves in bf16 mode),
    // with packed rows.
    const Tensor& compute() const;
    // Same, but a padded row stride is kept (for consumers that take a leading dimension).
    const Tensor& compute_strided() const;
    // bf16 shadow slot that the optimizer refreshes in the same pass as the fp32 master.
    Tensor shadow;
    uint64_t shadow_version = ~uint64_t(0);
};

size_t live_variables();

inline Var make_var(Matrix data, bool requires_grad = false) {
    return std::make_shared<Variable>(Value(std::move(data)), requires_grad);
}
inline Var make_var(Tensor data, bool requires_grad = false) {
    return std::make_shared<Variable>(Value(std::move(data)), requires_grad);
}
inline Var make_var(const Value& data, bool requires_grad = false) {
    return std::make_shared<Variable>(data, requires_grad);
}

// Reverse pass from a [1,1] root.
void backward(const Var& root);
void zero_grad(const std::vector<Var>& vars);

Var checkpoint(const std::function<Var(const Var&)>& fn, const Var& x);
// Extension (no counterpart in the reference, whose backward() needs a scalar root): reverse
// pass from a root of any shape, seeded with an upstream gradient of the same shape.
void backward_from(const Var& root, const Tensor& upstream);

bool grad_enabled();
// True while a checkpointed segment is being re-run on its private tape during backward.
bool recomputing();
class NoGrad {
public:
    NoGrad();
    ~NoGrad();
    NoGrad(const NoGrad&) = delete;
    NoGrad& operator=(const NoGrad&) = delete;

private:
    bool prev_;
};

namespace autograd {
// True when `v` is an interior node of a private sub-tape, this closure is its last pending
// consumer and nobody else references its buffer: the closure may then write a result of the same
// shape and dtype over v's data (after it has read it) instead of allocating.
bool disposable_input(const Var& v);
// After a node's closure has run during the top-level backward(), drop its closure and
// its gradient (interior nodes only; leaves keep theirs). On by default: interior
// gradients of a [tokens, d_model] network are most of the backward's memory. Switch
// off to inspect interior gradients after backward(), as the reference allows.
void set_release_interior(bool on);
bool release_interior();
// Called after the backward of each checkpointed segment, with a running index that
// restarts at 0 for every backward() call (segments finish in reverse forward order).
void set_segment_hook(std::function<void(int)> hook);
}  // namespace autograd

}  // namespace microtorch
