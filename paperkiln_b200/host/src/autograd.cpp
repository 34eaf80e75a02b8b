// The tape: Value (device array + lazy host mirror), Variable, backward(), and the
// activation-checkpoint scheduler. Contract in microtorch/autograd.hpp.
#include "microtorch/autograd.hpp"

#include <stdexcept>
#include <unordered_set>

#include "pk.h"

namespace microtorch {

namespace detail {
std::atomic<size_t> g_live_vars{0};
}

size_t live_variables() { return detail::g_live_vars.load(); }

// ---------------------------------------------------------------- Value
const Matrix& Value::host() const {
    if (deferred_) materialise();
    if (!host_valid_) {
        if (dev_valid_) {
            host_ = dev_.to_host();
        } else {
            host_ = Matrix();
        }
        host_valid_ = true;
    }
    return host_;
}

Value Value::deferred(size_t rows, size_t cols, std::function<Tensor()> produce) {
    Value v;
    v.deferred_ = std::move(produce);
    v.def_rows_ = rows;
    v.def_cols_ = cols;
    return v;
}

void Value::materialise() const {
    std::function<Tensor()> produce = std::move(deferred_);
    deferred_ = nullptr;
    dev_ = produce();
    dev_valid_ = true;
    host_valid_ = false;
}

Matrix& Value::mutable_host() {
    (void)host();
    dev_valid_ = false;
    ++version_;
    return host_;
}

Value& Value::operator=(const Matrix& m) {
    deferred_ = nullptr;
    // Keep a device buffer of the same shape as the home of the data (parameters are
    // windows of a flat buffer and must stay there): write through instead of rebinding.
    if (dev_.defined() && dev_.rows() == m.rows() && dev_.cols() == m.cols() && dev_valid_) {
        dev_.copy_from_host(m);
        host_ = m;
        host_valid_ = true;
    } else {
        host_ = m;
        host_valid_ = true;
        dev_valid_ = false;
        if (dev_.defined() && (dev_.rows() != m.rows() || dev_.cols() != m.cols())) dev_ = Tensor();
    }
    ++version_;
    return *this;
}

Value& Value::operator=(Matrix&& m) { return *this = static_cast<const Matrix&>(m); }

void Value::fill(float v) {
    if (deferred_) materialise();
    if (dev_valid_ && v == 0.0f) {
        dev_.zero_();
        host_valid_ = false;
        ++version_;
        return;
    }
    Matrix m(rows(), cols(), v);
    *this = m;
}

const Tensor& Value::device() const {
    if (deferred_) materialise();
    if (!dev_valid_) {
        if (!host_valid_) throw std::runtime_error("Value::device on an empty value");
        if (dev_.defined() && dev_.rows() == host_.rows() && dev_.cols() == host_.cols()) {
            dev_.copy_from_host(host_);
        } else {
            dev_ = Tensor::from_host(host_, DType::F32);
        }
        dev_valid_ = true;
    }
    return dev_;
}

void Value::set_device(Tensor t) {
    deferred_ = nullptr;
    dev_ = std::move(t);
    dev_valid_ = true;
    host_valid_ = false;
    host_ = Matrix();
    ++version_;
}

void Value::reset() {
    deferred_ = nullptr;
    dev_ = Tensor();
    host_ = Matrix();
    dev_valid_ = host_valid_ = false;
    ++version_;
}

// ---------------------------------------------------------------- Variable
DType Variable::grad_dtype() const { return is_param ? DType::F32 : device::compute_dtype(); }

const Tensor& Variable::compute() const {
    const DType want = device::compute_dtype();
    if (!data.device().is_dense()) {
        // a GEMM output with a padded row stride meets a consumer that wants packed rows
        Variable* self = const_cast<Variable*>(this);
        self->data.set_device(data.device().dense());
    }
    const Tensor& d = data.device();
    if (d.dtype() == want) return d;
    Variable* self = const_cast<Variable*>(this);
    if (!shadow.defined() || shadow.dtype() != want || shadow.rows() != d.rows() || shadow.cols() != d.cols()) {
        self->shadow = Tensor::empty(d.rows(), d.cols(), want,
                                     is_param ? device::Pool::Persistent : device::Pool::Activation);
        self->shadow_version = ~uint64_t(0);
    }
    if (shadow_version != data.version()) {
        device::check(pk_cast(device::stream(), d.dt(), d.ptr(), shadow.dt(), shadow.ptr(),
                              static_cast<int64_t>(d.numel())), "pk_cast");
        self->shadow_version = data.version();
    }
    return shadow;
}

const Tensor& Variable::compute_strided() const {
    const Tensor& d = data.device();
    if (d.dtype() == device::compute_dtype()) return d;
    return compute();
}

Tensor& Variable::grad_for_accumulate() {
    if (grad.empty()) {
        if (grad_home.defined()) {
            grad.set_device(grad_home);  // flat buffer window: zero by contract
        } else {
            grad.set_device(Tensor::zeros(data.rows(), data.cols(), grad_dtype(),
                                          is_param ? device::Pool::Persistent : device::Pool::Activation));
        }
    }
    grad.mark_device_modified();
    return const_cast<Tensor&>(grad.device());
}

void Variable::accumulate(const Tensor& g) {
    if (g.rows() != data.rows() || g.cols() != data.cols())
        throw std::runtime_error("accumulate: gradient shape mismatch");
    const DType want = grad_dtype();
    void* s = device::stream();
    if (grad.empty() && !grad_home.defined() && g.dtype() == want) {
        grad.set_device(g);  // adopt: no copy, no add
        return;
    }
    if (!g.is_dense() || (!grad.empty() && !grad.device().is_dense())) {
        // element-wise sums need packed rows on both sides
        const Tensor gd = g.dense();
        if (!grad.empty() && !grad.device().is_dense()) grad.set_device(grad.device().dense());
        accumulate(gd);
        return;
    }
    if (grad.empty()) {
        Tensor& dst = grad_for_accumulate();
        device::check(pk_axpy(s, dst.dt(), dst.ptr(), g.dt(), g.ptr(), 1.0f, static_cast<int64_t>(g.numel())), "pk_axpy");
        return;
    }
    const Tensor& cur = grad.device();
    if (cur.use_count() > 1 && !grad_home.defined()) {
        // The buffer was adopted from (and may still be referenced by) another node:
        // write the sum to a fresh buffer instead of updating it in place.
        Tensor sum = Tensor::empty(cur.rows(), cur.cols(), cur.dtype());
        if (g.dtype() == cur.dtype()) {
            device::check(pk_binary(s, cur.dt(), 0, cur.ptr(), g.ptr(), sum.ptr(), static_cast<int64_t>(g.numel())), "pk_binary");
        } else {
            device::check(pk_memcpy_d2d(sum.ptr(), cur.ptr(), cur.nbytes(), s), "pk_memcpy_d2d");
            device::check(pk_axpy(s, sum.dt(), sum.ptr(), g.dt(), g.ptr(), 1.0f, static_cast<int64_t>(g.numel())), "pk_axpy");
        }
        grad.set_device(std::move(sum));
        return;
    }
    device::check(pk_axpy(s, cur.dt(), cur.ptr(), g.dt(), g.ptr(), 1.0f, static_cast<int64_t>(g.numel())), "pk_axpy");
    grad.mark_device_modified();
}

void Variable::accumulate(const Matrix& g) {
    if (g.rows() != data.rows() || g.cols() != data.cols())
        throw std::runtime_error("accumulate: gradient shape mismatch");
    if (grad.empty() && !grad_home.defined() && !device::initialized()) {
        grad = g;
        return;
    }
    if (grad.empty() && !grad_home.defined() && g.rows() * g.cols() == 1) {
        grad = g;  // scalar seed: stays host-known, so the loss backward needs no readback
        return;
    }
    accumulate(Tensor::from_host(g, grad_dtype()));
}

// ---------------------------------------------------------------- backward
namespace {

thread_local bool g_grad_enabled = true;
thread_local int g_recompute_depth = 0;
bool g_release_interior = true;
std::function<void(int)> g_segment_hook;
int g_segment_counter = 0;

// Post-order DFS over parents (iterative: the depth of a tape must not be bounded by the
// C++ stack). Collects owning pointers so that nodes may drop their parents while the
// order is being walked.
void topo(const Var& root, std::vector<Var>& order) {
    std::unordered_set<Variable*> seen;
    std::vector<std::pair<Var, size_t>> stack;
    stack.emplace_back(root, 0);
    seen.insert(root.get());
    while (!stack.empty()) {
        auto& top = stack.back();
        if (top.second < top.first->parents.size()) {
            const Var& p = top.first->parents[top.second++];
            if (seen.insert(p.get()).second) stack.emplace_back(p, 0);
        } else {
            order.push_back(top.first);
            stack.pop_back();
        }
    }
}

// level 0: keep everything; 1: drop closure + gradient of interior nodes once used;
// 2: also drop their output data and parent links (private sub-tapes only).
void run_reverse(std::vector<Var>& order, int level, const Variable* keep_grad_of) {
    if (level >= 2) {
        // consumers per node (a node that appears twice among a consumer's parents counts twice)
        for (const Var& v : order) v->pending_consumers = 0;
        for (const Var& v : order)
            for (const Var& p : v->parents) ++p->pending_consumers;
    }
    for (auto it = order.rbegin(); it != order.rend(); ++it) {
        Variable* n = it->get();
        if (n->backward_fn && !n->grad.empty()) n->backward_fn();
        if (level >= 2) {
            // an input whose last consumer has now run is dead: free it here, not when its own
            // closure comes up (several closures later, with new gradients allocated in between)
            for (const Var& p : n->parents)
                if (p->pending_consumers > 0 && --p->pending_consumers == 0 && !p->is_leaf()) {
                    p->data.reset();
                    p->shadow = Tensor();
                }
        }
        if (level >= 1 && !n->is_leaf()) {
            n->backward_fn = nullptr;
            if (n != keep_grad_of) n->grad.reset();
            if (level >= 2) {
                n->data.reset();
                n->parents.clear();
            }
        }
        if (level >= 2) {
            n->pending_consumers = -1;
            it->reset();
        }
    }
}

}  // namespace

void backward(const Var& root) {
    if (root->data.rows() != 1 || root->data.cols() != 1)
        throw std::runtime_error("backward: root must be a [1,1] scalar (compose with mean/sum)");
    Matrix seed(1, 1);
    seed(0, 0) = 1.0f;
    root->accumulate(seed);
    g_segment_counter = 0;
    std::vector<Var> order;
    topo(root, order);
    run_reverse(order, g_release_interior ? 1 : 0, root.get());
}

void backward_from(const Var& root, const Tensor& upstream) {
    if (upstream.rows() != root->data.rows() || upstream.cols() != root->data.cols())
        throw std::runtime_error("backward_from: upstream gradient shape differs from the root's");
    root->accumulate(upstream);
    g_segment_counter = 0;
    std::vector<Var> order;
    topo(root, order);
    run_reverse(order, g_release_interior ? 1 : 0, root.get());
}

Var checkpoint(const std::function<Var(const Var&)>& fn, const Var& x) {
    if (!grad_enabled()) return fn(x);
    Value out_data;
    {
        NoGrad ng;
        Var y = fn(x);           // no tape: interior activations die as they go out of scope
        out_data = y->data;      // shares the device buffer, no copy
    }
    Var out = std::make_shared<Variable>(std::move(out_data), true);
    out->parents = {x};
    Variable* self = out.get();
    auto fn_copy = fn;
    out->backward_fn = [self, fn_copy]() {
        const Var xin = self->parents[0];
        // Recompute on a detached leaf that aliases the stored boundary activation.
        Var x2 = std::make_shared<Variable>(Value(xin->data.device()), true);
        ++g_recompute_depth;
        Var y2;
        try {
            y2 = fn_copy(x2);
        } catch (...) {
            --g_recompute_depth;
            throw;
        }
        --g_recompute_depth;
        if (y2->data.rows() != self->grad.rows() || y2->data.cols() != self->grad.cols())
            throw std::runtime_error("checkpoint: recomputed output shape mismatch");
        y2->accumulate(self->grad.device());
        std::vector<Var> order;
        topo(y2, order);
        y2.reset();
        run_reverse(order, 2, nullptr);
        order.clear();
        if (xin->requires_grad && !x2->grad.empty()) xin->accumulate(x2->grad.device());
        x2.reset();
        if (g_segment_hook) g_segment_hook(g_segment_counter);
        ++g_segment_counter;
    };
    return out;
}

void zero_grad(const std::vector<Var>& vars) {
    // Adjacent gradient windows of a flat buffer are cleared with one memset.
    void* run_begin = nullptr;
    size_t run_bytes = 0;
    auto flush = [&]() {
        if (run_begin) device::check(pk_memset(run_begin, 0, run_bytes, device::stream()), "pk_memset");
        run_begin = nullptr;
        run_bytes = 0;
    };
    for (const auto& v : vars) {
        if (v->grad.empty()) continue;
        if (!v->grad.on_device()) {
            v->grad.fill(0.0f);
            continue;
        }
        const Tensor& g = v->grad.device();
        v->grad.mark_device_modified();
        char* p = static_cast<char*>(g.ptr());
        if (run_begin && static_cast<char*>(run_begin) + run_bytes <= p &&
            p - (static_cast<char*>(run_begin) + run_bytes) <= 256 && v->grad_home.defined()) {
            run_bytes = static_cast<size_t>(p - static_cast<char*>(run_begin)) + g.nbytes();
        } else {
            flush();
            run_begin = p;
            run_bytes = g.nbytes();
        }
    }
    flush();
}

bool grad_enabled() { return g_grad_enabled; }
bool recomputing() { return g_recompute_depth > 0; }
NoGrad::NoGrad() : prev_(g_grad_enabled) { g_grad_enabled = false; }
NoGrad::~NoGrad() { g_grad_enabled = prev_; }

namespace autograd {
bool disposable_input(const Var& v) {
    return v && v->pending_consumers == 1 && !v->is_leaf() && !v->data.pending() && v->data.on_device() && v->data.device().use_count() == 1 &&
           v->data.device().is_dense() && !v->shadow.defined();
}
void set_release_interior(bool on) { g_release_interior = on; }
bool release_interior() { return g_release_interior; }
void set_segment_hook(std::function<void(int)> hook) { g_segment_hook = std::move(hook); }
}  // namespace autograd

}  // namespace microtorch
