// Gradient exchange of the data-parallel training step (microtorch/dp.hpp) over the collective
// group of libpk.
#include "microtorch/dp.hpp"

#include <stdexcept>
#include <string>

#include "microtorch/autograd.hpp"
#include "pk.h"

namespace microtorch {
namespace dp {

using device::check;

GradientExchange::GradientExchange(void* comm, std::vector<std::pair<float*, int64_t>> buckets,
                                   std::pair<float*, int64_t> flat)
    : comm_(comm), buckets_(std::move(buckets)), flat_(flat), sent_(buckets_.size(), false) {
    if (!comm_) throw std::runtime_error("GradientExchange: null communicator");
    if (buckets_.empty()) throw std::runtime_error("GradientExchange: no gradient buckets (the model must be packed)");
    single_ = flat_.first != nullptr && flat_.second * int64_t(sizeof(float)) <= kSingleCollectiveBytes;
}

GradientExchange::~GradientExchange() {
    detach();
    pk_comm_destroy(comm_);
}

void GradientExchange::attach() {
    autograd::set_segment_hook([this](int k) { on_segment(k); });
    attached_ = true;
}

void GradientExchange::detach() {
    if (attached_) autograd::set_segment_hook(nullptr);
    attached_ = false;
}

void GradientExchange::launch(size_t i) {
    check(pk_allreduce_async(comm_, buckets_[i].first, buckets_[i].second, device::stream()), "pk_allreduce_async");
    sent_[i] = true;
    ++launches_;
}

void GradientExchange::on_segment(int k) {
    if (!enabled_ || single_) return;
    const int n_blocks = static_cast<int>(buckets_.size()) - 1;
    const int i = n_blocks - 1 - k;
    if (i >= 0 && i < n_blocks && !sent_[static_cast<size_t>(i)]) launch(static_cast<size_t>(i));
}

void GradientExchange::finish() {
    if (single_) {
        check(pk_allreduce_async(comm_, flat_.first, flat_.second, device::stream()), "pk_allreduce_async");
        ++launches_;
    } else {
        for (size_t i = 0; i < buckets_.size(); ++i)
            if (!sent_[i]) launch(i);
    }
    check(pk_comm_wait(comm_, device::stream()), "pk_comm_wait");
    sent_.assign(buckets_.size(), false);
    launches_last_ = launches_;
    launches_ = 0;
}

void GradientExchange::set_flat_threshold(int64_t bytes) {
    single_ = flat_.first != nullptr && flat_.second * int64_t(sizeof(float)) <= bytes;
}

void GradientExchange::wait_host() { check(pk_comm_wait_host(comm_), "pk_comm_wait_host"); }
void GradientExchange::set_timeout(double seconds) { check(pk_comm_set_timeout(comm_, seconds), "pk_comm_set_timeout"); }

}  // namespace dp
}  // namespace microtorch
