#pragma once
// Batch-sharded data parallelism for the checkpointed training step, on the host side of the
// collective group of the C ABI (pk_comm_* / pk_allreduce_async in pk.h).
//
// Sequences are independent and the loss is a mean, so rank r runs B/g sequences of the global
// batch with its loss scaled by 1/g and the ranks exchange one thing: the SUM of their fp32
// parameter gradients. With packed parameters (nn::pack_parameters) the gradients of one
// transformer block are one contiguous range -- a bucket. GradientExchange starts the all-reduce
// of block i's bucket from the tape's segment hook, i.e. as soon as the backward of that block's
// checkpointed segment has been enqueued, so the transfer overlaps the recompute + backward of
// block i - 1; what is left (embeddings, final norm, head; every block of a model run without
// checkpointing) goes out in finish(), which then orders the compute stream behind all transfers
// without blocking the host. A model whose trainable gradients are small (LoRA adapters only) is
// exchanged as one flat buffer in one collective: it is latency-bound, not bandwidth-bound.
//
// The reference has no multi-GPU path; the identity is that of its gradient accumulation loop
// (tools/mtstudio.cpp:456-474).
#include <cstddef>
#include <cstdint>
#include <utility>
#include <vector>

namespace microtorch {
namespace dp {

class GradientExchange {
public:
    // `comm` is a handle from pk_comm_init / pk_comm_init_file (ownership passes to this object).
    // buckets: (device pointer, fp32 element count) per transformer block in forward order, then
    // one for everything else. flat: the whole gradient buffer (used when it is small).
    GradientExchange(void* comm, std::vector<std::pair<float*, int64_t>> buckets, std::pair<float*, int64_t> flat);
    ~GradientExchange();
    GradientExchange(const GradientExchange&) = delete;
    GradientExchange& operator=(const GradientExchange&) = delete;

    // Installs / removes this object as the tape's segment hook.
    void attach();
    void detach();
    // Under gradient accumulation the buckets are complete only after the last micro-batch.
    void set_enabled(bool on) { enabled_ = on; }
    // The k-th finished segment of a backward pass is block (n_blocks - 1 - k).
    void on_segment(int k);
    // Sends what has not been sent in this step, then makes the compute stream wait for all of it.
    void finish();
    // Blocks the host until the transfers are done; throws after the time limit (communicator aborted).
    void wait_host();
    void set_timeout(double seconds);
    bool single_collective() const { return single_; }
    // Gradient bytes up to which the whole buffer goes out as one collective (default 32 MiB).
    void set_flat_threshold(int64_t bytes);
    int64_t launches_last_step() const { return launches_last_; }
    static constexpr int64_t kSingleCollectiveBytes = int64_t(32) << 20;

private:
    void launch(size_t i);
    void* comm_;
    std::vector<std::pair<float*, int64_t>> buckets_;
    std::pair<float*, int64_t> flat_;
    std::vector<bool> sent_;
    bool enabled_ = true, attached_ = false, single_ = false;
    int64_t launches_ = 0, launches_last_ = 0;
};

}  // namespace dp
}  // namespace microtorch
