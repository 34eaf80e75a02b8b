#pragma once
// Surprise-routed attention of the reference's research models
// (include/microtorch/srd.hpp:26-64 there). Outside the checkpointed transformer-block training
// path: the class is declared so that code written against the reference's headers
// (tools/parity_model.hpp and what includes it) compiles unchanged; constructing it works,
// forward() throws std::runtime_error.
#include <vector>

#include "microtorch/nn.hpp"

namespace microtorch {
namespace nn {

class SurpriseRoutedAttention : public Module {
public:
    SurpriseRoutedAttention(size_t d, size_t n_heads, unsigned seed = 0);
    Var forward(const Var& x, size_t seq_len = 0) const;
    Var gate() const { return last_gate_; }
    std::shared_ptr<Linear> c_attn, c_proj;
    size_t H, dk;
    bool shuffle_predictor = false;
    mutable std::vector<float> forced_gate;

private:
    mutable Var last_gate_;
};

}  // namespace nn
}  // namespace microtorch
