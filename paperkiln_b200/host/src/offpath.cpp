// Entry points of the reference's research mechanisms that this library declares for source
// compatibility and does not provide (see the notes in microtorch/ops.hpp, nn.hpp, srd.hpp):
// Kimi linear attention, sliding-window attention, surprise-routed attention, the
// depth-attention stack. Layers that own plain Linear projections are constructible, so a model
// header that lists them compiles and builds; running one of them reports what is missing.
#include <stdexcept>
#include <string>

#include "microtorch/nn.hpp"
#include "microtorch/ops.hpp"
#include "microtorch/srd.hpp"

namespace microtorch {

namespace {
[[noreturn]] void not_provided(const char* what) {
    throw std::runtime_error(std::string(what) +
                             ": not provided by this build (outside the checkpointed transformer-block training path)");
}
void check_heads(size_t d, size_t n_heads, const char* what) {
    if (n_heads == 0 || d % n_heads != 0) throw std::runtime_error(std::string(what) + ": d must divide by n_heads");
}
}  // namespace

namespace ops {
Var kimi_attention(const Var&, const Var&, const Var&, bool) { not_provided("kimi_attention"); }
}  // namespace ops

namespace nn {

SlidingWindowAttention::SlidingWindowAttention(size_t d, size_t n_heads, size_t window_, size_t sinks_, unsigned seed)
    : H(n_heads), dk(n_heads ? d / n_heads : 0), window(window_), sinks(sinks_) {
    check_heads(d, n_heads, "SlidingWindowAttention");
    c_attn = mod<Linear>("c_attn", d, 3 * d, true, seed);
    c_proj = mod<Linear>("c_proj", d, d, true, seed + 1);
}
Var SlidingWindowAttention::forward(const Var&, size_t) const { not_provided("SlidingWindowAttention::forward"); }

KimiLinearAttention::KimiLinearAttention(size_t d, size_t n_heads, unsigned seed, bool causal_)
    : H(n_heads), dk(n_heads ? d / n_heads : 0), causal(causal_) {
    check_heads(d, n_heads, "KimiLinearAttention");
    c_attn = mod<Linear>("c_attn", d, 3 * d, true, seed);
    c_proj = mod<Linear>("c_proj", d, d, true, seed + 1);
}
Var KimiLinearAttention::forward(const Var&, size_t) const { not_provided("KimiLinearAttention::forward"); }

SurpriseRoutedAttention::SurpriseRoutedAttention(size_t d, size_t n_heads, unsigned seed)
    : H(n_heads), dk(n_heads ? d / n_heads : 0) {
    check_heads(d, n_heads, "SurpriseRoutedAttention");
    c_attn = mod<Linear>("c_attn", d, 3 * d, true, seed);
    c_proj = mod<Linear>("c_proj", d, d, true, seed + 1);
}
Var SurpriseRoutedAttention::forward(const Var&, size_t) const { not_provided("SurpriseRoutedAttention::forward"); }

AttnResStack::AttnResStack(std::vector<std::shared_ptr<Module>>, std::vector<std::function<Var(const Var&)>>, size_t,
                           size_t block_size_)
    : block_size(block_size_) {
    not_provided("AttnResStack");
}
Var AttnResStack::forward(const Var&) const { not_provided("AttnResStack::forward"); }

}  // namespace nn
}  // namespace microtorch
