#pragma once
// GGUF (version 3) export of a Llama-family state dict: the same entry point, configuration
// struct, tensor naming and byte layout as the reference's exporter
// (include/microtorch/gguf.hpp:20-66, src/gguf.cpp:27-166, which drives the writer of its vendored
// tree, third_party/transformer_cpp/src/gguf_export.cpp:265-366), so that a file written here is
// the file the reference would write from the same tensors.
//
// Layout: "GGUF", version 3, tensor count, key/value count (u64 each); key/value pairs in the
// order given below (key string, u32 type, value); per tensor: name, u32 rank, u64 extents
// (as the reference stores them: {out, in} for a projection whose values are [out][in]
// row-major), u32 type (0 = F32), u64 offset relative to the data section; zero padding
// to a multiple of 32; tensor data, each tensor starting on a multiple of 32.
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "microtorch/matrix.hpp"

namespace microtorch {
namespace gguf {

struct LlamaExportConfig {
    std::string name = "microtorch-model";
    std::string architecture = "llama";
    uint32_t context_length = 2048;
    uint32_t embedding_length = 0;     // d_model (required)
    uint32_t block_count = 0;          // layers (required)
    uint32_t feed_forward_length = 0;  // d_ff (required)
    uint32_t head_count = 0;           // query heads (required)
    uint32_t head_count_kv = 0;        // 0: same as head_count
    uint32_t vocab_size = 0;           // required
    float rms_eps = 1e-6f;
    float rope_freq_base = 10000.0f;
    // false: projections are stored [out, in] (HF checkpoints) and written as they are;
    // true: stored [in, out] (this library's Linear, y = x W) and transposed on export.
    bool weights_in_out = false;
    // Optional token list; empty: no tokenizer block.
    std::vector<std::string> tokens;
    std::string tokenizer_model = "word";
    uint32_t bos_token_id = 1, eos_token_id = 1;
    uint32_t unk_token_id = 0, pad_token_id = 0;
};

// state_dict names (a leading "model." is optional on each):
//   embed_tokens.weight -> token_embd.weight;  layers.N.self_attn.{q,k,v,o}_proj.weight ->
//   blk.N.attn_{q,k,v,output}.weight;  layers.N.input_layernorm.weight -> blk.N.attn_norm.weight;
//   layers.N.mlp.{gate,up,down}_proj.weight -> blk.N.ffn_{gate,up,down}.weight;
//   layers.N.post_attention_layernorm.weight -> blk.N.ffn_norm.weight;  norm.weight ->
//   output_norm.weight;  lm_head.weight -> output.weight (left out when absent: tied head).
// Entries that map to nothing are listed in `unmapped`. Throws std::runtime_error when a
// required tensor or configuration field is missing.
void export_gguf_llama(const std::string& path, const std::map<std::string, Matrix>& state_dict,
                       const LlamaExportConfig& cfg, std::vector<std::string>* unmapped = nullptr);

}  // namespace gguf
}  // namespace microtorch
