// GGUF v3 export (see the header for the layout and the reference it follows). The file is
// assembled in three byte strings -- key/value block, tensor directory, tensor data -- and
// written in one go, so offsets are known before anything reaches the disk.
#include "microtorch/gguf.hpp"

#include <cstring>
#include <fstream>
#include <stdexcept>

namespace microtorch {
namespace gguf {

namespace {

constexpr uint64_t kAlign = 32;
enum ValueType : uint32_t { kU32 = 4, kF32 = 6, kString = 8, kArray = 9 };

class Bytes {
public:
    template <typename T>
    void pod(T v) {  // little-endian host assumed, like the reference's writer
        const char* p = reinterpret_cast<const char*>(&v);
        buf_.append(p, sizeof(T));
    }
    void str(const std::string& s) {
        pod<uint64_t>(s.size());
        buf_.append(s);
    }
    void raw(const void* p, size_t n) { buf_.append(static_cast<const char*>(p), n); }
    void pad_to(uint64_t multiple) {
        while (buf_.size() % multiple != 0) buf_.push_back('\0');
    }
    size_t size() const { return buf_.size(); }
    const std::string& data() const { return buf_; }

private:
    std::string buf_;
};

struct KeyValues {
    Bytes out;
    uint64_t count = 0;
    void key(const std::string& k, ValueType t) {
        out.str(k);
        out.pod<uint32_t>(t);
        ++count;
    }
    void u32(const std::string& k, uint32_t v) {
        key(k, kU32);
        out.pod<uint32_t>(v);
    }
    void f32(const std::string& k, float v) {
        key(k, kF32);
        out.pod<float>(v);
    }
    void text(const std::string& k, const std::string& v) {
        key(k, kString);
        out.str(v);
    }
    void texts(const std::string& k, const std::vector<std::string>& v) {
        key(k, kArray);
        out.pod<uint32_t>(kString);
        out.pod<uint64_t>(v.size());
        for (const auto& s : v) out.str(s);
    }
    void floats(const std::string& k, const std::vector<float>& v) {
        key(k, kArray);
        out.pod<uint32_t>(kF32);
        out.pod<uint64_t>(v.size());
        for (const float f : v) out.pod<float>(f);
    }
};

struct Tensors {
    Bytes directory, data;
    uint64_t count = 0;
    // extents in the order they are stored (see `projection` below); values row-major
    void add(const std::string& name, const std::vector<uint64_t>& extents, const float* values, size_t n) {
        data.pad_to(kAlign);
        directory.str(name);
        directory.pod<uint32_t>(static_cast<uint32_t>(extents.size()));
        for (const uint64_t e : extents) directory.pod<uint64_t>(e);
        directory.pod<uint32_t>(0);  // F32
        directory.pod<uint64_t>(data.size());
        data.raw(values, n * sizeof(float));
        ++count;
    }
};

}  // namespace

void export_gguf_llama(const std::string& path, const std::map<std::string, Matrix>& state_dict,
                       const LlamaExportConfig& cfg, std::vector<std::string>* unmapped) {
    if (cfg.embedding_length == 0 || cfg.block_count == 0 || cfg.feed_forward_length == 0 || cfg.head_count == 0 ||
        cfg.vocab_size == 0)
        throw std::runtime_error("export_gguf_llama: embedding_length, block_count, feed_forward_length, "
                                 "head_count and vocab_size must all be set");
    const uint32_t kv_heads = cfg.head_count_kv ? cfg.head_count_kv : cfg.head_count;

    KeyValues kv;
    const std::string& a = cfg.architecture;
    kv.text("general.architecture", a);
    kv.text("general.name", cfg.name);
    kv.u32("general.alignment", static_cast<uint32_t>(kAlign));
    kv.u32(a + ".context_length", cfg.context_length);
    kv.u32(a + ".embedding_length", cfg.embedding_length);
    kv.u32(a + ".block_count", cfg.block_count);
    kv.u32(a + ".feed_forward_length", cfg.feed_forward_length);
    kv.u32(a + ".attention.head_count", cfg.head_count);
    kv.u32(a + ".attention.head_count_kv", kv_heads);
    kv.f32(a + ".attention.layer_norm_rms_epsilon", cfg.rms_eps);
    kv.u32(a + ".vocab_size", cfg.vocab_size);
    kv.f32(a + ".rope.freq_base", cfg.rope_freq_base);
    kv.u32(a + ".rope.dimension_count", cfg.embedding_length / cfg.head_count);
    if (!cfg.tokens.empty()) {
        kv.text("tokenizer.ggml.model", cfg.tokenizer_model);
        kv.texts("tokenizer.ggml.tokens", cfg.tokens);
        kv.floats("tokenizer.ggml.scores", std::vector<float>(cfg.tokens.size(), 0.0f));
        kv.u32("tokenizer.ggml.bos_token_id", cfg.bos_token_id);
        kv.u32("tokenizer.ggml.eos_token_id", cfg.eos_token_id);
        kv.u32("tokenizer.ggml.unknown_token_id", cfg.unk_token_id);
        kv.u32("tokenizer.ggml.padding_token_id", cfg.pad_token_id);
    }

    std::vector<std::string> used;
    auto lookup = [&](const std::string& key) -> const Matrix* {
        auto it = state_dict.find(key);
        if (it == state_dict.end()) it = state_dict.find("model." + key);
        return it == state_dict.end() ? nullptr : &it->second;
    };
    auto need = [&](const std::string& key) -> const Matrix& {
        const Matrix* m = lookup(key);
        if (!m) throw std::runtime_error("export_gguf_llama: missing tensor " + key);
        used.push_back(key);
        return *m;
    };

    Tensors t;
    std::vector<float> scratch;
    // A projection is written as [out][in] row-major values. The reference hands its writer the
    // shape {in, out} (src/gguf.cpp:80-96) and the writer stores a shape back to front
    // (gguf_export.cpp:296-299), so the directory holds {out, in}; kept, so that both exporters
    // write the same file. The same holds for the embedding ({vocab, hidden}).
    auto projection = [&](const Matrix& w, const std::string& name) {
        if (!cfg.weights_in_out) {  // stored [out, in] already
            t.add(name, {w.rows(), w.cols()}, w.data(), w.size());
            return;
        }
        const size_t in = w.rows(), out = w.cols();
        scratch.resize(in * out);
        const float* src = w.data();
        for (size_t i = 0; i < in; ++i)
            for (size_t j = 0; j < out; ++j) scratch[j * in + i] = src[i * out + j];
        t.add(name, {out, in}, scratch.data(), scratch.size());
    };
    auto gain = [&](const Matrix& g, const std::string& name) { t.add(name, {g.size()}, g.data(), g.size()); };

    {
        const Matrix& e = need("embed_tokens.weight");
        t.add("token_embd.weight", {e.rows(), e.cols()}, e.data(), e.size());
    }
    for (uint32_t l = 0; l < cfg.block_count; ++l) {
        const std::string from = "layers." + std::to_string(l) + ".", to = "blk." + std::to_string(l) + ".";
        projection(need(from + "self_attn.q_proj.weight"), to + "attn_q.weight");
        projection(need(from + "self_attn.k_proj.weight"), to + "attn_k.weight");
        projection(need(from + "self_attn.v_proj.weight"), to + "attn_v.weight");
        projection(need(from + "self_attn.o_proj.weight"), to + "attn_output.weight");
        gain(need(from + "input_layernorm.weight"), to + "attn_norm.weight");
        projection(need(from + "mlp.gate_proj.weight"), to + "ffn_gate.weight");
        projection(need(from + "mlp.up_proj.weight"), to + "ffn_up.weight");
        projection(need(from + "mlp.down_proj.weight"), to + "ffn_down.weight");
        gain(need(from + "post_attention_layernorm.weight"), to + "ffn_norm.weight");
    }
    gain(need("norm.weight"), "output_norm.weight");
    if (const Matrix* head = lookup("lm_head.weight")) {
        used.push_back("lm_head.weight");
        projection(*head, "output.weight");
    }
    if (unmapped) {
        for (const auto& [key, m] : state_dict) {
            (void)m;
            const std::string bare = key.rfind("model.", 0) == 0 ? key.substr(6) : key;
            bool hit = false;
            for (const auto& u : used) hit = hit || u == bare;
            if (!hit) unmapped->push_back(key);
        }
    }

    Bytes head;
    head.pod<uint32_t>(0x46554747u);  // "GGUF"
    head.pod<uint32_t>(3);
    head.pod<uint64_t>(t.count);
    head.pod<uint64_t>(kv.count);
    head.raw(kv.out.data().data(), kv.out.size());
    head.raw(t.directory.data().data(), t.directory.size());
    head.pad_to(kAlign);

    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("export_gguf_llama: cannot write " + path);
    f.write(head.data().data(), static_cast<std::streamsize>(head.size()));
    f.write(t.data.data().data(), static_cast<std::streamsize>(t.data.size()));
    if (!f) throw std::runtime_error("export_gguf_llama: write failed for " + path);
}

}  // namespace gguf
}  // namespace microtorch
