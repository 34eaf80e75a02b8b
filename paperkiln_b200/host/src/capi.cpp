// C driver entry points (include/mt_capi.h) over the C++ host library.
#include "mt_capi.h"

#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>

#include "pk.h"

#include "microtorch/dp.hpp"
#include "microtorch/flex.hpp"
#include "microtorch/gguf.hpp"
#include "microtorch/llama.hpp"
#include "microtorch/nn.hpp"
#include "microtorch/safetensors.hpp"

using namespace microtorch;

namespace {

thread_local std::string g_err;

struct Model {
    std::string family;
    std::shared_ptr<nn::Llama> llama;
    std::shared_ptr<nn::GPT2> gpt2;
    std::shared_ptr<parity::FlexLM> flex;
    std::shared_ptr<nn::LlamaBlock> block;   // family "block": one Llama block, no embedding / head
    Var bx, by;                               // its input leaf and pending output
    Tensor bdy;                               // upstream gradient
    std::vector<int> bpos;
    size_t bseq = 0;
    bool block_ckpt = false;
    std::vector<std::pair<std::string, Var>> named;   // registration order
    std::vector<Var> params;                          // packed order (blocks first)
    std::vector<std::pair<size_t, size_t>> buckets;   // [first, last] index into params
    nn::ParamPack pack;
    bool packed = false;
    std::unique_ptr<nn::AdamW> opt;
    std::unique_ptr<dp::GradientExchange> exchange;   // data-parallel gradient exchange (mt_dp_*)
    float lr = 1e-3f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f, wd = 0.01f;
    int64_t live_after_fwd = 0;
    size_t loss_chunk = 16384;
    bool accumulate = false;   // mt_model_step keeps the gradients it finds

    Var forward(const std::vector<int>& ids, size_t seq_len) const {
        if (block) throw std::runtime_error("a block has no token interface: use mt_block_set_input / forward / backward");
        if (llama) return llama->forward(ids, seq_len);
        if (gpt2) return gpt2->forward(ids, seq_len);
        return flex->forward(ids, seq_len);
    }
    Var loss(const std::vector<int>& ids, const std::vector<int>& targets, size_t seq_len) const {
        if (block) throw std::runtime_error("a block has no token interface: use mt_block_set_input / forward / backward");
        if (loss_chunk == 0) return ops::cross_entropy(forward(ids, seq_len), targets);
        if (llama) return llama->loss(ids, targets, seq_len, loss_chunk);
        if (gpt2) return gpt2->loss(ids, targets, seq_len, loss_chunk);
        return flex->loss(ids, targets, seq_len, loss_chunk);
    }
    void set_ckpt(bool on) {
        if (llama) llama->checkpoint_blocks = on;
        if (gpt2) gpt2->checkpoint_blocks = on;
        if (flex) flex->checkpoint_blocks = on;
        block_ckpt = on;
    }
};

std::map<std::string, std::string> parse_spec(const char* spec) {
    std::map<std::string, std::string> kv;
    std::stringstream ss(spec ? spec : "");
    std::string item;
    while (std::getline(ss, item, ';')) {
        if (item.empty()) continue;
        const size_t eq = item.find('=');
        if (eq == std::string::npos) throw std::runtime_error("model spec: expected key=value, got '" + item + "'");
        kv[item.substr(0, eq)] = item.substr(eq + 1);
    }
    return kv;
}

struct SpecReader {
    std::map<std::string, std::string> kv;
    std::map<std::string, bool> used;
    std::string str(const std::string& k, const std::string& d) {
        used[k] = true;
        auto it = kv.find(k);
        return it == kv.end() ? d : it->second;
    }
    long num(const std::string& k, long d) {
        used[k] = true;
        auto it = kv.find(k);
        return it == kv.end() ? d : std::stol(it->second);
    }
    double real(const std::string& k, double d) {
        used[k] = true;
        auto it = kv.find(k);
        return it == kv.end() ? d : std::stod(it->second);
    }
    void finish() {
        for (auto& e : kv)
            if (!used.count(e.first)) throw std::runtime_error("model spec: unknown key '" + e.first + "'");
    }
};

// Rows per chunk of the fused head + loss: about 2^29 logits per chunk (1 GiB in bf16), so a wide
// vocabulary gets shorter chunks; 1024 ... 16384 rows, a multiple of 1024.
size_t default_loss_chunk(size_t vocab) {
    size_t rows = (size_t(1) << 29) / (vocab ? vocab : 1) / 1024 * 1024;
    if (rows < 1024) rows = 1024;
    if (rows > 16384) rows = 16384;
    return rows;
}

// Index of the transformer block a parameter belongs to, or -1.
long block_of(const std::string& name) {
    for (const char* prefix : {"layers.", "h."}) {
        const size_t n = std::strlen(prefix);
        if (name.compare(0, n, prefix) == 0) {
            size_t end = n;
            while (end < name.size() && std::isdigit(static_cast<unsigned char>(name[end]))) ++end;
            if (end > n && end < name.size() && name[end] == '.') return std::stol(name.substr(n, end - n));
        }
    }
    return -1;
}

template <typename F>
int guard(F f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    } catch (...) {
        g_err = "unknown exception";
        return 1;
    }
}

Model* M(void* h) {
    if (!h) throw std::runtime_error("null model handle");
    return static_cast<Model*>(h);
}

mt_segment_cb g_cb = nullptr;
void* g_cb_user = nullptr;

}  // namespace

extern "C" {

const char* mt_last_error(void) { return g_err.c_str(); }

int mt_init(int dev, int dtype) {
    return guard([&] {
        if (dtype != 0 && dtype != 1) throw std::runtime_error("mt_init: dtype must be 0 (fp32) or 1 (bf16)");
        device::init(dev);
        device::set_compute_dtype(dtype == 1 ? DType::BF16 : DType::F32);
    });
}
int mt_set_stream(void* s) {
    return guard([&] { device::set_stream(s); });
}
int mt_sync(void) {
    return guard([&] { device::synchronize(); });
}

int mt_model_create(const char* spec, void** out) {
    return guard([&] {
        if (!out) throw std::runtime_error("null output");
        SpecReader r{parse_spec(spec), {}};
        auto m = std::make_unique<Model>();
        m->family = r.str("family", "llama");
        const unsigned seed = static_cast<unsigned>(r.num("seed", 0));
        const bool ckpt = r.num("ckpt", 0) != 0;
        const bool pack = r.num("pack", 1) != 0;
        if (m->family == "llama") {
            nn::LlamaConfig c;
            c.vocab = r.num("vocab", 4096);
            c.d = r.num("d", 128);
            c.n_layers = r.num("layers", 2);
            c.n_heads = r.num("heads", 4);
            c.n_kv_heads = r.num("kv_heads", 0);
            c.d_ff = r.num("dff", 512);
            c.n_ctx = r.num("nctx", 256);
            c.rope_theta = static_cast<float>(r.real("theta", 10000.0));
            c.tie_embeddings = r.num("tie", 1) != 0;
            c.rope_all_heads = r.num("rope_all", 0) != 0;
            c.qlora = r.num("qlora", 0) != 0;
            c.lora_rank = r.num("rank", 16);
            c.lora_alpha = static_cast<float>(r.real("alpha", 32.0));
            r.finish();
            m->llama = std::make_shared<nn::Llama>(c, seed);
            m->named = m->llama->named_parameters();
            m->loss_chunk = default_loss_chunk(c.vocab);
        } else if (m->family == "gpt2") {
            nn::GPT2Config c;
            c.vocab = r.num("vocab", 50257);
            c.n_ctx = r.num("nctx", 1024);
            c.d = r.num("d", 768);
            c.n_layers = r.num("layers", 12);
            c.n_heads = r.num("heads", 12);
            r.finish();
            m->gpt2 = std::make_shared<nn::GPT2>(c, seed);
            m->named = m->gpt2->named_parameters();
            m->loss_chunk = default_loss_chunk(c.vocab);
        } else if (m->family == "flex") {
            parity::FlexConfig c;
            c.vocab = r.num("vocab", 97);
            c.d = r.num("d", 128);
            c.n_layers = r.num("layers", 2);
            c.n_heads = r.num("heads", 4);
            c.d_ff = r.num("dff", 512);
            c.n_ctx = r.num("nctx", 128);
            c.norm = r.str("norm", "layernorm");
            c.act = r.str("act", "gelu");
            c.pos = r.str("pos", "learned");
            r.finish();
            m->flex = std::make_shared<parity::FlexLM>(c, seed);
            m->named = m->flex->named_parameters();
            m->loss_chunk = default_loss_chunk(c.vocab);
        } else if (m->family == "block") {
            nn::LlamaConfig c;
            c.d = r.num("d", 128);
            c.n_heads = r.num("heads", 4);
            c.n_kv_heads = r.num("kv_heads", 0);
            c.d_ff = r.num("dff", 512);
            c.rope_theta = static_cast<float>(r.real("theta", 10000.0));
            c.rope_all_heads = r.num("rope_all", 1) != 0;
            r.finish();
            m->block = std::make_shared<nn::LlamaBlock>(c, seed);
            m->named = m->block->named_parameters();
        } else {
            throw std::runtime_error("model spec: family must be llama, gpt2, flex or block");
        }
        m->set_ckpt(ckpt);
        // Packed order: block 0, block 1, ..., then everything else.
        long n_blocks = 0;
        for (auto& np : m->named) n_blocks = std::max(n_blocks, block_of(np.first) + 1);
        for (long b = 0; b < n_blocks; ++b) {
            const size_t first = m->params.size();
            for (auto& np : m->named)
                if (block_of(np.first) == b) m->params.push_back(np.second);
            if (m->params.size() > first) m->buckets.emplace_back(first, m->params.size() - 1);
        }
        const size_t first = m->params.size();
        for (auto& np : m->named)
            if (block_of(np.first) < 0) m->params.push_back(np.second);
        if (m->params.size() > first) m->buckets.emplace_back(first, m->params.size() - 1);
        if (pack) {
            m->pack = nn::pack_parameters(m->params);
            m->packed = true;
        }
        *out = m.release();
    });
}

int mt_model_destroy(void* h) {
    return guard([&] { delete static_cast<Model*>(h); });
}
int mt_model_set_checkpoint(void* h, int on) {
    return guard([&] { M(h)->set_ckpt(on != 0); });
}
int mt_model_set_loss_chunk(void* h, int64_t rows) {
    return guard([&] {
        if (rows < 0) throw std::runtime_error("negative chunk size");
        M(h)->loss_chunk = static_cast<size_t>(rows);
    });
}
int mt_model_num_params(void* h, int64_t* n) {
    return guard([&] { *n = static_cast<int64_t>(M(h)->named.size()); });
}
int mt_model_param_info(void* h, int64_t i, char* name, size_t cap, int64_t* rows, int64_t* cols) {
    return guard([&] {
        Model* m = M(h);
        if (i < 0 || static_cast<size_t>(i) >= m->named.size()) throw std::runtime_error("parameter index out of range");
        if (name && cap) std::snprintf(name, cap, "%s", m->named[i].first.c_str());
        if (rows) *rows = static_cast<int64_t>(m->named[i].second->data.rows());
        if (cols) *cols = static_cast<int64_t>(m->named[i].second->data.cols());
    });
}
int mt_model_param_get(void* h, int64_t i, float* out) {
    return guard([&] {
        Model* m = M(h);
        if (i < 0 || static_cast<size_t>(i) >= m->named.size()) throw std::runtime_error("parameter index out of range");
        const Matrix& v = m->named[i].second->data.host();
        std::memcpy(out, v.data(), v.size() * sizeof(float));
    });
}
int mt_model_param_set(void* h, int64_t i, const float* in) {
    return guard([&] {
        Model* m = M(h);
        if (i < 0 || static_cast<size_t>(i) >= m->named.size()) throw std::runtime_error("parameter index out of range");
        Var& p = m->named[i].second;
        Matrix v(p->data.rows(), p->data.cols());
        std::memcpy(v.data(), in, v.size() * sizeof(float));
        p->data = v;
    });
}
int mt_model_grad_get(void* h, int64_t i, float* out, int* has) {
    return guard([&] {
        Model* m = M(h);
        if (i < 0 || static_cast<size_t>(i) >= m->named.size()) throw std::runtime_error("parameter index out of range");
        Var& p = m->named[i].second;
        if (p->grad.empty()) {
            if (has) *has = 0;
            return;
        }
        if (has) *has = 1;
        const Matrix& v = p->grad.host();
        std::memcpy(out, v.data(), v.size() * sizeof(float));
    });
}

// ---- checkpoint files -------------------------------------------------------------------
static nn::AdamW& optimizer(Model* m);
static size_t optimizer_index(Model* m, int64_t i);

int mt_safetensors_copy(const char* in_path, const char* out_path, int64_t* n_loaded, int64_t* n_skipped) {
    return guard([&] {
        std::map<std::string, std::string> skipped;
        const auto tensors = load_safetensors(in_path, &skipped);
        save_safetensors(out_path, tensors);
        if (n_loaded) *n_loaded = static_cast<int64_t>(tensors.size());
        if (n_skipped) *n_skipped = static_cast<int64_t>(skipped.size());
    });
}
int mt_model_save(void* h, const char* weights_path, const char* optimizer_path) {
    return guard([&] {
        Model* m = M(h);
        if (!weights_path) throw std::runtime_error("null path");
        std::map<std::string, Matrix> w;
        for (auto& [name, p] : m->named) w[name] = p->data.host();
        save_safetensors(weights_path, w);
        if (!optimizer_path) return;
        std::map<std::string, Matrix> o;
        nn::AdamW& opt = optimizer(m);
        for (size_t i = 0; i < m->named.size(); ++i) {
            const Var& p = m->named[i].second;
            Matrix mm(p->data.rows(), p->data.cols()), vv(p->data.rows(), p->data.cols());
            opt.export_state(optimizer_index(m, static_cast<int64_t>(i)), mm.data(), vv.data());
            o["m." + m->named[i].first] = std::move(mm);
            o["v." + m->named[i].first] = std::move(vv);
        }
        // the step count as two fp32 halves (each below 2^24, so exact): t = hi * 2^24 + lo
        Matrix t(1, 2);
        const long steps = opt.steps_taken();
        t(0, 0) = static_cast<float>(steps & 0xffffff);
        t(0, 1) = static_cast<float>(steps >> 24);
        o["t"] = std::move(t);
        save_safetensors(optimizer_path, o);
    });
}
int mt_model_load(void* h, const char* weights_path, const char* optimizer_path) {
    return guard([&] {
        Model* m = M(h);
        auto fetch = [](const std::map<std::string, Matrix>& src, const std::string& name, size_t rows,
                        size_t cols) -> const Matrix& {
            auto it = src.find(name);
            if (it == src.end()) throw std::runtime_error("checkpoint has no tensor " + name);
            if (it->second.rows() != rows || it->second.cols() != cols)
                throw std::runtime_error("checkpoint tensor " + name + " is [" + std::to_string(it->second.rows()) + ", " +
                                         std::to_string(it->second.cols()) + "], the model wants [" +
                                         std::to_string(rows) + ", " + std::to_string(cols) + "]");
            return it->second;
        };
        if (weights_path) {
            const auto w = load_safetensors(weights_path);
            // every tensor is checked before the first one is written
            for (auto& [name, p] : m->named) fetch(w, name, p->data.rows(), p->data.cols());
            for (auto& [name, p] : m->named) p->data = fetch(w, name, p->data.rows(), p->data.cols());
        }
        if (optimizer_path) {
            const auto o = load_safetensors(optimizer_path);
            for (auto& [name, p] : m->named) {
                fetch(o, "m." + name, p->data.rows(), p->data.cols());
                fetch(o, "v." + name, p->data.rows(), p->data.cols());
            }
            const Matrix& t = fetch(o, "t", 1, 2);
            nn::AdamW& opt = optimizer(m);
            for (size_t i = 0; i < m->named.size(); ++i) {
                const Var& p = m->named[i].second;
                const std::string& name = m->named[i].first;
                opt.import_state(optimizer_index(m, static_cast<int64_t>(i)),
                                 fetch(o, "m." + name, p->data.rows(), p->data.cols()).data(),
                                 fetch(o, "v." + name, p->data.rows(), p->data.cols()).data());
            }
            opt.set_steps_taken(static_cast<long>(t(0, 0)) + (static_cast<long>(t(0, 1)) << 24));
        }
    });
}

int mt_model_load_base(void* h, const char* weights_path) {
    return guard([&] {
        Model* m = M(h);
        if (!weights_path) throw std::runtime_error("null path");
        if (!m->llama) throw std::runtime_error("load_base: only the llama family has a QLoRA mode");
        m->llama->load_frozen_base(load_safetensors(weights_path));
    });
}

int mt_model_save_merged(void* h, const char* weights_path) {
    return guard([&] {
        Model* m = M(h);
        if (!weights_path) throw std::runtime_error("null path");
        if (!m->llama) throw std::runtime_error("save_merged: only the llama family has a QLoRA mode");
        save_safetensors(weights_path, m->llama->merged_state());
    });
}

int mt_gguf_export_llama(const char* weights_path, const char* gguf_path, const char* spec, const char* tokens_path,
                         int64_t* n_unmapped) {
    return guard([&] {
        if (!weights_path || !gguf_path) throw std::runtime_error("null path");
        SpecReader r{parse_spec(spec), {}};
        gguf::LlamaExportConfig c;
        c.name = r.str("name", c.name);
        c.architecture = r.str("arch", c.architecture);
        c.context_length = static_cast<uint32_t>(r.num("ctx", c.context_length));
        c.embedding_length = static_cast<uint32_t>(r.num("d", 0));
        c.block_count = static_cast<uint32_t>(r.num("layers", 0));
        c.feed_forward_length = static_cast<uint32_t>(r.num("dff", 0));
        c.head_count = static_cast<uint32_t>(r.num("heads", 0));
        c.head_count_kv = static_cast<uint32_t>(r.num("kv_heads", 0));
        c.vocab_size = static_cast<uint32_t>(r.num("vocab", 0));
        c.rms_eps = static_cast<float>(r.real("eps", c.rms_eps));
        c.rope_freq_base = static_cast<float>(r.real("theta", c.rope_freq_base));
        c.weights_in_out = r.num("in_out", 0) != 0;
        r.finish();
        if (tokens_path) {  // one token per line
            std::ifstream tf(tokens_path);
            if (!tf) throw std::runtime_error(std::string("cannot open ") + tokens_path);
            std::string line;
            while (std::getline(tf, line)) c.tokens.push_back(line);
        }
        std::vector<std::string> unmapped;
        gguf::export_gguf_llama(gguf_path, load_safetensors(weights_path), c, &unmapped);
        if (n_unmapped) *n_unmapped = static_cast<int64_t>(unmapped.size());
    });
}
int mt_model_export_gguf(void* h, const char* gguf_path, const char* name, int64_t context_length) {
    return guard([&] {
        Model* m = M(h);
        if (!gguf_path) throw std::runtime_error("null path");
        if (!m->llama) throw std::runtime_error("export_gguf: only the llama family maps onto the GGUF llama layout");
        const nn::LlamaConfig& lc = m->llama->cfg;
        gguf::LlamaExportConfig c;
        if (name) c.name = name;
        c.context_length = static_cast<uint32_t>(context_length);
        c.embedding_length = static_cast<uint32_t>(lc.d);
        c.block_count = static_cast<uint32_t>(lc.n_layers);
        c.feed_forward_length = static_cast<uint32_t>(lc.d_ff);
        c.head_count = static_cast<uint32_t>(lc.n_heads);
        c.head_count_kv = static_cast<uint32_t>(lc.n_kv_heads);
        c.vocab_size = static_cast<uint32_t>(lc.vocab);
        c.rms_eps = 1e-5f;  // what ops::rmsnorm computes with
        c.rope_freq_base = lc.rope_theta;
        c.weights_in_out = true;  // Linear stores [in, out]
        gguf::export_gguf_llama(gguf_path, m->llama->merged_state(), c, nullptr);
    });
}

int mt_model_step(void* h, const int32_t* ids_h, const int32_t* targets_h, int64_t n, int64_t seq_len,
                  float loss_scale, int do_backward, float* loss_h) {
    return guard([&] {
        Model* m = M(h);
        if (n < 0 || seq_len < 0) throw std::runtime_error("negative size");
        std::vector<int> ids(ids_h, ids_h + n), targets(targets_h, targets_h + n);
        device::step_begin();
        float loss_value = 0.0f;
        if (do_backward) {
            if (!m->accumulate) zero_grad(m->params);
            const size_t live0 = live_variables();
            Var loss = m->loss(ids, targets, static_cast<size_t>(seq_len));
            m->live_after_fwd = static_cast<int64_t>(live_variables() - live0);
            Var root = loss_scale == 1.0f ? loss : ops::scale(loss, loss_scale);
            backward(root);
            loss_value = loss->data.host()(0, 0);
        } else {
            NoGrad ng;
            Var loss = m->loss(ids, targets, static_cast<size_t>(seq_len));
            loss_value = loss->data.host()(0, 0);
        }
        device::step_end();
        if (loss_h) *loss_h = loss_value;
        // The loss readback has synchronised the stream: a kernel whose bounded wait gave up has
        // left the step's results incomplete, which must not pass for a finished step.
        int status = 0;
        device::check(pk_kernel_status(&status, 1), "pk_kernel_status");
        if (status != 0)
            throw std::runtime_error("mt_model_step: a tensor-core kernel abandoned a bounded wait (status " +
                                     std::to_string(status) + ", PK_ERR_TIMEOUT = 4); the results of this step are incomplete");
    });
}

// ---- single block (family "block") ----------------------------------------------------
int mt_block_set_input(void* h, const float* x_h, const float* dy_h, int64_t rows, int64_t seq_len) {
    return guard([&] {
        Model* m = M(h);
        if (!m->block) throw std::runtime_error("mt_block_set_input: the model is not a block");
        if (rows <= 0 || seq_len <= 0 || rows % seq_len != 0) throw std::runtime_error("rows must be a positive multiple of seq_len");
        const size_t R = static_cast<size_t>(rows), d = m->block->ln1_w->data.cols();
        Matrix x(R, d), dy(R, d);
        std::memcpy(x.data(), x_h, R * d * sizeof(float));
        std::memcpy(dy.data(), dy_h, R * d * sizeof(float));
        m->by.reset();
        m->bx = make_var(Tensor::from_host(x, device::compute_dtype(), device::Pool::Persistent), true);
        m->bdy = Tensor::from_host(dy, device::compute_dtype(), device::Pool::Persistent);
        m->bpos.resize(R);
        for (size_t i = 0; i < R; ++i) m->bpos[i] = static_cast<int>(i % static_cast<size_t>(seq_len));
        m->bseq = static_cast<size_t>(seq_len);
    });
}
int mt_block_forward(void* h) {
    return guard([&] {
        Model* m = M(h);
        if (!m->block || !m->bx) throw std::runtime_error("mt_block_forward: no block input set");
        device::step_begin();
        zero_grad(m->params);
        m->bx->grad = Value();
        auto blk = m->block;
        auto pos = m->bpos;
        const size_t seq = m->bseq;
        const size_t live0 = live_variables();
        m->by = m->block_ckpt ? checkpoint([blk, pos, seq](const Var& in) { return blk->forward(in, pos, seq); }, m->bx)
                              : blk->forward(m->bx, pos, seq);
        m->live_after_fwd = static_cast<int64_t>(live_variables() - live0);
    });
}
int mt_block_backward(void* h) {
    return guard([&] {
        Model* m = M(h);
        if (!m->by) throw std::runtime_error("mt_block_backward: no pending forward");
        Var y = m->by;
        m->by.reset();
        backward_from(y, m->bdy);
        y.reset();
        device::step_end();
    });
}
int mt_block_output(void* h, float* y_h) {
    return guard([&] {
        Model* m = M(h);
        if (!m->by) throw std::runtime_error("mt_block_output: no pending forward");
        const Matrix& v = m->by->data.host();
        std::memcpy(y_h, v.data(), v.size() * sizeof(float));
    });
}
int mt_block_input_grad(void* h, float* dx_h) {
    return guard([&] {
        Model* m = M(h);
        if (!m->bx || m->bx->grad.empty()) throw std::runtime_error("mt_block_input_grad: no gradient yet");
        const Matrix& v = m->bx->grad.host();
        std::memcpy(dx_h, v.data(), v.size() * sizeof(float));
    });
}

int mt_model_live_after_forward(void* h, int64_t* n) {
    return guard([&] { *n = M(h)->live_after_fwd; });
}

int mt_model_set_adamw(void* h, float lr, float b1, float b2, float eps, float wd) {
    return guard([&] {
        Model* m = M(h);
        if (m->opt) throw std::runtime_error("optimizer already created; set hyper-parameters before the first step");
        m->lr = lr; m->b1 = b1; m->b2 = b2; m->eps = eps; m->wd = wd;
    });
}
static nn::AdamW& optimizer(Model* m) {
    if (!m->opt) m->opt = std::make_unique<nn::AdamW>(m->params, m->lr, m->b1, m->b2, m->eps, m->wd);
    return *m->opt;
}
// The optimizer is built over the packed order; the state entries use the registration
// order of mt_model_param_info like every other per-parameter entry.
static size_t optimizer_index(Model* m, int64_t i) {
    if (i < 0 || static_cast<size_t>(i) >= m->named.size()) throw std::runtime_error("parameter index out of range");
    const Var& p = m->named[i].second;
    for (size_t k = 0; k < m->params.size(); ++k)
        if (m->params[k] == p) return k;
    throw std::runtime_error("parameter is not trainable");
}
int mt_model_optimizer_step(void* h) {
    return guard([&] { optimizer(M(h)).step(); });
}
int mt_model_set_accumulate(void* h, int on) {
    return guard([&] { M(h)->accumulate = on != 0; });
}
int mt_model_zero_grad(void* h) {
    return guard([&] { zero_grad(M(h)->params); });
}
int mt_model_optimizer_steps_get(void* h, int64_t* t) {
    return guard([&] { *t = M(h)->opt ? static_cast<int64_t>(M(h)->opt->steps_taken()) : 0; });
}
int mt_model_optimizer_steps_set(void* h, int64_t t) {
    return guard([&] {
        if (t < 0) throw std::runtime_error("negative step count");
        optimizer(M(h)).set_steps_taken(static_cast<long>(t));
    });
}
int mt_model_optimizer_state_get(void* h, int64_t i, float* m_h, float* v_h) {
    return guard([&] {
        Model* m = M(h);
        optimizer(m).export_state(optimizer_index(m, i), m_h, v_h);
    });
}
int mt_model_optimizer_state_set(void* h, int64_t i, const float* m_h, const float* v_h) {
    return guard([&] {
        Model* m = M(h);
        optimizer(m).import_state(optimizer_index(m, i), m_h, v_h);
    });
}
int mt_model_clip_grad_norm(void* h, float max_norm, float* norm) {
    return guard([&] {
        const float n = ops::clip_grad_norm(M(h)->params, max_norm);
        if (norm) *norm = n;
    });
}

int mt_clip_grad_norm_arrays(int n, const int64_t* rows_h, const int64_t* cols_h, float* const* grads_h, float max_norm,
                             float* norm_h) {
    return guard([&] {
        if (n < 0 || (n > 0 && (!rows_h || !cols_h || !grads_h))) throw std::runtime_error("bad argument");
        std::vector<Var> vars;
        for (int i = 0; i < n; ++i) {
            const size_t r = static_cast<size_t>(rows_h[i]), c = static_cast<size_t>(cols_h[i]);
            Var v = make_var(Matrix(r, c), true);
            Matrix g(r, c);
            std::memcpy(g.data(), grads_h[i], r * c * sizeof(float));
            v->accumulate(g);
            vars.push_back(v);
        }
        const float total = ops::clip_grad_norm(vars, max_norm);
        for (int i = 0; i < n; ++i) {
            const Matrix& g = vars[i]->grad.host();
            std::memcpy(grads_h[i], g.data(), g.rows() * g.cols() * sizeof(float));
        }
        if (norm_h) *norm_h = total;
    });
}

int mt_model_num_buckets(void* h, int64_t* n) {
    return guard([&] { *n = static_cast<int64_t>(M(h)->buckets.size()); });
}
int mt_model_bucket(void* h, int64_t i, void** ptr, int64_t* count) {
    return guard([&] {
        Model* m = M(h);
        if (!m->packed) throw std::runtime_error("gradient buckets need a packed model (pack=1)");
        if (i < 0 || static_cast<size_t>(i) >= m->buckets.size()) throw std::runtime_error("bucket index out of range");
        const size_t first = m->buckets[i].first, last = m->buckets[i].second;
        const size_t begin = m->pack.offset[first];
        const size_t end = last + 1 < m->pack.offset.size() ? m->pack.offset[last + 1] : m->pack.total;
        *ptr = m->pack.grad.f32() + begin;
        *count = static_cast<int64_t>(end - begin);
    });
}

// ---- data parallelism over the collective group of libpk -----------------------------------
namespace {
void dp_attach(Model* m, void* comm) {
    if (!m->packed) {
        pk_comm_destroy(comm);
        throw std::runtime_error("data parallelism needs a packed model (pack=1)");
    }
    std::vector<std::pair<float*, int64_t>> buckets;
    for (const auto& b : m->buckets) {
        const size_t begin = m->pack.offset[b.first];
        const size_t end = b.second + 1 < m->pack.offset.size() ? m->pack.offset[b.second + 1] : m->pack.total;
        buckets.emplace_back(m->pack.grad.f32() + begin, static_cast<int64_t>(end - begin));
    }
    m->exchange.reset();
    m->exchange = std::make_unique<dp::GradientExchange>(
        comm, std::move(buckets), std::make_pair(m->pack.grad.f32(), static_cast<int64_t>(m->pack.total)));
    m->exchange->attach();
}
dp::GradientExchange& DPX(void* h) {
    Model* m = M(h);
    if (!m->exchange) throw std::runtime_error("the model has no gradient exchange (call mt_dp_init first)");
    return *m->exchange;
}
}  // namespace

int mt_dp_unique_id(void* id_h, size_t cap) {
    return guard([&] { device::check(pk_comm_unique_id(id_h, cap), "pk_comm_unique_id"); });
}
int mt_dp_init(void* h, const void* id_h, int rank, int world, int max_ctas) {
    return guard([&] {
        Model* m = M(h);
        void* comm = nullptr;
        device::check(pk_comm_init(id_h, rank, world, max_ctas, &comm), "pk_comm_init");
        dp_attach(m, comm);
    });
}
int mt_dp_enable(void* h, int on) {
    return guard([&] { DPX(h).set_enabled(on != 0); });
}
int mt_dp_finish(void* h) {
    return guard([&] { DPX(h).finish(); });
}
int mt_dp_wait_host(void* h) {
    return guard([&] { DPX(h).wait_host(); });
}
int mt_dp_set_timeout(void* h, double seconds) {
    return guard([&] { DPX(h).set_timeout(seconds); });
}
int mt_dp_set_flat_threshold(void* h, int64_t bytes) {
    return guard([&] { DPX(h).set_flat_threshold(bytes); });
}
int mt_dp_stats(void* h, int64_t* launches_last_step_h, int* single_collective_h) {
    return guard([&] {
        if (launches_last_step_h) *launches_last_step_h = DPX(h).launches_last_step();
        if (single_collective_h) *single_collective_h = DPX(h).single_collective() ? 1 : 0;
    });
}
int mt_dp_destroy(void* h) {
    return guard([&] { M(h)->exchange.reset(); });
}

int mt_set_segment_hook(mt_segment_cb cb, void* user) {
    return guard([&] {
        g_cb = cb;
        g_cb_user = user;
        if (cb) autograd::set_segment_hook([](int k) { if (g_cb) g_cb(k, g_cb_user); });
        else autograd::set_segment_hook(nullptr);
    });
}

int mt_mem_stats(uint64_t* out) {
    return guard([&] {
        const device::MemStats s = device::mem_stats();
        out[0] = s.in_use[0]; out[1] = s.peak[0]; out[2] = s.in_use[1]; out[3] = s.peak[1];
        out[4] = s.reserved; out[5] = s.driver_allocs;
    });
}
int mt_mem_peak_blocks(uint64_t* sizes_h, uint64_t* counts_h, int cap, int* n_h) {
    return guard([&] {
        const auto blocks = device::peak_activation_blocks();
        if (n_h) *n_h = static_cast<int>(blocks.size());
        for (size_t i = 0; i < blocks.size() && static_cast<int>(i) < cap; ++i) {
            if (sizes_h) sizes_h[i] = blocks[i].first;
            if (counts_h) counts_h[i] = blocks[i].second;
        }
    });
}
int mt_reset_peak(void) {
    return guard([&] { device::reset_peak(); });
}
int mt_empty_cache(void) {
    return guard([&] { device::empty_cache(); });
}
int mt_live_variables(int64_t* n) {
    return guard([&] { *n = static_cast<int64_t>(live_variables()); });
}

}  // extern "C"
