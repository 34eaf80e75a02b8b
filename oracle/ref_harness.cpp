// TEST INFRASTRUCTURE -- not part of the shipped library.
//
// Command-line harness that drives the UNMODIFIED reference implementation
// (paperkiln / microtorch, CPU fp32) so that its results can be written out as
// golden vectors and its training step can be timed as the CPU baseline.
// This file is compiled together with the reference's own sources (see the
// Makefile beside it); nothing from the reference is copied here -- models
// that the reference does not ship (grouped-query Llama, a Q8_0 QLoRA Llama,
// a checkpoint-wrapped flex LM) are composed from the reference's own ops in
// the same way its tools/parity_model.hpp composes FlexLM.
//
// Sub-commands
//   step   one or more train steps of a model family; dumps params, loss,
//          grads and post-AdamW params as .npy files
//   ops    per-op goldens at awkward shapes (R=67, C=133; tests/test_cuda_ops.cpp:63)
//   quant  Q8_0 (block 32, fp16 scale) quantize / dequantize goldens
//   bench  timed train steps, prints one JSON line with tokens/s
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <random>
#include <string>
#include <vector>

#include "microtorch/llama.hpp"
#include "microtorch/nn.hpp"
#include "microtorch/ops.hpp"
#include "microtorch/quant.hpp"
#include "parity_model.hpp"

using namespace microtorch;

namespace {

// ---------------------------------------------------------------- npy writer
void write_npy_raw(const std::string& path, const void* data, size_t nbytes, const char* descr,
                   const std::vector<size_t>& shape) {
    std::string hdr = "{'descr': '" + std::string(descr) + "', 'fortran_order': False, 'shape': (";
    for (size_t i = 0; i < shape.size(); ++i) hdr += std::to_string(shape[i]) + ",";
    hdr += "), }";
    size_t total = 10 + hdr.size() + 1;
    size_t pad = (64 - total % 64) % 64;
    hdr += std::string(pad, ' ');
    hdr += "\n";
    std::ofstream f(path, std::ios::binary);
    const char magic[] = {'\x93', 'N', 'U', 'M', 'P', 'Y', 1, 0};
    f.write(magic, 8);
    uint16_t hl = static_cast<uint16_t>(hdr.size());
    f.write(reinterpret_cast<const char*>(&hl), 2);
    f.write(hdr.data(), hdr.size());
    f.write(reinterpret_cast<const char*>(data), nbytes);
}

void write_matrix(const std::string& dir, const std::string& name, const Matrix& m) {
    std::vector<float> buf(m.rows() * m.cols());
    for (size_t i = 0; i < m.rows(); ++i)
        for (size_t j = 0; j < m.cols(); ++j) buf[i * m.cols() + j] = m(i, j);
    write_npy_raw(dir + "/" + name + ".npy", buf.data(), buf.size() * 4, "<f4", {m.rows(), m.cols()});
}

void write_ints(const std::string& dir, const std::string& name, const std::vector<int>& v) {
    std::vector<int32_t> buf(v.begin(), v.end());
    write_npy_raw(dir + "/" + name + ".npy", buf.data(), buf.size() * 4, "<i4", {buf.size()});
}

Matrix read_matrix_bin(const std::string& path, size_t rows, size_t cols) {
    // raw little-endian fp32, row-major (written by the test driver)
    std::ifstream f(path, std::ios::binary);
    if (!f) {
        std::fprintf(stderr, "cannot open %s\n", path.c_str());
        std::exit(2);
    }
    std::vector<float> buf(rows * cols);
    f.read(reinterpret_cast<char*>(buf.data()), buf.size() * 4);
    Matrix m(rows, cols);
    for (size_t i = 0; i < rows; ++i)
        for (size_t j = 0; j < cols; ++j) m(i, j) = buf[i * cols + j];
    return m;
}

// ---------------------------------------------------------------- arguments
struct Args {
    std::map<std::string, std::string> kv;
    std::string get(const std::string& k, const std::string& d) const {
        auto it = kv.find(k);
        return it == kv.end() ? d : it->second;
    }
    long geti(const std::string& k, long d) const {
        auto it = kv.find(k);
        return it == kv.end() ? d : std::stol(it->second);
    }
    double getf(const std::string& k, double d) const {
        auto it = kv.find(k);
        return it == kv.end() ? d : std::stod(it->second);
    }
};

Args parse(int argc, char** argv, int first) {
    Args a;
    for (int i = first; i + 1 < argc; i += 2) {
        std::string k = argv[i];
        if (k.rfind("--", 0) == 0) k = k.substr(2);
        a.kv[k] = argv[i + 1];
    }
    return a;
}

// Token stream used throughout: the reference tests' own pattern
// (tests/test_checkpointing.cpp:28-33): mt19937(seed), id = rng() % vocab.
std::vector<int> random_ids(size_t n, unsigned seed, int vocab) {
    std::mt19937 rng(seed);
    std::vector<int> ids(n);
    for (auto& t : ids) t = static_cast<int>(rng() % vocab);
    return ids;
}

Matrix filled_uniform(size_t r, size_t c, unsigned seed, float lo, float hi) {
    Matrix m(r, c);
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> u(lo, hi);
    for (size_t i = 0; i < r; ++i)
        for (size_t j = 0; j < c; ++j) m(i, j) = u(rng);
    return m;
}

Matrix filled_normal(size_t r, size_t c, unsigned seed, float std) {
    Matrix m(r, c);
    std::mt19937 rng(seed);
    std::normal_distribution<float> d(0.0f, std);
    for (size_t i = 0; i < r; ++i)
        for (size_t j = 0; j < c; ++j) m(i, j) = d(rng);
    return m;
}

// ---------------------------------------------------------------- Q8_0 helper
// Reference quantizer (src/quant.cpp:11-37) at block 32, then each fp32 scale
// is rounded to IEEE binary16 (round-to-nearest-even). Dequantisation stays the
// reference's single fp32 multiply (src/quant.cpp:39-48).
QuantizedTensor quantize_q8_0(const Matrix& W) {
    QuantizedTensor t = quantize_int8(W, 32);
    // Re-quantize against the rounded scale so that q is consistent with the
    // scale that is actually stored.
    const size_t bpr = (t.cols + 31) / 32;
    for (size_t i = 0; i < t.rows; ++i)
        for (size_t b = 0; b < bpr; ++b) {
            float s = t.scales[i * bpr + b];
            float s16 = static_cast<float>(static_cast<_Float16>(s));
            if (s16 == 0.0f) s16 = static_cast<float>(static_cast<_Float16>(6.103515625e-05f));
            t.scales[i * bpr + b] = s16;
            const size_t j0 = b * 32, j1 = std::min(j0 + 32, t.cols);
            for (size_t j = j0; j < j1; ++j) {
                const float v = W(i, j) / s16;
                t.q[i * t.cols + j] =
                    static_cast<int8_t>(std::lround(std::max(-127.0f, std::min(127.0f, v))));
            }
        }
    return t;
}

// ---------------------------------------------------------------- harness models
// Frozen-or-trainable linear layer with an optional Q8_0 base and an optional
// LoRA side path, composed exactly like nn::QLoRALinear::forward
// (src/quant.cpp:114-119) but with the Q8_0 (fp16-scale) base weight.
struct HLinear : nn::Module {
    Var W;            // trainable dense weight (mode 0)
    Matrix Wdq;       // frozen dequantized base (mode 1, 2)
    Var A, B;         // LoRA (mode 2)
    float scaling = 0.0f;
    int mode = 0;     // 0 dense trainable, 1 frozen q8, 2 frozen q8 + lora
    HLinear(size_t in, size_t out, unsigned seed, int mode_, size_t rank, float alpha,
            unsigned lora_seed)
        : mode(mode_) {
        Matrix W0 = filled_normal(in, out, seed * 7919u + 1u, 0.02f);  // == nn::Linear init
        if (mode == 0) {
            W = reg("weight", W0);
        } else {
            Wdq = dequantize(quantize_q8_0(W0));
            if (mode == 2) {
                A = reg("lora_A", filled_normal(in, rank, lora_seed * 31u + 5u, 0.02f));
                B = reg("lora_B", filled_normal(rank, out, lora_seed * 31u + 6u, 0.01f));
                scaling = alpha / static_cast<float>(rank);
            }
        }
    }
    Var forward(const Var& x) const {
        if (mode == 0) return ops::matmul(x, W);
        Var base = ops::matmul(x, make_var(Wdq));
        if (mode == 1) return base;
        Var delta = ops::matmul(ops::matmul(x, A), B);
        return ops::add(base, ops::scale(delta, scaling));
    }
};

struct GQAConfig {
    size_t vocab = 256, d = 64, n_layers = 2, n_heads = 4, n_kv_heads = 2, d_ff = 128;
    float rope_theta = 10000.0f;
    bool tie = true;
    bool qlora = false;  // frozen Q8_0 base + LoRA on q,v
    size_t rank = 16;
    float alpha = 32.0f;
};

// Llama block with grouped-query attention and all-heads RoPE: per head the
// reference's apply_rope is applied to a 3*dk wide concat, so d == head_dim
// inside the op and the whole head is rotated.
struct GQABlock : nn::Module {
    Var ln1_w, ln2_w;
    std::shared_ptr<HLinear> q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj;
    size_t H, Hkv, dk;
    float theta;
    bool frozen_norms;
    Matrix ln1_m, ln2_m;
    GQABlock(const GQAConfig& c, unsigned seed)
        : H(c.n_heads), Hkv(c.n_kv_heads), dk(c.d / c.n_heads), theta(c.rope_theta),
          frozen_norms(c.qlora) {
        if (frozen_norms) {
            ln1_m = Matrix(1, c.d, 1.0f);
            ln2_m = Matrix(1, c.d, 1.0f);
        } else {
            ln1_w = reg("input_layernorm.weight", Matrix(1, c.d, 1.0f));
            ln2_w = reg("post_attention_layernorm.weight", Matrix(1, c.d, 1.0f));
        }
        const int base = c.qlora ? 1 : 0;
        const int lora = c.qlora ? 2 : 0;
        q_proj = mod<HLinear>("self_attn.q_proj", c.d, H * dk, seed + 1, lora, c.rank, c.alpha, seed + 1);
        k_proj = mod<HLinear>("self_attn.k_proj", c.d, Hkv * dk, seed + 2, base, c.rank, c.alpha, seed + 2);
        v_proj = mod<HLinear>("self_attn.v_proj", c.d, Hkv * dk, seed + 3, lora, c.rank, c.alpha, seed + 3);
        o_proj = mod<HLinear>("self_attn.o_proj", H * dk, c.d, seed + 4, base, c.rank, c.alpha, seed + 4);
        gate_proj = mod<HLinear>("mlp.gate_proj", c.d, c.d_ff, seed + 5, base, c.rank, c.alpha, seed + 5);
        up_proj = mod<HLinear>("mlp.up_proj", c.d, c.d_ff, seed + 6, base, c.rank, c.alpha, seed + 6);
        down_proj = mod<HLinear>("mlp.down_proj", c.d_ff, c.d, seed + 7, base, c.rank, c.alpha, seed + 7);
    }
    Var forward(const Var& x, const std::vector<int>& pos, size_t seq_len) const {
        Var w1 = frozen_norms ? make_var(ln1_m) : ln1_w;
        Var w2 = frozen_norms ? make_var(ln2_m) : ln2_w;
        Var h = ops::rmsnorm(x, w1);
        Var q = q_proj->forward(h), k = k_proj->forward(h), v = v_proj->forward(h);
        const float sc = 1.0f / std::sqrt(static_cast<float>(dk));
        const size_t group = H / Hkv;
        std::vector<Var> heads;
        for (size_t hh = 0; hh < H; ++hh) {
            const size_t g = hh / group;
            Var qh = ops::slice_cols(q, hh * dk, (hh + 1) * dk);
            Var kh = ops::slice_cols(k, g * dk, (g + 1) * dk);
            Var vh = ops::slice_cols(v, g * dk, (g + 1) * dk);
            Var r = ops::apply_rope(ops::concat_cols({qh, kh, vh}), pos, theta, dk);
            qh = ops::slice_cols(r, 0, dk);
            kh = ops::slice_cols(r, dk, 2 * dk);
            heads.push_back(ops::fused_attention(qh, kh, vh, sc, seq_len, true));
        }
        Var x1 = ops::add(x, o_proj->forward(ops::concat_cols(heads)));
        Var h2 = ops::rmsnorm(x1, w2);
        Var ffn = down_proj->forward(
            ops::mul(ops::silu(gate_proj->forward(h2)), up_proj->forward(h2)));
        return ops::add(x1, ffn);
    }
};

struct GQALlama : nn::Module {
    GQAConfig cfg;
    bool checkpoint_blocks = false;
    Var embed;        // trainable unless qlora
    Matrix embed_m;   // frozen copy (qlora)
    Var norm_w;
    Matrix norm_m;
    std::vector<std::shared_ptr<GQABlock>> blocks;
    GQALlama(const GQAConfig& c, unsigned seed) : cfg(c) {
        Matrix E = filled_normal(c.vocab, c.d, (seed + 11) * 104729u + 3u, 0.02f);  // == nn::Embedding
        if (c.qlora) {
            embed_m = E;
            norm_m = Matrix(1, c.d, 1.0f);
        } else {
            embed = reg("embed_tokens.weight", E);
        }
        for (size_t i = 0; i < c.n_layers; ++i)
            blocks.push_back(mod<GQABlock>("layers." + std::to_string(i), c,
                                           seed + 100 * static_cast<unsigned>(i + 1)));
        if (!c.qlora) norm_w = reg("norm.weight", Matrix(1, c.d, 1.0f));
    }
    Var forward(const std::vector<int>& ids, size_t seq_len) const {
        const size_t sl = seq_len == 0 ? ids.size() : seq_len;
        std::vector<int> pos(ids.size());
        for (size_t i = 0; i < pos.size(); ++i) pos[i] = static_cast<int>(i % sl);
        Var table = cfg.qlora ? make_var(embed_m) : embed;
        Var h = ops::embedding(table, ids);
        // With every base weight frozen the embedding output carries no
        // requires_grad, and checkpoint() still forces the segment output to
        // require grad (src/autograd.cpp:76-79), so LoRA grads flow.
        for (const auto& b : blocks) {
            h = checkpoint_blocks && grad_enabled()
                    ? checkpoint([b, pos, seq_len](const Var& in) { return b->forward(in, pos, seq_len); }, h)
                    : b->forward(h, pos, seq_len);
        }
        h = ops::rmsnorm(h, cfg.qlora ? make_var(norm_m) : norm_w);
        return ops::matmul(h, ops::transpose(table));
    }
};

// Flex LM with the per-block checkpoint wrapper the reference's GPT-2 uses
// (src/nn.cpp:249-253) around parity::FlexBlock.
struct CkptFlexLM {
    parity::FlexLM lm;
    bool checkpoint_blocks = false;
    CkptFlexLM(const parity::FlexConfig& c, unsigned seed) : lm(c, seed) {}
    std::vector<Var> parameters() const { return lm.parameters(); }
    std::vector<std::pair<std::string, Var>> named_parameters() const { return lm.named_parameters(); }
    Var forward(const std::vector<int>& ids, size_t seq_len) const {
        const size_t sl = seq_len == 0 ? ids.size() : seq_len;
        std::vector<int> pos(ids.size());
        for (size_t i = 0; i < pos.size(); ++i) pos[i] = static_cast<int>(i % sl);
        Var h;
        if (lm.wpe) {
            h = ops::add(lm.wte->forward(ids), lm.wpe->forward(pos));
        } else {
            Matrix pe(ids.size(), lm.cfg.d);
            for (size_t r = 0; r < ids.size(); ++r)
                for (size_t j = 0; j < lm.cfg.d; ++j) pe(r, j) = lm.sin_table(pos[r], j);
            h = ops::add(lm.wte->forward(ids), make_var(std::move(pe), false));
        }
        for (auto& b : lm.blocks) {
            h = checkpoint_blocks && grad_enabled()
                    ? checkpoint([b, seq_len](const Var& in) { return b->forward(in, seq_len); }, h)
                    : b->forward(h, seq_len);
        }
        Var n = lm.ln_f_ln ? lm.ln_f_ln->forward(h) : ops::rmsnorm(h, lm.ln_f_w);
        return lm.head->forward(n);
    }
};

// Frozen tensors of the QLoRA harness (dequantized Q8_0 bases, embedding): written next
// to the parameters so that a checker can rebuild the model without the C++ generator.
template <class Model>
void dump_frozen(const Model&, const std::string&) {}
void dump_frozen(const GQALlama& m, const std::string& out) {
    if (!m.cfg.qlora) return;
    write_matrix(out, "frozen.embed_tokens.weight", m.embed_m);
    for (size_t i = 0; i < m.blocks.size(); ++i) {
        const std::string pre = "frozen.layers." + std::to_string(i) + ".";
        const GQABlock& b = *m.blocks[i];
        write_matrix(out, pre + "self_attn.q_proj.weight", b.q_proj->Wdq);
        write_matrix(out, pre + "self_attn.k_proj.weight", b.k_proj->Wdq);
        write_matrix(out, pre + "self_attn.v_proj.weight", b.v_proj->Wdq);
        write_matrix(out, pre + "self_attn.o_proj.weight", b.o_proj->Wdq);
        write_matrix(out, pre + "mlp.gate_proj.weight", b.gate_proj->Wdq);
        write_matrix(out, pre + "mlp.up_proj.weight", b.up_proj->Wdq);
        write_matrix(out, pre + "mlp.down_proj.weight", b.down_proj->Wdq);
    }
}

// ---------------------------------------------------------------- step driver
struct StepResult {
    double fwd_s = 0, bwd_s = 0, opt_s = 0;
    float loss = 0;
    size_t live = 0;
};

template <class Model>
StepResult run_steps(Model& model, const Args& a, const std::string& out) {
    const int vocab = static_cast<int>(a.geti("vocab", 97));
    const size_t B = a.geti("batch", 1), S = a.geti("seq", 16);
    const unsigned data_seed = static_cast<unsigned>(a.geti("data-seed", 0));
    const int steps = static_cast<int>(a.geti("steps", 1));
    const bool do_opt = a.geti("adamw", 1) != 0;
    const float clip = static_cast<float>(a.getf("clip", 0.0));
    const size_t seq_len = a.geti("stack", 1) ? S : 0;

    auto named = model.named_parameters();
    std::vector<Var> params;
    for (auto& [n, p] : named) params.push_back(p);

    // Optional parameter override from raw fp32 files (name.bin) so that the
    // harness and the library under test start from the same bits.
    const std::string pin = a.get("params-in", "");
    if (!pin.empty()) {
        for (auto& [n, p] : named) p->data = read_matrix_bin(pin + "/" + n + ".bin", p->data.rows(), p->data.cols());
    }
    if (!out.empty()) {
        std::ofstream names(out + "/names.txt");
        for (auto& [n, p] : named) {
            names << n << " " << p->data.rows() << " " << p->data.cols() << "\n";
            write_matrix(out, "param." + n, p->data);
        }
        dump_frozen(model, out);
    }

    nn::AdamW opt(params, static_cast<float>(a.getf("lr", 1e-3)));
    auto ids = random_ids(B * S + 1, data_seed, vocab);
    std::vector<int> x(ids.begin(), ids.end() - 1), y(ids.begin() + 1, ids.end());
    if (!out.empty()) {
        write_ints(out, "ids", x);
        write_ints(out, "targets", y);
    }

    StepResult r;
    std::vector<float> losses;
    for (int s = 0; s < steps; ++s) {
        zero_grad(params);
        const size_t live0 = live_variables();
        auto t0 = std::chrono::steady_clock::now();
        Var logits = model.forward(x, seq_len);
        Var loss = ops::cross_entropy(logits, y);
        r.live = live_variables() - live0;
        auto t1 = std::chrono::steady_clock::now();
        backward(loss);
        auto t2 = std::chrono::steady_clock::now();
        r.loss = loss->data(0, 0);
        losses.push_back(r.loss);
        if (!out.empty() && s == 0) {
            for (auto& [n, p] : named)
                if (p->grad.rows() != 0) write_matrix(out, "grad." + n, p->grad);
        }
        float gnorm = 0.0f;
        if (clip > 0.0f) gnorm = ops::clip_grad_norm(params, clip);
        (void)gnorm;
        auto t3 = std::chrono::steady_clock::now();
        if (do_opt) opt.step();
        auto t4 = std::chrono::steady_clock::now();
        if (s >= static_cast<int>(a.geti("warmup", 0))) {  // warm-up steps run but are not timed
            r.fwd_s += std::chrono::duration<double>(t1 - t0).count();
            r.bwd_s += std::chrono::duration<double>(t2 - t1).count();
            r.opt_s += std::chrono::duration<double>(t4 - t3).count();
        }
    }
    if (!out.empty()) {
        Matrix lm(1, losses.size());
        for (size_t i = 0; i < losses.size(); ++i) lm(0, i) = losses[i];
        write_matrix(out, "losses", lm);
        if (do_opt)
            for (auto& [n, p] : named) write_matrix(out, "after." + n, p->data);
        Matrix live(1, 1);
        live(0, 0) = static_cast<float>(r.live);
        write_matrix(out, "live_after_fwd", live);
    }
    return r;
}

StepResult dispatch_family(const Args& a, const std::string& out) {
    const std::string fam = a.get("family", "llama");
    const unsigned seed = static_cast<unsigned>(a.geti("seed", 0));
    const bool ckpt = a.geti("ckpt", 0) != 0;
    if (fam == "llama") {
        nn::LlamaConfig c;
        c.vocab = a.geti("vocab", 97);
        c.d = a.geti("d", 32);
        c.n_layers = a.geti("layers", 2);
        c.n_heads = a.geti("heads", 4);
        c.d_ff = a.geti("dff", 64);
        c.n_ctx = a.geti("nctx", 256);
        c.rope_theta = static_cast<float>(a.getf("theta", 10000.0));
        c.tie_embeddings = a.geti("tie", 1) != 0;
        nn::Llama m(c, seed);
        m.checkpoint_blocks = ckpt;
        return run_steps(m, a, out);
    }
    if (fam == "gpt2") {
        nn::GPT2Config c;
        c.vocab = a.geti("vocab", 97);
        c.n_ctx = a.geti("nctx", 64);
        c.d = a.geti("d", 32);
        c.n_layers = a.geti("layers", 2);
        c.n_heads = a.geti("heads", 4);
        nn::GPT2 m(c, seed);
        m.checkpoint_blocks = ckpt;
        return run_steps(m, a, out);
    }
    if (fam == "flex") {
        parity::FlexConfig c;
        c.vocab = a.geti("vocab", 97);
        c.d = a.geti("d", 32);
        c.n_layers = a.geti("layers", 2);
        c.n_heads = a.geti("heads", 4);
        c.d_ff = a.geti("dff", 64);
        c.n_ctx = a.geti("nctx", 64);
        c.norm = a.get("norm", "layernorm");
        c.act = a.get("act", "gelu");
        c.pos = a.get("pos", "learned");
        CkptFlexLM m(c, seed);
        m.checkpoint_blocks = ckpt;
        return run_steps(m, a, out);
    }
    if (fam == "llamagqa" || fam == "qlora") {
        GQAConfig c;
        c.vocab = a.geti("vocab", 97);
        c.d = a.geti("d", 32);
        c.n_layers = a.geti("layers", 2);
        c.n_heads = a.geti("heads", 4);
        c.n_kv_heads = a.geti("kv-heads", 2);
        c.d_ff = a.geti("dff", 64);
        c.rope_theta = static_cast<float>(a.getf("theta", 10000.0));
        c.qlora = fam == "qlora";
        c.rank = a.geti("rank", 16);
        c.alpha = static_cast<float>(a.getf("alpha", 32.0));
        GQALlama m(c, seed);
        m.checkpoint_blocks = ckpt;
        return run_steps(m, a, out);
    }
    std::fprintf(stderr, "unknown family %s\n", fam.c_str());
    std::exit(2);
}

// ---------------------------------------------------------------- op goldens
void dump_ops(const std::string& out) {
    const size_t R = 67, C = 133;
    Matrix x = filled_uniform(R, C, 1, -1.5f, 1.5f);
    Matrix dy = filled_uniform(R, C, 2, -1.0f, 1.0f);
    Matrix w = filled_uniform(1, C, 3, 0.5f, 1.5f);
    Matrix bb = filled_uniform(1, C, 4, -0.5f, 0.5f);
    write_matrix(out, "x", x);
    write_matrix(out, "dy", dy);
    write_matrix(out, "w", w);
    write_matrix(out, "b", bb);

    // Pushes dy through `y` by building loss = sum(y .* dy) as mean * N.
    auto run = [&](const std::string& name, std::vector<Var> leaves, Var y,
                   std::vector<std::string> leaf_names, const Matrix& up) {
        write_matrix(out, name + ".y", y->data);
        Var prod = ops::mul(y, make_var(up));
        Var loss = ops::scale(ops::mean(prod), static_cast<float>(up.rows() * up.cols()));
        backward(loss);
        for (size_t i = 0; i < leaves.size(); ++i)
            if (leaves[i]->grad.rows() != 0) write_matrix(out, name + ".d" + leaf_names[i], leaves[i]->grad);
    };
    {
        Var vx = make_var(x, true), vw = make_var(w, true);
        run("rmsnorm", {vx, vw}, ops::rmsnorm(vx, vw), {"x", "w"}, dy);
    }
    {
        Var vx = make_var(x, true), vw = make_var(w, true), vb = make_var(bb, true);
        run("layernorm", {vx, vw, vb}, ops::layernorm(vx, vw, vb, 1e-5f), {"x", "w", "b"}, dy);
    }
    {
        Var vx = make_var(x, true);
        run("gelu", {vx}, ops::gelu(vx), {"x"}, dy);
    }
    {
        Var vx = make_var(x, true);
        run("silu", {vx}, ops::silu(vx), {"x"}, dy);
    }
    {
        Var vx = make_var(x, true);
        run("relu", {vx}, ops::relu(vx), {"x"}, dy);
    }
    {
        Matrix u = filled_uniform(R, C, 5, -1.5f, 1.5f);
        write_matrix(out, "u", u);
        Var vg = make_var(x, true), vu = make_var(u, true);
        run("swiglu", {vg, vu}, ops::mul(ops::silu(vg), vu), {"g", "u"}, dy);
    }
    {
        Var vx = make_var(x, true), vb = make_var(bb, true);
        run("add_bias", {vx, vb}, ops::add_bias(vx, vb), {"x", "b"}, dy);
    }
    {   // rope on a fused [T, 3d] tensor: d = 16, head_dim = 8 (two heads: the
        // reference rotates only the first head of q and of k)
        const size_t T = 24, d = 16, hd = 8;
        Matrix qkv = filled_uniform(T, 3 * d, 6, -1.0f, 1.0f);
        Matrix up = filled_uniform(T, 3 * d, 7, -1.0f, 1.0f);
        std::vector<int> pos(T);
        for (size_t i = 0; i < T; ++i) pos[i] = static_cast<int>(i % 12);
        write_matrix(out, "rope.qkv", qkv);
        write_matrix(out, "rope.up", up);
        write_ints(out, "rope.pos", pos);
        Var v = make_var(qkv, true);
        run("rope", {v}, ops::apply_rope(v, pos, 10000.0f, hd), {"qkv"}, up);
    }
    {   // one attention head, stacked batch of 3 sequences of 20, dk = 8
        const size_t T = 60, dk = 8, sl = 20;
        Matrix q = filled_uniform(T, dk, 8, -1.0f, 1.0f), k = filled_uniform(T, dk, 9, -1.0f, 1.0f),
               v = filled_uniform(T, dk, 10, -1.0f, 1.0f), up = filled_uniform(T, dk, 11, -1.0f, 1.0f);
        write_matrix(out, "attn.q", q);
        write_matrix(out, "attn.k", k);
        write_matrix(out, "attn.v", v);
        write_matrix(out, "attn.up", up);
        Var vq = make_var(q, true), vk = make_var(k, true), vv = make_var(v, true);
        run("attn", {vq, vk, vv},
            ops::fused_attention(vq, vk, vv, 1.0f / std::sqrt(static_cast<float>(dk)), sl, true),
            {"q", "k", "v"}, up);
    }
    {   // matmul 37x53 . 53x29 (tests/test_resident_parity.cpp:53-54)
        Matrix A = filled_uniform(37, 53, 12, -1.0f, 1.0f), Bm = filled_uniform(53, 29, 13, -1.0f, 1.0f),
               up = filled_uniform(37, 29, 14, -1.0f, 1.0f);
        write_matrix(out, "mm.a", A);
        write_matrix(out, "mm.b", Bm);
        write_matrix(out, "mm.up", up);
        Var va = make_var(A, true), vb = make_var(Bm, true);
        run("mm", {va, vb}, ops::matmul(va, vb), {"a", "b"}, up);
    }
    {   // embedding + cross entropy
        const size_t V = 50, d = 12, T = 40;
        Matrix table = filled_uniform(V, d, 15, -1.0f, 1.0f);
        auto ids = random_ids(T, 16, static_cast<int>(V));
        auto tg = random_ids(T, 17, static_cast<int>(d));
        write_matrix(out, "ce.table", table);
        write_ints(out, "ce.ids", ids);
        write_ints(out, "ce.targets", tg);
        Var vt = make_var(table, true);
        Var e = ops::embedding(vt, ids);  // [T, d] used directly as logits over d classes
        Var loss = ops::cross_entropy(e, tg);
        write_matrix(out, "ce.loss", loss->data);
        backward(loss);
        write_matrix(out, "ce.dtable", vt->grad);
    }
    {   // AdamW: three steps on one tensor with fixed grads
        Matrix p0 = filled_uniform(5, 7, 18, -1.0f, 1.0f);
        write_matrix(out, "adamw.p0", p0);
        Var p = make_var(p0, true);
        nn::AdamW opt({p}, 1e-3f);
        for (int s = 0; s < 3; ++s) {
            Matrix g = filled_uniform(5, 7, 19 + s, -1.0f, 1.0f);
            write_matrix(out, "adamw.g" + std::to_string(s), g);
            p->grad = g;
            opt.step();
            write_matrix(out, "adamw.p" + std::to_string(s + 1), p->data);
        }
    }
    {   // clip_grad_norm
        Var p = make_var(Matrix(3, 4), true), q = make_var(Matrix(2, 5), true);
        p->grad = filled_uniform(3, 4, 30, -2.0f, 2.0f);
        q->grad = filled_uniform(2, 5, 31, -2.0f, 2.0f);
        write_matrix(out, "clip.g0", p->grad);
        write_matrix(out, "clip.g1", q->grad);
        const float n = ops::clip_grad_norm({p, q}, 1.0f);
        Matrix nm(1, 1);
        nm(0, 0) = n;
        write_matrix(out, "clip.norm", nm);
        write_matrix(out, "clip.c0", p->grad);
        write_matrix(out, "clip.c1", q->grad);
    }
}

void dump_quant(const std::string& out) {
    // reference int8 (block 64, fp32 scale) and Q8_0 (block 32, fp16 scale)
    Matrix W = filled_uniform(24, 96, 1, -1.0f, 1.0f);
    for (size_t j = 0; j < 32; ++j) W(3, j) = 0.0f;  // an all-zero block (scale 1.0 rule)
    write_matrix(out, "q.W", W);
    QuantizedTensor t64 = quantize_int8(W, 64);
    QuantizedTensor t32 = quantize_q8_0(W);
    auto dumpq = [&](const std::string& name, const QuantizedTensor& t) {
        write_npy_raw(out + "/" + name + ".q.npy", t.q.data(), t.q.size(), "|i1", {t.rows, t.cols});
        const size_t bpr = (t.cols + t.block - 1) / t.block;
        write_npy_raw(out + "/" + name + ".scales.npy", t.scales.data(), t.scales.size() * 4, "<f4",
                      {t.rows, bpr});
        write_matrix(out, name + ".deq", dequantize(t));
    };
    dumpq("q.ref64", t64);
    dumpq("q.q8_0", t32);
    // QLoRA linear: forward/backward with the harness layer (Q8_0 base + LoRA)
    HLinear lin(96, 64, 5, 2, 4, 8.0f, 9);
    Matrix x = filled_uniform(10, 96, 2, -1.0f, 1.0f), up = filled_uniform(10, 64, 3, -1.0f, 1.0f);
    write_matrix(out, "ql.x", x);
    write_matrix(out, "ql.up", up);
    write_matrix(out, "ql.W0", filled_normal(96, 64, 5 * 7919u + 1u, 0.02f));
    write_matrix(out, "ql.Wdq", lin.Wdq);
    write_matrix(out, "ql.A", lin.A->data);
    write_matrix(out, "ql.B", lin.B->data);
    Var vx = make_var(x, true);
    Var y = lin.forward(vx);
    write_matrix(out, "ql.y", y->data);
    Var loss = ops::scale(ops::mean(ops::mul(y, make_var(up))), 640.0f);
    backward(loss);
    write_matrix(out, "ql.dx", vx->grad);
    write_matrix(out, "ql.dA", lin.A->grad);
    write_matrix(out, "ql.dB", lin.B->grad);
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: ref_harness step|ops|quant|bench [--key value ...]\n");
        return 2;
    }
    const std::string cmd = argv[1];
    Args a = parse(argc, argv, 2);
    const std::string out = a.get("out", "");
    if (cmd == "ops") {
        dump_ops(out);
        return 0;
    }
    if (cmd == "quant") {
        dump_quant(out);
        return 0;
    }
    if (cmd == "step") {
        StepResult r = dispatch_family(a, out);
        std::printf("{\"loss\": %.9g, \"live_after_fwd\": %zu, \"fwd_s\": %.4f, \"bwd_s\": %.4f, \"opt_s\": %.4f}\n",
                    r.loss, r.live, r.fwd_s, r.bwd_s, r.opt_s);
        return 0;
    }
    if (cmd == "bench") {
        // warm-up steps are run as a separate short invocation by the caller;
        // here every step is timed.
        auto t0 = std::chrono::steady_clock::now();
        StepResult r = dispatch_family(a, "");
        auto t1 = std::chrono::steady_clock::now();
        const double secs = std::chrono::duration<double>(t1 - t0).count();
        const double step_s = r.fwd_s + r.bwd_s + r.opt_s;
        const long steps = a.geti("steps", 1) - a.geti("warmup", 0);  // timed steps
        const double tokens = static_cast<double>(a.geti("batch", 1)) * a.geti("seq", 16) * steps;
        std::printf("{\"tokens_per_s\": %.4f, \"step_s\": %.5f, \"wall_s\": %.4f, \"loss\": %.9g, \"steps\": %ld}\n",
                    tokens / step_s, step_s / steps, secs, r.loss, steps);
        return 0;
    }
    std::fprintf(stderr, "unknown command %s\n", cmd.c_str());
    return 2;
}
