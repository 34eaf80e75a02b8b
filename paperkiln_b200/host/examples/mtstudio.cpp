// mtstudio-compatible run driver over libmicrotorch: reads the run spec the reference's trainer
// reads (tools/mtstudio.cpp:83-169 there), runs its batch / accum training loop (:448-518) on the
// GPU with per-block activation checkpointing for every family, and emits the same JSONL events
// (:181-192, 482-486, 561-566) on stdout and in <out_dir>/events.jsonl, so a consumer of that
// stream (the reference's studio page) works unchanged.
//
//   mtstudio run spec.json        execute the spec
//   mtstudio plan spec.json       print the resolved plan and exit
//
// Spec keys honoured: name; arch.preset (gpt2-nano, gpt2-small, llama-tiny) or arch.custom {d, layers,
// heads, norm, activation, position, d_ff}; data {corpus, vocab, vocab_cap, T}; train {steps, lr, clip,
// eval_every, checkpoint_every, batch, accum, checkpoint_activations, seed, early_stopping {patience,
// min_delta}}; export.formats (safetensors, gguf); out_dir. Added keys: train.dtype ("fp32" | "bf16",
// default: MICROTORCH_DTYPE or fp32) and data.synthetic_tokens (length of a seeded random token
// stream used when no corpus is given). Differences from the reference, all on purpose:
//   * train.checkpoint_activations works for the gpt2 / flex families too (the reference refuses);
//   * the vocabulary is a text file with one token per line, or is built from the corpus (most
//     frequent words first); a .gguf vocabulary is not read;
//   * besides model.safetensors + state.txt a checkpoint holds the AdamW state (optimizer.bin), so a
//     resumed run continues with its moments instead of restarting them;
//   * the kimi / srd / swa / attnres presets and the muon optimizer are outside this library.
#include <sys/stat.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <map>
#include <memory>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "microtorch/flex.hpp"
#include "microtorch/gguf.hpp"
#include "microtorch/llama.hpp"
#include "microtorch/ops.hpp"
#include "microtorch/safetensors.hpp"

using namespace microtorch;

namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, booleans, null, // comments) ----
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    const Json* find(const std::string& key) const {
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    const Json& at(const std::string& key) const {
        static const Json none;
        const Json* j = find(key);
        return j ? *j : none;
    }
    double number(const std::string& key, double d) const {
        const Json* j = find(key);
        return j && j->kind == Num ? j->num : d;
    }
    std::string string(const std::string& key, const std::string& d) const {
        const Json* j = find(key);
        return j && j->kind == Str ? j->str : d;
    }
    bool boolean(const std::string& key, bool d) const {
        const Json* j = find(key);
        return j && j->kind == Bool ? j->b : d;
    }
};

class JsonReader {
public:
    explicit JsonReader(const std::string& text) : s_(text) {}
    Json parse() {
        Json v = value();
        skip();
        if (i_ != s_.size()) fail("trailing characters");
        return v;
    }

private:
    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error("spec: " + std::string(what) + " at offset " + std::to_string(i_));
    }
    void skip() {
        for (;;) {
            while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
            if (i_ + 1 < s_.size() && s_[i_] == '/' && s_[i_ + 1] == '/') {
                while (i_ < s_.size() && s_[i_] != '\n') ++i_;
                continue;
            }
            return;
        }
    }
    Json value() {
        skip();
        if (i_ >= s_.size()) fail("unexpected end");
        const char c = s_[i_];
        Json v;
        if (c == '{') {
            v.kind = Json::Obj;
            ++i_;
            skip();
            if (i_ < s_.size() && s_[i_] == '}') { ++i_; return v; }
            for (;;) {
                skip();
                Json k = value();
                if (k.kind != Json::Str) fail("object key must be a string");
                skip();
                if (i_ >= s_.size() || s_[i_] != ':') fail("expected ':'");
                ++i_;
                v.obj.emplace_back(k.str, value());
                skip();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == '}') { ++i_; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v.kind = Json::Arr;
            ++i_;
            skip();
            if (i_ < s_.size() && s_[i_] == ']') { ++i_; return v; }
            for (;;) {
                v.arr.push_back(value());
                skip();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == ']') { ++i_; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            v.kind = Json::Str;
            ++i_;
            while (i_ < s_.size() && s_[i_] != '"') {
                if (s_[i_] == '\\' && i_ + 1 < s_.size()) {
                    const char e = s_[++i_];
                    v.str.push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e);
                } else {
                    v.str.push_back(s_[i_]);
                }
                ++i_;
            }
            if (i_ >= s_.size()) fail("unterminated string");
            ++i_;
            return v;
        }
        if (s_.compare(i_, 4, "true") == 0) { v.kind = Json::Bool; v.b = true; i_ += 4; return v; }
        if (s_.compare(i_, 5, "false") == 0) { v.kind = Json::Bool; v.b = false; i_ += 5; return v; }
        if (s_.compare(i_, 4, "null") == 0) { i_ += 4; return v; }
        size_t used = 0;
        try {
            v.num = std::stod(s_.substr(i_, 64), &used);
        } catch (...) {
            fail("unexpected token");
        }
        v.kind = Json::Num;
        i_ += used;
        return v;
    }
    const std::string& s_;
    size_t i_ = 0;
};

std::string quote(const std::string& s) {
    std::string out = "\"";
    for (char c : s) {
        if (c == '"' || c == '\\') out.push_back('\\');
        if (c == '\n') { out += "\\n"; continue; }
        out.push_back(c);
    }
    return out + "\"";
}
std::string num(double v) {
    char buf[48];
    std::snprintf(buf, sizeof(buf), "%.9g", v);
    return buf;
}

// One JSON object per line, to stdout and to <out>/events.jsonl.
struct Events {
    std::ofstream file;
    explicit Events(const std::string& path) : file(path, std::ios::app) {}
    void emit(const std::vector<std::pair<std::string, std::string>>& fields) {
        std::string line = "{";
        for (size_t i = 0; i < fields.size(); ++i) line += (i ? "," : "") + quote(fields[i].first) + ":" + fields[i].second;
        line += "}";
        std::printf("%s\n", line.c_str());
        std::fflush(stdout);
        file << line << "\n";
        file.flush();
    }
};

struct Spec {
    std::string name = "run", family = "gpt2", norm, activation, position, corpus, vocab, out_dir = "mtstudio_out";
    std::string dtype;
    size_t d = 128, layers = 2, heads = 4, T = 128, d_ff = 0, vocab_cap = 4096, synthetic_tokens = 200000;
    int steps = 500, eval_every = 50, ckpt_every = 100, batch = 1, accum = 1;
    float lr = 3e-3f, clip = 1.0f, es_min_delta = 0.0f;
    bool ckpt_act = false, exp_safetensors = true, exp_gguf = false;
    unsigned seed = 7;
    size_t es_patience = 0;
};

Spec parse_spec(const std::string& path) {
    std::ifstream f(path);
    if (!f) throw std::runtime_error("cannot open spec " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    const Json j = JsonReader(text).parse();
    Spec s;
    s.name = j.string("name", s.name);
    const Json& arch = j.at("arch");
    const std::string preset = arch.string("preset", "");
    if (!preset.empty()) {
        // name -> {d, layers, heads, T} (the reference's table, tools/mtstudio.cpp:73-81)
        static const std::map<std::string, std::vector<size_t>> presets = {
            {"gpt2-nano", {128, 2, 4, 128}}, {"llama-tiny", {128, 2, 4, 128}}, {"gpt2-small", {256, 4, 8, 256}}};
        auto it = presets.find(preset);
        if (it == presets.end())
            throw std::runtime_error("preset " + preset + " is not provided (gpt2-nano, gpt2-small, llama-tiny are)");
        s.d = it->second[0]; s.layers = it->second[1]; s.heads = it->second[2]; s.T = it->second[3];
        if (preset.rfind("llama", 0) == 0) s.family = "llama";
    }
    const Json& c = arch.at("custom");
    s.d = static_cast<size_t>(c.number("d", s.d));
    s.layers = static_cast<size_t>(c.number("layers", s.layers));
    s.heads = static_cast<size_t>(c.number("heads", s.heads));
    s.norm = c.string("norm", "");
    s.activation = c.string("activation", "");
    s.position = c.string("position", "");
    s.d_ff = static_cast<size_t>(c.number("d_ff", 0));
    const std::string attention = c.string("attention", "exact");
    if (attention != "exact") throw std::runtime_error("attention " + attention + " is outside this library (exact only)");
    if (s.position == "rope") {
        if ((!s.norm.empty() && s.norm != "rmsnorm") || (!s.activation.empty() && s.activation != "swiglu"))
            throw std::runtime_error("position=rope implies the llama block (rmsnorm + swiglu)");
        s.family = "llama";
    } else if (!s.norm.empty() || !s.activation.empty() || !s.position.empty() || s.family == "gpt2") {
        // the flex family with its defaults (layernorm, gelu, learned positions) is the GPT-2 block
        if (s.family != "llama") s.family = "flex";
    }
    const Json& data = j.at("data");
    s.corpus = data.string("corpus", "");
    s.vocab = data.string("vocab", "");
    s.vocab_cap = static_cast<size_t>(data.number("vocab_cap", s.vocab_cap));
    s.T = static_cast<size_t>(data.number("T", s.T));
    s.synthetic_tokens = static_cast<size_t>(data.number("synthetic_tokens", s.synthetic_tokens));
    const Json& tr = j.at("train");
    s.steps = static_cast<int>(tr.number("steps", s.steps));
    s.lr = static_cast<float>(tr.number("lr", s.lr));
    s.clip = static_cast<float>(tr.number("clip", s.clip));
    s.eval_every = static_cast<int>(tr.number("eval_every", s.eval_every));
    s.ckpt_every = static_cast<int>(tr.number("checkpoint_every", s.ckpt_every));
    s.batch = static_cast<int>(tr.number("batch", s.batch));
    s.accum = static_cast<int>(tr.number("accum", s.accum));
    s.ckpt_act = tr.boolean("checkpoint_activations", s.ckpt_act);
    s.seed = static_cast<unsigned>(tr.number("seed", s.seed));
    s.dtype = tr.string("dtype", "");
    if (tr.string("optimizer", "adamw") != "adamw") throw std::runtime_error("only the adamw optimizer is provided");
    const Json& es = tr.at("early_stopping");
    s.es_patience = static_cast<size_t>(es.number("patience", 0));
    s.es_min_delta = static_cast<float>(es.number("min_delta", 0.0));
    const Json* formats = j.at("export").find("formats");
    if (formats && formats->kind == Json::Arr) {
        s.exp_safetensors = s.exp_gguf = false;
        for (const Json& fm : formats->arr) {
            if (fm.str == "gguf") s.exp_gguf = true;
            if (fm.str == "safetensors") s.exp_safetensors = true;
        }
    }
    s.out_dir = j.string("out_dir", s.out_dir);
    if (s.batch < 1 || s.accum < 1 || s.steps < 0 || s.T < 2) throw std::runtime_error("spec: batch, accum >= 1, T >= 2");
    return s;
}

// Tokens of the run: a word-level vocabulary (file with one token per line, or the corpus' most
// frequent words) and the corpus as ids; without a corpus a seeded random stream.
void load_data(const Spec& s, std::vector<std::string>& tokens, std::vector<int>& ids) {
    if (s.corpus.empty()) {
        tokens.resize(s.vocab_cap);
        for (size_t i = 0; i < tokens.size(); ++i) tokens[i] = "t" + std::to_string(i);
        std::mt19937 rng(4242 + s.seed);
        ids.resize(std::max(s.synthetic_tokens, 4 * s.T + 8));
        for (auto& t : ids) t = static_cast<int>(rng() % s.vocab_cap);
        return;
    }
    std::ifstream f(s.corpus);
    if (!f) throw std::runtime_error("cannot open corpus " + s.corpus);
    std::vector<std::string> words;
    for (std::string w; f >> w;) {
        std::transform(w.begin(), w.end(), w.begin(), [](unsigned char ch) { return static_cast<char>(std::tolower(ch)); });
        words.push_back(w);
    }
    std::map<std::string, int> index;
    if (!s.vocab.empty()) {
        if (s.vocab.size() > 5 && s.vocab.substr(s.vocab.size() - 5) == ".gguf")
            throw std::runtime_error("a .gguf vocabulary is not read; give a text file with one token per line");
        std::ifstream vf(s.vocab);
        if (!vf) throw std::runtime_error("cannot open vocabulary " + s.vocab);
        for (std::string t; std::getline(vf, t) && tokens.size() < s.vocab_cap;) tokens.push_back(t);
    } else {
        std::map<std::string, size_t> freq;
        for (const auto& w : words) ++freq[w];
        std::vector<std::pair<size_t, std::string>> order;
        for (const auto& kv : freq) order.emplace_back(kv.second, kv.first);
        std::sort(order.begin(), order.end(), [](const auto& a, const auto& b) { return a.first != b.first ? a.first > b.first : a.second < b.second; });
        tokens.push_back("<unk>");
        for (size_t i = 0; i < order.size() && tokens.size() < s.vocab_cap; ++i) tokens.push_back(order[i].second);
    }
    for (size_t i = 0; i < tokens.size(); ++i) index.emplace(tokens[i], static_cast<int>(i));
    ids.reserve(words.size());
    for (const auto& w : words) {
        auto it = index.find(w);
        ids.push_back(it == index.end() ? 0 : it->second);
    }
    if (ids.size() < 4 * s.T + 8) throw std::runtime_error("corpus too short for T");
}

void save_optimizer(const std::string& path, nn::AdamW& opt, const std::vector<Var>& params) {
    std::ofstream f(path, std::ios::binary);
    const long t = opt.steps_taken();
    f.write(reinterpret_cast<const char*>(&t), sizeof(t));
    for (size_t i = 0; i < params.size(); ++i) {
        const size_t n = params[i]->data.rows() * params[i]->data.cols();
        std::vector<float> m(n), v(n);
        opt.export_state(i, m.data(), v.data());
        f.write(reinterpret_cast<const char*>(m.data()), static_cast<std::streamsize>(n * sizeof(float)));
        f.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(n * sizeof(float)));
    }
}
bool load_optimizer(const std::string& path, nn::AdamW& opt, const std::vector<Var>& params) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    long t = 0;
    f.read(reinterpret_cast<char*>(&t), sizeof(t));
    for (size_t i = 0; i < params.size() && f; ++i) {
        const size_t n = params[i]->data.rows() * params[i]->data.cols();
        std::vector<float> m(n), v(n);
        f.read(reinterpret_cast<char*>(m.data()), static_cast<std::streamsize>(n * sizeof(float)));
        f.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(n * sizeof(float)));
        if (f) opt.import_state(i, m.data(), v.data());
    }
    if (!f) return false;
    opt.set_steps_taken(t);
    return true;
}

int run(const Spec& s, bool plan_only) {
    std::vector<std::string> tokens;
    std::vector<int> ids;
    load_data(s, tokens, ids);
    const size_t d_ff = s.d_ff ? s.d_ff : (s.family == "llama" ? 3 * s.d : 4 * s.d);
    if (plan_only) {
        std::printf("plan: %s family=%s d=%zu layers=%zu heads=%zu T=%zu d_ff=%zu vocab=%zu steps=%d batch=%d accum=%d "
                    "checkpoint_activations=%d out_dir=%s tokens=%zu\n",
                    s.name.c_str(), s.family.c_str(), s.d, s.layers, s.heads, s.T, d_ff, tokens.size(), s.steps, s.batch,
                    s.accum, s.ckpt_act ? 1 : 0, s.out_dir.c_str(), ids.size());
        return 0;
    }
    mkdir(s.out_dir.c_str(), 0755);
    Events ev(s.out_dir + "/events.jsonl");

    device::set_from_env();
    if (s.dtype == "bf16") device::set_compute_dtype(DType::BF16);
    else if (s.dtype == "fp32") device::set_compute_dtype(DType::F32);
    else if (!s.dtype.empty()) throw std::runtime_error("train.dtype must be fp32 or bf16");
    device::init(0);

    std::shared_ptr<nn::Llama> llama;
    std::shared_ptr<parity::FlexLM> flex;
    if (s.family == "llama") {
        nn::LlamaConfig lc;
        lc.vocab = tokens.size(); lc.d = s.d; lc.n_layers = s.layers; lc.n_heads = s.heads; lc.d_ff = d_ff; lc.n_ctx = s.T;
        llama = std::make_shared<nn::Llama>(lc, s.seed);
        llama->checkpoint_blocks = s.ckpt_act;
    } else {
        parity::FlexConfig fc;
        fc.vocab = tokens.size(); fc.d = s.d; fc.n_layers = s.layers; fc.n_heads = s.heads; fc.d_ff = d_ff; fc.n_ctx = s.T;
        if (!s.norm.empty()) fc.norm = s.norm;
        if (!s.activation.empty()) fc.act = s.activation;
        if (!s.position.empty()) fc.pos = s.position;
        flex = std::make_shared<parity::FlexLM>(fc, s.seed);
        flex->checkpoint_blocks = s.ckpt_act;
    }
    nn::Module& model = llama ? static_cast<nn::Module&>(*llama) : static_cast<nn::Module&>(*flex);
    auto loss_of = [&](const std::vector<int>& x, const std::vector<int>& y, size_t seq_len) {
        return llama ? llama->loss(x, y, seq_len) : flex->loss(x, y, seq_len);
    };
    const std::string r_norm = flex ? flex->cfg.norm : "rmsnorm", r_act = flex ? flex->cfg.act : "swiglu",
                      r_pos = flex ? flex->cfg.pos : "rope";
    ev.emit({{"event", quote("model")}, {"family", quote(s.family)}, {"attention", quote("exact")}, {"d", num(s.d)},
             {"layers", num(s.layers)}, {"heads", num(s.heads)}, {"T", num(s.T)}, {"norm", quote(r_norm)},
             {"activation", quote(r_act)}, {"position", quote(r_pos)}, {"d_ff", num(d_ff)}, {"vocab", num(tokens.size())},
             {"batch", num(s.batch)}, {"accum", num(s.accum)}, {"lr", num(s.lr)}, {"seed", num(s.seed)},
             {"checkpoint_activations", s.ckpt_act ? "true" : "false"}, {"params", num(model.parameter_count())}});
    model.train();
    const std::vector<Var> params = model.parameters();
    nn::AdamW opt(params, s.lr);

    const std::string ckpt = s.out_dir + "/model.safetensors", state_path = s.out_dir + "/state.txt",
                      opt_path = s.out_dir + "/optimizer.bin";
    int start_step = 0;
    {
        std::ifstream st(state_path);
        if (st >> start_step && start_step > 0) {
            model.load_state_dict(load_safetensors(ckpt));
            load_optimizer(opt_path, opt, params);
            ev.emit({{"event", quote("resume")}, {"step", num(start_step)}});
        } else {
            start_step = 0;
        }
    }
    // data order: the reference's generator and seed rule; a resumed run replays the draws it skipped
    std::mt19937 rng(123 + 1000003u * s.seed);
    for (int i = 0; i < start_step * s.accum * s.batch; ++i) rng();
    const size_t val_start = ids.size() - ids.size() / 10;   // last tenth held out
    auto save = [&](int step) {
        save_safetensors(ckpt, model.state_dict());
        save_optimizer(opt_path, opt, params);
        std::ofstream st(state_path);
        st << step << "\n";
    };

    const auto t0 = std::chrono::steady_clock::now();
    float best_val = 1e30f;
    size_t evals_flat = 0;
    bool stopped_early = false;
    int last_step = start_step;
    for (int step = start_step + 1; step <= s.steps; ++step) {
        last_step = step;
        const size_t lim = val_start - s.T - 1;
        opt.zero_grad();
        float task_mean = 0.0f;
        for (int k = 0; k < s.accum; ++k) {
            std::vector<int> x, y;
            x.reserve(s.batch * s.T);
            y.reserve(s.batch * s.T);
            for (int b = 0; b < s.batch; ++b) {
                const size_t at = rng() % lim;
                x.insert(x.end(), ids.begin() + at, ids.begin() + at + s.T);
                y.insert(y.end(), ids.begin() + at + 1, ids.begin() + at + s.T + 1);
            }
            Var task = loss_of(x, y, s.batch > 1 ? s.T : 0);
            backward(s.accum == 1 ? task : ops::scale(task, 1.0f / static_cast<float>(s.accum)));
            task_mean += task->data.host()(0, 0) / static_cast<float>(s.accum);
        }
        const float total_norm = ops::clip_grad_norm(params, s.clip);
        opt.step();
        ev.emit({{"event", quote("step")}, {"step", num(step)}, {"loss", num(task_mean)}, {"grad_norm", num(total_norm)}});

        if (s.eval_every > 0 && step % s.eval_every == 0) {
            NoGrad ng;
            model.eval();
            double vl = 0.0;
            const int NV = 8;
            std::mt19937 vrng(999);
            for (int k = 0; k < NV; ++k) {
                const size_t va = val_start + vrng() % (ids.size() - val_start - s.T - 1);
                std::vector<int> vx(ids.begin() + va, ids.begin() + va + s.T), vy(ids.begin() + va + 1, ids.begin() + va + s.T + 1);
                vl += loss_of(vx, vy, 0)->data.host()(0, 0);
            }
            vl /= NV;
            model.train();
            ev.emit({{"event", quote("eval")}, {"step", num(step)}, {"val_loss", num(vl)}});
            if (s.es_patience > 0) {
                if (vl < best_val - s.es_min_delta) {
                    best_val = static_cast<float>(vl);
                    evals_flat = 0;
                } else if (++evals_flat >= s.es_patience) {
                    ev.emit({{"event", quote("early_stop")}, {"step", num(step)}, {"best_val", num(best_val)}});
                    stopped_early = true;
                }
            } else if (vl < best_val) {
                best_val = static_cast<float>(vl);
            }
        }
        if ((s.ckpt_every > 0 && step % s.ckpt_every == 0) || stopped_early || step == s.steps) {
            save(step);
            if (stopped_early) break;
        }
    }

    if (s.exp_safetensors) {
        const std::string path = s.out_dir + "/" + s.name + ".safetensors";
        save_safetensors(path, model.state_dict());
        ev.emit({{"event", quote("export")}, {"format", quote("safetensors")}, {"path", quote(path)}});
    }
    if (s.exp_gguf) {
        if (llama) {
            auto sd = model.state_dict();
            if (!sd.count("lm_head.weight")) sd.emplace("lm_head.weight", llama->embed_tokens->weight->data.host().transpose());
            gguf::LlamaExportConfig gc;
            gc.name = s.name;
            gc.embedding_length = static_cast<uint32_t>(s.d);
            gc.block_count = static_cast<uint32_t>(s.layers);
            gc.head_count = static_cast<uint32_t>(s.heads);
            gc.feed_forward_length = static_cast<uint32_t>(d_ff);
            gc.vocab_size = static_cast<uint32_t>(tokens.size());
            gc.context_length = static_cast<uint32_t>(s.T);
            gc.rms_eps = 1e-6f;
            gc.weights_in_out = true;
            gc.tokens = tokens;
            const std::string path = s.out_dir + "/" + s.name + ".gguf";
            gguf::export_gguf_llama(path, sd, gc);
            ev.emit({{"event", quote("export")}, {"format", quote("gguf")}, {"path", quote(path)}});
        } else {
            ev.emit({{"event", quote("export_skipped")}, {"format", quote("gguf")},
                     {"reason", quote("gpt2-family blocks are not llama-shaped")}});
        }
    }
    const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    ev.emit({{"event", quote("done")}, {"best_val", num(best_val)}, {"early_stopped", stopped_early ? "true" : "false"},
             {"final_step", num(last_step)}, {"wall_seconds", num(wall)}});
    {
        const double tps = wall > 0 ? (last_step - start_step) * static_cast<double>(s.batch) * s.accum * s.T / wall : 0.0;
        std::ofstream rf(s.out_dir + "/result.json");
        rf << "{\n  \"name\": " << quote(s.name) << ",\n  \"family\": " << quote(s.family) << ",\n  \"d\": " << s.d
           << ",\n  \"layers\": " << s.layers << ",\n  \"heads\": " << s.heads << ",\n  \"T\": " << s.T << ",\n  \"batch\": "
           << s.batch << ",\n  \"accum\": " << s.accum << ",\n  \"lr\": " << num(s.lr) << ",\n  \"seed\": " << s.seed
           << ",\n  \"checkpoint_activations\": " << (s.ckpt_act ? "true" : "false") << ",\n  \"params\": "
           << model.parameter_count() << ",\n  \"steps_requested\": " << s.steps << ",\n  \"final_step\": " << last_step
           << ",\n  \"best_val\": " << num(best_val) << ",\n  \"early_stopped\": " << (stopped_early ? "true" : "false")
           << ",\n  \"wall_seconds\": " << num(wall) << ",\n  \"tokens_per_second\": " << num(tps) << "\n}\n";
    }
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 3 || (std::string(argv[1]) != "run" && std::string(argv[1]) != "plan")) {
        std::fprintf(stderr, "usage: mtstudio run|plan spec.json\n");
        return 2;
    }
    try {
        return run(parse_spec(argv[2]), std::string(argv[1]) == "plan");
    } catch (const std::exception& e) {
        std::fprintf(stderr, "mtstudio: %s\n", e.what());
        return 1;
    }
}
