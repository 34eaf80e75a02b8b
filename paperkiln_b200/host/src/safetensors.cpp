// safetensors reader / writer. The header is a small, flat JSON object, so a recursive-descent
// reader for exactly the value kinds that can occur in it (objects, arrays, strings, numbers,
// true / false / null) is all that is needed; no JSON library is linked.
#include "microtorch/safetensors.hpp"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <vector>

namespace microtorch {

namespace {

struct TensorMeta {
    std::string dtype;
    std::vector<std::uint64_t> shape;
    std::vector<std::uint64_t> offsets;
};

class HeaderReader {
public:
    explicit HeaderReader(const std::string& text) : s_(text) {}

    // {"name": {...}, ...} -> one TensorMeta per tensor entry, in file order of the keys
    std::vector<std::pair<std::string, TensorMeta>> parse() {
        std::vector<std::pair<std::string, TensorMeta>> out;
        ws();
        expect('{');
        ws();
        if (peek() == '}') {
            ++i_;
            return out;
        }
        for (;;) {
            ws();
            std::string name = string();
            ws();
            expect(':');
            ws();
            if (name == "__metadata__") {
                skip_value();
            } else {
                out.emplace_back(std::move(name), tensor());
            }
            ws();
            if (peek() == ',') {
                ++i_;
                continue;
            }
            expect('}');
            break;
        }
        return out;
    }

private:
    const std::string& s_;
    size_t i_ = 0;

    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error(std::string("safetensors: malformed header (") + what + " at byte " +
                                 std::to_string(i_) + ")");
    }
    char peek() const {
        if (i_ >= s_.size()) fail("unexpected end");
        return s_[i_];
    }
    void expect(char c) {
        if (peek() != c) fail("unexpected character");
        ++i_;
    }
    void ws() {
        while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
    }
    std::string string() {
        expect('"');
        std::string out;
        for (;;) {
            const char c = peek();
            ++i_;
            if (c == '"') break;
            if (c != '\\') {
                out.push_back(c);
                continue;
            }
            const char e = peek();
            ++i_;
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'n': out.push_back('\n'); break;
                case 't': out.push_back('\t'); break;
                case 'r': out.push_back('\r'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'u': {  // tensor names are ASCII in practice: keep code points below 0x80, replace the rest
                    if (i_ + 4 > s_.size()) fail("short \\u escape");
                    const unsigned long cp = std::stoul(s_.substr(i_, 4), nullptr, 16);
                    i_ += 4;
                    out.push_back(cp < 0x80 ? static_cast<char>(cp) : '?');
                    break;
                }
                default: fail("bad escape");
            }
        }
        return out;
    }
    std::uint64_t unsigned_int() {
        const size_t start = i_;
        std::uint64_t v = 0;
        while (i_ < s_.size() && s_[i_] >= '0' && s_[i_] <= '9') {
            v = v * 10 + static_cast<std::uint64_t>(s_[i_] - '0');
            ++i_;
        }
        if (i_ == start) fail("expected a non-negative integer");
        return v;
    }
    std::vector<std::uint64_t> int_array() {
        std::vector<std::uint64_t> out;
        expect('[');
        ws();
        if (peek() == ']') {
            ++i_;
            return out;
        }
        for (;;) {
            ws();
            out.push_back(unsigned_int());
            ws();
            if (peek() == ',') {
                ++i_;
                continue;
            }
            expect(']');
            break;
        }
        return out;
    }
    TensorMeta tensor() {
        TensorMeta m;
        expect('{');
        for (;;) {
            ws();
            const std::string key = string();
            ws();
            expect(':');
            ws();
            if (key == "dtype") m.dtype = string();
            else if (key == "shape") m.shape = int_array();
            else if (key == "data_offsets") m.offsets = int_array();
            else skip_value();
            ws();
            if (peek() == ',') {
                ++i_;
                continue;
            }
            expect('}');
            break;
        }
        if (m.dtype.empty() || m.offsets.size() != 2) fail("tensor entry without dtype / data_offsets");
        return m;
    }
    void skip_value() {
        ws();
        const char c = peek();
        if (c == '"') {
            string();
        } else if (c == '{' || c == '[') {
            const char close = c == '{' ? '}' : ']';
            ++i_;
            ws();
            if (peek() == close) {
                ++i_;
                return;
            }
            for (;;) {
                ws();
                if (c == '{') {
                    string();
                    ws();
                    expect(':');
                }
                skip_value();
                ws();
                if (peek() == ',') {
                    ++i_;
                    continue;
                }
                expect(close);
                break;
            }
        } else {  // number, true, false, null
            while (i_ < s_.size() && s_[i_] != ',' && s_[i_] != '}' && s_[i_] != ']' && s_[i_] != ' ' &&
                   s_[i_] != '\n' && s_[i_] != '\t' && s_[i_] != '\r')
                ++i_;
        }
    }
};

std::string quoted(const std::string& s) {
    std::string out = "\"";
    for (const char c : s) {
        if (c == '"' || c == '\\') {
            out.push_back('\\');
            out.push_back(c);
        } else if (static_cast<unsigned char>(c) < 0x20) {
            char buf[8];
            std::snprintf(buf, sizeof(buf), "\\u%04x", static_cast<unsigned>(static_cast<unsigned char>(c)));
            out += buf;
        } else {
            out.push_back(c);
        }
    }
    out.push_back('"');
    return out;
}

}  // namespace

std::map<std::string, Matrix> load_safetensors(const std::string& path,
                                               std::map<std::string, std::string>* skipped) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("safetensors: cannot open " + path);
    unsigned char lenb[8];
    f.read(reinterpret_cast<char*>(lenb), 8);
    std::uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | lenb[i];
    if (!f || hlen == 0 || hlen > (1u << 26)) throw std::runtime_error("safetensors: implausible header length");
    std::string htext(hlen, '\0');
    f.read(htext.data(), static_cast<std::streamsize>(hlen));
    if (!f) throw std::runtime_error("safetensors: short header");
    const auto entries = HeaderReader(htext).parse();
    const std::streamoff base = 8 + static_cast<std::streamoff>(hlen);
    f.seekg(0, std::ios::end);
    const std::uint64_t file_size = static_cast<std::uint64_t>(f.tellg());
    const std::uint64_t data_size = file_size - static_cast<std::uint64_t>(base);

    std::map<std::string, Matrix> out;
    std::vector<std::uint16_t> half;
    for (const auto& [raw_name, meta] : entries) {
        std::string name = raw_name;
        if (name.rfind("transformer.", 0) == 0) name = name.substr(12);
        if (meta.shape.size() > 2) {
            if (skipped) (*skipped)[name] = "rank " + std::to_string(meta.shape.size());
            continue;
        }
        const bool f32 = meta.dtype == "F32", bf16 = meta.dtype == "BF16";
        if (!f32 && !bf16)
            throw std::runtime_error("safetensors: " + name + " is " + meta.dtype + "; this loader reads F32 and BF16");
        const size_t rows = meta.shape.size() == 2 ? meta.shape[0] : 1;
        const size_t cols = meta.shape.size() == 2 ? meta.shape[1] : (meta.shape.empty() ? 1 : meta.shape[0]);
        // Nothing is allocated before the header's claims have been checked against each other and
        // against the file: the byte range lies inside the data section, the element count does
        // not overflow, and shape x element size is exactly the range.
        if (meta.offsets[1] < meta.offsets[0] || meta.offsets[1] > data_size)
            throw std::runtime_error("safetensors: data range of " + name + " lies outside the file");
        const std::uint64_t nbytes = meta.offsets[1] - meta.offsets[0];
        const std::uint64_t esize = f32 ? 4 : 2;
        const std::uint64_t r64 = rows, c64 = cols;
        if (r64 != 0 && c64 > (std::uint64_t(1) << 62) / r64)
            throw std::runtime_error("safetensors: shape of " + name + " overflows");
        if (r64 * c64 > nbytes / esize || r64 * c64 * esize != nbytes)
            throw std::runtime_error("safetensors: size mismatch at " + name);
        Matrix m(rows, cols);
        f.seekg(base + static_cast<std::streamoff>(meta.offsets[0]));
        if (f32) {
            f.read(reinterpret_cast<char*>(m.data()), static_cast<std::streamsize>(nbytes));
        } else {
            half.resize(rows * cols);
            f.read(reinterpret_cast<char*>(half.data()), static_cast<std::streamsize>(nbytes));
            float* dst = m.data();
            for (size_t i = 0; i < half.size(); ++i) {  // bf16 -> fp32: the upper 16 bits
                const std::uint32_t bits = static_cast<std::uint32_t>(half[i]) << 16;
                std::memcpy(dst + i, &bits, 4);
            }
        }
        if (!f) throw std::runtime_error("safetensors: short read at " + name);
        out.emplace(std::move(name), std::move(m));
    }
    return out;
}

void save_safetensors(const std::string& path, const std::map<std::string, Matrix>& tensors) {
    // keys in sorted order (std::map), entry keys sorted too: "data_offsets", "dtype", "shape"
    std::string htext = "{";
    std::uint64_t offset = 0;
    bool first = true;
    for (const auto& [name, m] : tensors) {
        const std::uint64_t nbytes = static_cast<std::uint64_t>(m.rows()) * m.cols() * sizeof(float);
        if (!first) htext += ",";
        first = false;
        htext += quoted(name) + ":{\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + nbytes) +
                 "],\"dtype\":\"F32\",\"shape\":[" + std::to_string(m.rows()) + "," + std::to_string(m.cols()) + "]}";
        offset += nbytes;
    }
    htext += "}";
    while (htext.size() % 8 != 0) htext.push_back(' ');  // tensor data starts 8-byte aligned

    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("safetensors: cannot write " + path);
    const std::uint64_t hlen = htext.size();
    unsigned char lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = static_cast<unsigned char>((hlen >> (8 * i)) & 0xff);
    f.write(reinterpret_cast<const char*>(lenb), 8);
    f.write(htext.data(), static_cast<std::streamsize>(hlen));
    for (const auto& [name, m] : tensors) {
        (void)name;
        f.write(reinterpret_cast<const char*>(m.data()), static_cast<std::streamsize>(m.size() * sizeof(float)));
    }
    if (!f) throw std::runtime_error("safetensors: write failed " + path);
}

}  // namespace microtorch
