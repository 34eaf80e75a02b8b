// Generates tests/golden/ref_export_*.gguf: loads a safetensors file with the UNMODIFIED reference
// reader and exports it with the reference's GGUF exporter (src/gguf.cpp:27-166 on top of
// third_party/transformer_cpp/src/gguf_export.cpp), so that the committed files pin the
// reference's byte layout. Built and run once, where the reference tree is available (REF = its
// root, TP = REF/third_party/transformer_cpp, JSON = a directory holding nlohmann/json.hpp, OBJ =
// objects of TP/src/{components,matrix,matmul_optimized,vector_ops}.cpp as oracle/Makefile
// builds them):
//   g++ -O1 -std=c++17 -fopenmp -I$REF/include -I$TP/include -I$TP/third_party -I$JSON \
//       gguf_ref_writer.cpp $REF/src/safetensors.cpp $REF/src/gguf.cpp $TP/src/gguf_export.cpp \
//       $OBJ/tp_*.o -Wl,--unresolved-symbols=ignore-all -o gguf_ref_writer
// (the linker flag: gguf_export.cpp also holds an exporter for the vendored tree's own model
// classes, which are not linked and not used here)
//   ./gguf_ref_writer gguf_in_out.safetensors ref_export_in_out.gguf 1 1     (in_out, tokens)
//   ./gguf_ref_writer gguf_out_in.safetensors ref_export_out_in.gguf 0 0
// The inputs are written by tests/test_gguf_cpu.py::make_state (numpy RandomState(11); vocab 11,
// d 8, 2 heads, 1 kv head, d_ff 16, 2 blocks; the second one carries an untied lm_head and a
// tensor with no place in the layout).
#include <cstdio>
#include <cstdlib>

#include "microtorch/gguf.hpp"
#include "microtorch/safetensors.hpp"

int main(int argc, char** argv) {
    if (argc != 5) return 2;
    auto sd = microtorch::load_safetensors(argv[1]);
    microtorch::gguf::LlamaExportConfig c;
    c.name = "tiny";
    c.context_length = 64;
    c.embedding_length = 8;
    c.block_count = 2;
    c.feed_forward_length = 16;
    c.head_count = 2;
    c.head_count_kv = 1;
    c.vocab_size = 11;
    c.rms_eps = 1e-5f;
    c.rope_freq_base = 10000.0f;
    c.weights_in_out = std::atoi(argv[3]) != 0;
    if (std::atoi(argv[4]) != 0) c.tokens = {"<unk>", "<s>", "a", "b", "cc", "ddd", "e", "f", "g", "h", "ii"};
    std::vector<std::string> unmapped;
    microtorch::gguf::export_gguf_llama(argv[2], sd, c, &unmapped);
    std::printf("unmapped %zu\n", unmapped.size());
    return 0;
}
