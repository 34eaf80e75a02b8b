// Generates tests/golden/ref_writer.safetensors: loads a safetensors file with the UNMODIFIED
// reference reader and writes it back with the reference writer (src/safetensors.cpp:12-94), so
// that the committed file pins the reference's byte layout. Built and run once, where the
// reference tree is available (REF = its root, TP = REF/third_party/transformer_cpp, JSON = a
// directory holding nlohmann/json.hpp, OBJ = objects of TP/src/{components,matrix,
// matmul_optimized,vector_ops}.cpp as oracle/Makefile builds them):
//   g++ -O1 -std=c++17 -fopenmp -I$REF/include -I$TP/include -I$TP/third_party -I$JSON \
//       safetensors_ref_writer.cpp $REF/src/safetensors.cpp $OBJ/tp_*.o -o ref_writer
//   ./ref_writer in.safetensors ref_writer.safetensors
// in.safetensors was written by tests/test_safetensors_cpu.py::write_file with numpy
// RandomState(1): "layers.0.wq" = randn(5, 9), "final_norm.weight" = randn(9), both float32.
#include <cstdio>

#include "microtorch/safetensors.hpp"

int main(int argc, char** argv) {
    if (argc != 3) return 2;
    auto t = microtorch::load_safetensors(argv[1]);
    for (auto& [n, m] : t) std::printf("%s %zu %zu %.6f\n", n.c_str(), m.rows(), m.cols(), m(0, 0));
    microtorch::save_safetensors(argv[2], t);
    return 0;
}
