#pragma once
// safetensors files: 8-byte little-endian header length, a JSON header
// {name: {"dtype", "shape", "data_offsets"}}, then the raw little-endian tensor bytes.
// Same two functions, signatures and file layout as the reference
// (include/microtorch/safetensors.hpp:20-28, src/safetensors.cpp:12-94), so a file written by
// either side loads on the other; the loader here additionally accepts BF16 tensors (the
// reference's loader is F32-only, src/safetensors.cpp:40-44) and widens them to fp32.
#include <map>
#include <string>

#include "microtorch/matrix.hpp"

namespace microtorch {

// Every F32 / BF16 tensor as a Matrix: [n] -> [1, n], [r, c] -> [r, c], scalars -> [1, 1].
// Tensors of rank > 2 are skipped and listed in `skipped` (name -> "rank N"), a leading
// "transformer." is stripped from names, "__metadata__" is ignored -- the reference's rules.
std::map<std::string, Matrix> load_safetensors(const std::string& path,
                                               std::map<std::string, std::string>* skipped = nullptr);

// F32, every Matrix as [rows, cols], tensors laid out in the map's (sorted) order, the header
// padded with spaces to a multiple of 8 bytes: identical dicts give byte-identical files.
void save_safetensors(const std::string& path, const std::map<std::string, Matrix>& tensors);

}  // namespace microtorch
