#pragma once
// Host-side dense matrix: row-major float32. This is the type the tape exposes
// at its host boundary (parameter initialisation, state_dict, values read back
// by tests or bindings); the arithmetic of the training step never runs on it.
// Same surface as the matrix type the reference's tape is written against
// (rows(), cols(), operator()(i,j), data(), fill) so code written for the
// reference's Variable::data / ::grad reads unchanged. Like the reference's matrix type it
// lives in the global namespace (code written for the reference names it unqualified) and is
// also visible as microtorch::Matrix.
#include <cstddef>
#include <stdexcept>
#include <vector>

class Matrix {
public:
    Matrix() = default;
    Matrix(size_t rows, size_t cols, float init = 0.0f)
        : rows_(rows), cols_(cols), buf_(rows * cols, init) {}

    size_t rows() const { return rows_; }
    size_t cols() const { return cols_; }
    size_t size() const { return buf_.size(); }
    bool empty() const { return buf_.empty(); }

    float& operator()(size_t i, size_t j) { return buf_[index(i, j)]; }
    const float& operator()(size_t i, size_t j) const { return buf_[index(i, j)]; }

    float* data() { return buf_.data(); }
    const float* data() const { return buf_.data(); }
    float* get_data() { return buf_.data(); }
    const float* get_data() const { return buf_.data(); }

    void fill(float v) { buf_.assign(buf_.size(), v); }

    Matrix transpose() const {
        Matrix t(cols_, rows_);
        for (size_t i = 0; i < rows_; ++i)
            for (size_t j = 0; j < cols_; ++j) t.buf_[j * rows_ + i] = buf_[i * cols_ + j];
        return t;
    }

private:
    size_t index(size_t i, size_t j) const {
        if (i >= rows_ || j >= cols_) throw std::out_of_range("Matrix index out of range");
        return i * cols_ + j;
    }
    size_t rows_ = 0, cols_ = 0;
    std::vector<float> buf_;
};

namespace microtorch {
using ::Matrix;
}  // namespace microtorch
