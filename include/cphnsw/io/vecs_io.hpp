// fvecs / ivecs files (the SIFT-1M / GIST-1M distribution format) for the evaluation programs
// that feed the index: same layout and the same reading rules as the reference's loaders
// (evaluation/datasets/dataset_loader.hpp:40-108): every record is a little-endian int32 length
// followed by that many 4-byte values; the length of the FIRST record is the dimension of the
// file, the record count is file_size / record_size (a trailing partial record is ignored) and
// later length fields are read but not checked.
// Header-only, host-only; no dependency on the GPU library.
#pragma once

#include <cmath>
#include <cstdint>
#include <fstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace cphnsw {
namespace io {

namespace detail {
template <class T>
inline std::vector<T> load_vecs(const std::string& path, size_t& dim, size_t& count, size_t max_count) {
    static_assert(sizeof(T) == 4, "fvecs / ivecs hold 4-byte values");
    std::ifstream file(path, std::ios::binary);
    if (!file) throw std::runtime_error("Cannot open file: " + path);  // dataset_loader.hpp:42-44
    int32_t d = 0;
    file.read(reinterpret_cast<char*>(&d), sizeof(int32_t));
    if (!file || d <= 0) throw std::runtime_error("Not an fvecs/ivecs file (bad first length): " + path);
    dim = size_t(d);
    file.seekg(0, std::ios::end);
    const size_t file_size = size_t(file.tellg());
    const size_t record = sizeof(int32_t) + dim * 4;
    count = file_size / record;
    if (max_count && count > max_count) count = max_count;
    std::vector<T> data(count * dim);
    file.seekg(0, std::ios::beg);
    // whole records are read in blocks and the length fields dropped while copying
    const size_t block = 4096;
    std::vector<char> buf(block * record);
    for (size_t i = 0; i < count; i += block) {
        const size_t m = count - i < block ? count - i : block;
        file.read(buf.data(), std::streamsize(m * record));
        if (!file) throw std::runtime_error("Short read: " + path);
        for (size_t j = 0; j < m; ++j)
            std::char_traits<char>::copy(reinterpret_cast<char*>(data.data() + (i + j) * dim), buf.data() + j * record + 4, dim * 4);
    }
    return data;
}

template <class T>
inline void save_vecs(const std::string& path, const T* data, size_t count, size_t dim) {
    static_assert(sizeof(T) == 4, "fvecs / ivecs hold 4-byte values");
    std::ofstream file(path, std::ios::binary);
    if (!file) throw std::runtime_error("Cannot create file: " + path);
    const int32_t d = int32_t(dim);
    for (size_t i = 0; i < count; ++i) {
        file.write(reinterpret_cast<const char*>(&d), 4);
        file.write(reinterpret_cast<const char*>(data + i * dim), std::streamsize(dim * 4));
    }
    if (!file) throw std::runtime_error("Write failed: " + path);
}
}  // namespace detail

// float[count][dim] row-major; max_count = 0 reads everything
inline std::vector<float> load_fvecs(const std::string& path, size_t& dim, size_t& count, size_t max_count = 0) {
    return detail::load_vecs<float>(path, dim, count, max_count);
}

// uint32[count][k] row-major (ground-truth neighbour ids; the reference returns one vector per row)
inline std::vector<uint32_t> load_ivecs(const std::string& path, size_t& k, size_t& count, size_t max_count = 0) {
    return detail::load_vecs<uint32_t>(path, k, count, max_count);
}

inline void save_fvecs(const std::string& path, const float* data, size_t count, size_t dim) {
    detail::save_vecs<float>(path, data, count, dim);
}
inline void save_ivecs(const std::string& path, const uint32_t* data, size_t count, size_t k) {
    detail::save_vecs<uint32_t>(path, data, count, k);
}

// in-place L2 normalisation of every row, the rule of the reference's normalize_vectors
// (evaluation/datasets/dataset_loader.hpp:225-240): squared norm accumulated in fp32 in d order,
// rows of norm <= 1e-10 left as they are, every coordinate multiplied by 1.0f / norm
inline void normalize_rows(float* data, size_t count, size_t dim) {
    for (size_t i = 0; i < count; ++i) {
        float* v = data + i * dim;
        float norm_sq = 0;
        for (size_t d = 0; d < dim; ++d) norm_sq += v[d] * v[d];
        const float norm = std::sqrt(norm_sq);
        if (norm > 1e-10f) {
            const float inv = 1.0f / norm;
            for (size_t d = 0; d < dim; ++d) v[d] *= inv;
        }
    }
}

}  // namespace io
}  // namespace cphnsw
