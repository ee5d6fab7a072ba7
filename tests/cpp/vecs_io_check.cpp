// Round trip of include/cphnsw/io/vecs_io.hpp for tests/test_vecs_io.py:
//   vecs_io_check read  <fvecs|ivecs> <path>            -> prints "dim count" and every value as a 32-bit hex word
//   vecs_io_check write <fvecs|ivecs> <path> <count> <dim>  -> writes value(i, d) = i * 1000 + d (float or uint32)
//   vecs_io_check norm  <path-in> <path-out>            -> fvecs in, rows normalised, fvecs out
#include <cstdio>
#include <cstring>
#include <string>

#include "cphnsw/io/vecs_io.hpp"

int main(int argc, char** argv) {
    using namespace cphnsw::io;
    try {
        if (argc >= 4 && !std::strcmp(argv[1], "read")) {
            size_t dim = 0, count = 0;
            if (!std::strcmp(argv[2], "fvecs")) {
                auto v = load_fvecs(argv[3], dim, count);
                std::printf("%zu %zu\n", dim, count);
                for (float f : v) {
                    uint32_t u;
                    std::memcpy(&u, &f, 4);
                    std::printf("%08x\n", u);
                }
            } else {
                auto v = load_ivecs(argv[3], dim, count);
                std::printf("%zu %zu\n", dim, count);
                for (uint32_t u : v) std::printf("%08x\n", u);
            }
            return 0;
        }
        if (argc >= 6 && !std::strcmp(argv[1], "write")) {
            const size_t count = std::stoul(argv[4]), dim = std::stoul(argv[5]);
            if (!std::strcmp(argv[2], "fvecs")) {
                std::vector<float> v(count * dim);
                for (size_t i = 0; i < count; ++i)
                    for (size_t d = 0; d < dim; ++d) v[i * dim + d] = float(i * 1000 + d);
                save_fvecs(argv[3], v.data(), count, dim);
            } else {
                std::vector<uint32_t> v(count * dim);
                for (size_t i = 0; i < count; ++i)
                    for (size_t d = 0; d < dim; ++d) v[i * dim + d] = uint32_t(i * 1000 + d);
                save_ivecs(argv[3], v.data(), count, dim);
            }
            return 0;
        }
        if (argc >= 4 && !std::strcmp(argv[1], "norm")) {
            size_t dim = 0, count = 0;
            auto v = load_fvecs(argv[2], dim, count);
            normalize_rows(v.data(), count, dim);
            save_fvecs(argv[3], v.data(), count, dim);
            return 0;
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 2;
    }
    std::fprintf(stderr, "usage: see the head of vecs_io_check.cpp\n");
    return 1;
}
