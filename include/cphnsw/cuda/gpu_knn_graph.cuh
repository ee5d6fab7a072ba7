// cphnsw::cuda::GPUKNNGraphBuilder and KNNEdgeList with the interface of the reference's
// (include/cphnsw/cuda/gpu_knn_graph.cuh:28-125), on the B200 library.  The reference builds the
// kNN graph under the fp32 cosine distance with cuBLAS; here the graph is built under the CP-code
// distance (number of differing code components), the metric the index is built and walked with:
// vectors are encoded (K rotations, ComponentT components) and the kNN kernel sweeps all pairs.
// Neighbours ascend by (distance, id), self loops never appear, rows are padded with 0xFFFFFFFF
// when N - 1 < k.  Header-only; plain C++ except build_device, which needs the CUDA runtime header.
#pragma once

#include <cstddef>
#include <cstdint>
#include <limits>
#include <utility>
#include <vector>

#if defined(__has_include)
#if __has_include(<cuda_runtime_api.h>)
#include <cuda_runtime_api.h>
#define CPHNSW_B200_HAVE_CUDART 1
#endif
#endif

#include "gpu_encoder.cuh"

namespace cphnsw {
namespace cuda {

template <typename ComponentT = uint8_t, size_t K = 32>
class CodeKNNGraphBuilder {
public:
    // k <= 64 neighbours per node
    CodeKNNGraphBuilder(size_t dim, size_t k, uint64_t seed = 42, int fht_convention = CPHNSW_B200_FHT_AVX512, int device = 0)
        : dim_(dim), k_(k) {
        detail::check(cphnsw_b200_create(dim, uint32_t(K), uint32_t(sizeof(ComponentT)), 1, 1, seed, fht_convention, device, &h_));
    }
    ~CodeKNNGraphBuilder() { cphnsw_b200_destroy(h_); }
    CodeKNNGraphBuilder(const CodeKNNGraphBuilder&) = delete;
    CodeKNNGraphBuilder& operator=(const CodeKNNGraphBuilder&) = delete;

    // h_vectors [N x dim] -> h_neighbors [N x k], h_distances [N x k] (optional; code distances as
    // floats, +inf where a row is padded).  The batch and tile sizes of the reference's signature are
    // accepted and ignored: the kernel tiles by itself.   (gpu_knn_graph.cuh:42-55)
    void build(const Float* h_vectors, size_t N, uint32_t* h_neighbors, Float* h_distances = nullptr, size_t /*query_batch_size*/ = 0,
               size_t /*base_tile_size*/ = 0) {
        std::vector<ComponentT> codes(N * K);
        detail::check(cphnsw_b200_encode(h_, h_vectors, N, codes.data()));
        std::vector<uint16_t> d(h_distances ? N * k_ : 0);
        detail::check(cphnsw_b200_knn_graph(h_, codes.data(), N, uint32_t(k_), 0, N, h_neighbors, h_distances ? d.data() : nullptr));
        widen(d, N, h_neighbors, h_distances);
    }

#ifdef CPHNSW_B200_HAVE_CUDART
    // the same with the vectors on the device, [N x dim]; outputs on the host   (gpu_knn_graph.cuh:57-63)
    void build_device(const Float* d_vectors, size_t N, uint32_t* h_neighbors, Float* h_distances = nullptr,
                      size_t /*query_batch_size*/ = 0, size_t /*base_tile_size*/ = 0) {
        if (N == 0) return;
        Scratch codes(N * K * sizeof(ComponentT)), nbrs(N * k_ * 4), dist(h_distances ? N * k_ * 2 : 0);
        detail::check(cphnsw_b200_encode_dev(h_, d_vectors, N, codes.p, nullptr, nullptr, nullptr));
        detail::check(cphnsw_b200_knn_graph_dev(h_, codes.p, N, uint32_t(k_), 0, N, static_cast<uint32_t*>(nbrs.p),
                                                static_cast<uint16_t*>(dist.p), nullptr));
        cuda_check(cudaMemcpy(h_neighbors, nbrs.p, N * k_ * 4, cudaMemcpyDeviceToHost));
        std::vector<uint16_t> d(h_distances ? N * k_ : 0);
        if (h_distances) cuda_check(cudaMemcpy(d.data(), dist.p, N * k_ * 2, cudaMemcpyDeviceToHost));
        detail::check(cphnsw_b200_check_device_status(h_));
        widen(d, N, h_neighbors, h_distances);
    }
#endif

    // gpu_knn_graph.cuh:65-70: nothing to tune here; the whole problem is one batch and one tile
    static void get_recommended_sizes(size_t N, size_t /*dim*/, size_t /*k*/, size_t /*available_memory_gb*/, size_t& query_batch,
                                      size_t& base_tile) {
        query_batch = N;
        base_tile = N;
    }

    size_t dim() const { return dim_; }
    size_t k() const { return k_; }

private:
    cphnsw_b200_index* h_ = nullptr;
    size_t dim_, k_;

    void widen(const std::vector<uint16_t>& d, size_t N, const uint32_t* h_neighbors, Float* h_distances) const {
        if (!h_distances) return;
        for (size_t i = 0; i < N * k_; ++i)
            h_distances[i] = h_neighbors[i] == CPHNSW_B200_INVALID_NODE ? std::numeric_limits<Float>::infinity() : Float(d[i]);
    }

#ifdef CPHNSW_B200_HAVE_CUDART
    static void cuda_check(cudaError_t e) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
    }
    struct Scratch {  // device memory for the length of one call
        void* p = nullptr;
        explicit Scratch(size_t bytes) {
            if (bytes) cuda_check(cudaMalloc(&p, bytes));
        }
        ~Scratch() { cudaFree(p); }
        Scratch(const Scratch&) = delete;
        Scratch& operator=(const Scratch&) = delete;
    };
#endif
};

// the reference's class name: uint8_t components, K = 32 rotations (its CPHNSWIndex8 configuration)
using GPUKNNGraphBuilder = CodeKNNGraphBuilder<uint8_t, 32>;

// Edge-list view of an N x k neighbour matrix (gpu_knn_graph.cuh:103-125): padded entries and self
// loops are dropped.
struct KNNEdgeList {
    std::vector<uint32_t> sources, targets;
    std::vector<float> distances;  // empty when built without distances
    size_t num_nodes = 0, k = 0;

    static KNNEdgeList from_matrix(const uint32_t* neighbors, const float* distances, size_t N, size_t k) {
        KNNEdgeList e;
        e.num_nodes = N, e.k = k;
        e.offsets_.assign(N + 1, 0);
        for (size_t i = 0; i < N; ++i) {
            for (size_t j = 0; j < k; ++j) {
                const uint32_t t = neighbors[i * k + j];
                if (t == CPHNSW_B200_INVALID_NODE || t == uint32_t(i)) continue;
                e.sources.push_back(uint32_t(i));
                e.targets.push_back(t);
                if (distances) e.distances.push_back(distances[i * k + j]);
            }
            e.offsets_[i + 1] = e.targets.size();
        }
        return e;
    }

    // (pointer to the node's targets, their count)
    std::pair<const uint32_t*, size_t> get_neighbors(uint32_t node_id) const {
        if (node_id >= num_nodes) return {nullptr, 0};
        return {targets.data() + offsets_[node_id], offsets_[node_id + 1] - offsets_[node_id]};
    }

private:
    std::vector<size_t> offsets_;
};

}  // namespace cuda
}  // namespace cphnsw
