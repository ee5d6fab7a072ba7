// One index over several GPUs of one box, behind the C ABI: one process, one replica handle per
// device, NCCL between them.
//
// Build (add_batch_parallel): rows are split into contiguous blocks, one per device.  Every device
// uploads and encodes its block; the code blocks are exchanged (NCCL all-gather; grouped broadcasts
// when the blocks are not all equal) so that every device holds all n codes; every device computes
// the kNN rows and the pruned adjacency rows of its block against them; the adjacency blocks and the
// vector blocks are exchanged the same way and every device installs the complete index.  Search: the
// query batch is split across the devices, every replica answers its share, nothing is exchanged.
// Every exchanged block is in the device's own memory before a kernel reads it: no kernel of this
// library ever reads peer memory.
//
// NCCL is loaded at run time (libnccl.so.2) and only when more than one device is used.
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "common.cuh"

namespace cpb {
namespace {

// The handful of NCCL entry points used, declared here so that building the library needs no NCCL header.
typedef struct ncclComm* ncclComm_t;
constexpr int kNcclUint8 = 1;  // ncclDataType_t: ncclUint8
struct Nccl {
    void* lib = nullptr;
    int (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

int load_nccl(Nccl& n) {
    static std::mutex mu;
    static Nccl loaded;
    std::lock_guard<std::mutex> lock(mu);
    if (!loaded.lib) {
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) {
            set_error("more than one GPU needs NCCL and libnccl.so.2 could not be loaded: %s", dlerror());
            return CPHNSW_B200_E_UNSUPPORTED;
        }
        Nccl t;
        t.lib = lib;
        t.CommInitAll = reinterpret_cast<decltype(t.CommInitAll)>(dlsym(lib, "ncclCommInitAll"));
        t.CommDestroy = reinterpret_cast<decltype(t.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
        t.AllGather = reinterpret_cast<decltype(t.AllGather)>(dlsym(lib, "ncclAllGather"));
        t.Broadcast = reinterpret_cast<decltype(t.Broadcast)>(dlsym(lib, "ncclBroadcast"));
        t.GroupStart = reinterpret_cast<decltype(t.GroupStart)>(dlsym(lib, "ncclGroupStart"));
        t.GroupEnd = reinterpret_cast<decltype(t.GroupEnd)>(dlsym(lib, "ncclGroupEnd"));
        t.GetErrorString = reinterpret_cast<decltype(t.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
        if (!t.CommInitAll || !t.CommDestroy || !t.AllGather || !t.Broadcast || !t.GroupStart || !t.GroupEnd) {
            set_error("libnccl.so.2 lacks an entry point this library needs");
            return CPHNSW_B200_E_UNSUPPORTED;
        }
        loaded = t;
    }
    n = loaded;
    return 0;
}

void shard_range(uint64_t n, int g, int G, uint64_t* begin, uint64_t* end) {
    const uint64_t base = n / G, rem = n % G;
    *begin = g * base + (uint64_t(g) < rem ? g : rem);
    *end = *begin + base + (uint64_t(g) < rem ? 1 : 0);
}

constexpr int kShardedStages = CPHNSW_B200_SHARDED_STAGES;
enum { kShardedEncode = 0, kShardedGatherCodes, kShardedKnn, kShardedPrune, kShardedGatherAdjacency, kShardedInstall };

double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace
}  // namespace cpb

using namespace cpb;

struct cphnsw_b200_sharded {
    int G = 0;
    std::vector<int> devices;
    std::vector<cphnsw_b200_index*> h;      // one replica per device
    std::vector<cudaStream_t> streams;      // one stream per device for the exchanges
    std::vector<ncclComm_t> comms;
    Nccl nccl;
    std::mutex mu;                          // build calls exclude one another
    std::atomic<uint32_t> next_replica{0};  // single-query calls go round the replicas
    double stage_ms[kShardedStages] = {0, 0, 0, 0, 0, 0};
    ~cphnsw_b200_sharded() {
        for (size_t g = 0; g < comms.size(); ++g)
            if (comms[g]) nccl.CommDestroy(comms[g]);
        for (size_t g = 0; g < streams.size(); ++g)
            if (streams[g]) {
                cudaSetDevice(devices[g]);
                cudaStreamDestroy(streams[g]);
            }
        for (auto* x : h) cphnsw_b200_destroy(x);
    }
};

namespace {

// runs fn(g) for every device on a thread of its own; the first failure's code and message win
template <class F>
int per_device(cphnsw_b200_sharded* s, F fn) {
    if (s->G == 1) {  // nothing to run side by side: the calling thread does it
        CPB_CUDA(cudaSetDevice(s->devices[0]));
        return fn(0);
    }
    std::vector<int> rc(s->G, 0);
    std::vector<std::string> msg(s->G);
    std::vector<std::thread> th;
    for (int g = 0; g < s->G; ++g)
        th.emplace_back([&, g]() {
            rc[g] = cudaSetDevice(s->devices[g]) == cudaSuccess ? fn(g) : CPHNSW_B200_E_CUDA;
            if (rc[g] != 0) msg[g] = cphnsw_b200_last_error();  // the message lives on this thread
        });
    for (auto& t : th) t.join();
    for (int g = 0; g < s->G; ++g)
        if (rc[g] != 0) {
            set_error("device %d: %s", s->devices[g], msg[g].c_str());
            return rc[g];
        }
    return 0;
}

// Every device ends up with all row blocks of a [n][row_bytes] array whose own block it has filled in place.
// Equal blocks: one in-place all-gather; otherwise one broadcast per block, all in one NCCL group.
int exchange_blocks(cphnsw_b200_sharded* s, std::vector<unsigned char*>& bufs, uint64_t n, size_t row_bytes) {
    if (s->G == 1) return 0;
    const Nccl& nc = s->nccl;
    const bool equal = n % s->G == 0;
    int rc = nc.GroupStart();
    for (int g = 0; g < s->G && rc == 0; ++g) {
        if (equal) {
            const size_t count = size_t(n / s->G) * row_bytes;
            rc = nc.AllGather(bufs[g] + size_t(g) * count, bufs[g], count, kNcclUint8, s->comms[g], s->streams[g]);
        } else {
            for (int root = 0; root < s->G && rc == 0; ++root) {
                uint64_t b, e;
                shard_range(n, root, s->G, &b, &e);
                unsigned char* p = bufs[g] + size_t(b) * row_bytes;
                rc = nc.Broadcast(p, p, size_t(e - b) * row_bytes, kNcclUint8, root, s->comms[g], s->streams[g]);
            }
        }
    }
    const int rc2 = nc.GroupEnd();
    if (rc == 0) rc = rc2;
    if (rc != 0) {
        set_error("NCCL error %d (%s) while exchanging row blocks", rc, nc.GetErrorString ? nc.GetErrorString(rc) : "?");
        return CPHNSW_B200_E_CUDA;
    }
    for (int g = 0; g < s->G; ++g) {
        CPB_CUDA(cudaSetDevice(s->devices[g]));
        CPB_CUDA(cudaStreamSynchronize(s->streams[g]));
    }
    return 0;
}

// streams, communicators and one small rehearsal exchange: NCCL connects the peers and sets its channels up at the
// first collective of a communicator, which would otherwise be paid inside the first build
int init_exchange(cphnsw_b200_sharded* s) {
    const int G = s->G;
    s->streams.assign(G, nullptr);
    s->comms.assign(G, nullptr);
    for (int g = 0; g < G; ++g) {
        CPB_CUDA(cudaSetDevice(s->devices[g]));
        CPB_CUDA(cudaStreamCreateWithFlags(&s->streams[g], cudaStreamNonBlocking));
    }
    if (G == 1) return 0;
    CPB_TRY(load_nccl(s->nccl));
    const int rc = s->nccl.CommInitAll(s->comms.data(), G, s->devices.data());
    if (rc != 0) {
        set_error("ncclCommInitAll failed: %d (%s)", rc, s->nccl.GetErrorString ? s->nccl.GetErrorString(rc) : "?");
        for (auto& c : s->comms) c = nullptr;
        return CPHNSW_B200_E_CUDA;
    }
    std::vector<DevBuf> buf(G);
    std::vector<unsigned char*> p(G);
    for (uint64_t rows : {uint64_t(G) * 64, uint64_t(G) * 64 + 1}) {  // equal blocks (all-gather), unequal (broadcasts)
        for (int g = 0; g < G; ++g) {
            CPB_CUDA(cudaSetDevice(s->devices[g]));
            CPB_TRY(buf[g].reserve(rows * 64));
            CPB_CUDA(cudaMemset(buf[g].p, 0, rows * 64));
            p[g] = buf[g].as<unsigned char>();
        }
        CPB_TRY(exchange_blocks(s, p, rows, 64));
    }
    for (int g = 0; g < G; ++g) {
        CPB_CUDA(cudaSetDevice(s->devices[g]));
        buf[g].release();
    }
    return 0;
}

}  // namespace

extern "C" {

int cphnsw_b200_sharded_create(uint64_t dim, uint32_t K, uint32_t component_bytes, uint32_t M, uint32_t ef_construction,
                               uint64_t seed, int fht_convention, int binary_codes, int n_gpus, const int* devices,
                               cphnsw_b200_sharded** out) {
    if (!out) {
        set_error("sharded_create: out is null");
        return CPHNSW_B200_E_INVALID;
    }
    *out = nullptr;
    const int have = cphnsw_b200_device_count();
    if (n_gpus == 0) n_gpus = have;  // all visible sm_100 devices
    if (n_gpus < 1 || (have > 0 && n_gpus > have && !devices)) {
        set_error("sharded_create: n_gpus = %d but %d usable devices", n_gpus, have);
        return have == 0 ? CPHNSW_B200_E_CUDA : CPHNSW_B200_E_INVALID;
    }
    std::unique_ptr<cphnsw_b200_sharded> s(new cphnsw_b200_sharded());
    s->G = n_gpus;
    for (int g = 0; g < n_gpus; ++g) s->devices.push_back(devices ? devices[g] : g);
    for (int g = 0; g < n_gpus; ++g)
        for (int f = 0; f < g; ++f)
            if (s->devices[f] == s->devices[g]) {
                set_error("sharded_create: device %d listed twice", s->devices[g]);
                return CPHNSW_B200_E_INVALID;
            }
    for (int g = 0; g < n_gpus; ++g) {
        cphnsw_b200_index* h = nullptr;
        const int rc = binary_codes ? cphnsw_b200_create_binary(dim, K, M, ef_construction, seed, fht_convention, s->devices[g], &h)
                                    : cphnsw_b200_create(dim, K, component_bytes, M, ef_construction, seed, fht_convention,
                                                         s->devices[g], &h);
        if (rc != 0) return rc;
        s->h.push_back(h);
    }
    CPB_TRY(init_exchange(s.get()));
    *out = s.release();
    return 0;
}

int cphnsw_b200_sharded_load(const char* path, int n_gpus, const int* devices, cphnsw_b200_sharded** out) {
    if (!out || !path) {
        set_error("sharded_load: null argument");
        return CPHNSW_B200_E_INVALID;
    }
    *out = nullptr;
    const int have = cphnsw_b200_device_count();
    if (n_gpus == 0) n_gpus = have;
    if (n_gpus < 1) {
        set_error("sharded_load: no usable device");
        return CPHNSW_B200_E_CUDA;
    }
    std::unique_ptr<cphnsw_b200_sharded> s(new cphnsw_b200_sharded());
    s->G = n_gpus;
    for (int g = 0; g < n_gpus; ++g) s->devices.push_back(devices ? devices[g] : g);
    for (int g = 0; g < n_gpus; ++g) {
        cphnsw_b200_index* h = nullptr;
        CPB_TRY(cphnsw_b200_load(path, s->devices[g], &h));
        s->h.push_back(h);
    }
    CPB_TRY(init_exchange(s.get()));
    *out = s.release();
    return 0;
}

int cphnsw_b200_sharded_destroy(cphnsw_b200_sharded* s) {
    delete s;
    return 0;
}

int cphnsw_b200_sharded_gpus(const cphnsw_b200_sharded* s) { return s ? s->G : 0; }

cphnsw_b200_index* cphnsw_b200_sharded_replica(const cphnsw_b200_sharded* s, int g) {
    return (s && g >= 0 && g < s->G) ? s->h[g] : nullptr;
}

uint64_t cphnsw_b200_sharded_size(const cphnsw_b200_sharded* s) { return s ? cphnsw_b200_size(s->h[0]) : 0; }

int cphnsw_b200_sharded_set_param(cphnsw_b200_sharded* s, const char* name, double value) {
    if (!s) {
        set_error("null sharded index");
        return CPHNSW_B200_E_INVALID;
    }
    for (int g = 0; g < s->G; ++g) CPB_TRY(cphnsw_b200_set_param(s->h[g], name, value));
    return 0;
}

int cphnsw_b200_sharded_stage_times(const cphnsw_b200_sharded* s, double* ms_out) {
    if (!s || !ms_out) {
        set_error("sharded_stage_times: null argument");
        return CPHNSW_B200_E_INVALID;
    }
    std::memcpy(ms_out, s->stage_ms, sizeof(s->stage_ms));
    return 0;
}

int cphnsw_b200_sharded_add_batch_parallel(cphnsw_b200_sharded* s, const float* x, uint64_t n) {
    if (!s) {
        set_error("null sharded index");
        return CPHNSW_B200_E_INVALID;
    }
    if (n == 0) return 0;
    if (!x) {
        set_error("add_batch_parallel: null pointer");
        return CPHNSW_B200_E_INVALID;
    }
    std::lock_guard<std::mutex> lock(s->mu);
    const uint64_t old_n = cphnsw_b200_size(s->h[0]);
    double seeded = 0;
    cphnsw_b200_get_param(s->h[0], "build_seed", &seeded);
    if (s->G == 1 || old_n != 0 || seeded != 0 || s->h[0]->exact_edges || n < uint64_t(s->G) * 64) {
        // one device, an index that already holds nodes, a seeded build, links on exact distances or a handful of rows:
        // every replica does
        // the whole call (same input, same kernels: the replicas stay identical)
        return per_device(s, [&](int g) { return cphnsw_b200_add_batch_parallel(s->h[g], x, n); });
    }
    if (n >= 0x80000000ull) {
        set_error("add_batch_parallel: at most 2^31-1 nodes");
        return CPHNSW_B200_E_INVALID;
    }
    cphnsw_b200_index* h0 = s->h[0];
    const uint64_t dim = h0->dim;
    const size_t rb = size_t(h0->K) * h0->comp_bytes;
    const uint32_t M = h0->M;
    uint32_t k = h0->knn_k ? h0->knn_k : (2 * M < 64 ? 2 * M : 64);
    if (k < M) k = M;
    if (k > 64) k = 64;
    if (!h0->prune) k = M;
    const bool rank = h0->prune && h0->rank_prune;
    const int G = s->G;
    std::vector<DevBuf> vec(G), codes(G), adj(G), cand(G), kept(G);
    std::vector<unsigned char*> p_vec(G), p_codes(G), p_adj(G), p_cand(G), p_kept(G);
    double t0 = now_ms(), t1;
    auto lap = [&](int stage) {
        t1 = now_ms();
        s->stage_ms[stage] = t1 - t0;
        t0 = t1;
    };
    // ---- upload + encode of the own block, in place in the full-size arrays
    CPB_TRY(per_device(s, [&](int g) {
        uint64_t b, e;
        shard_range(n, g, G, &b, &e);
        CPB_TRY(vec[g].reserve(n * dim * 4));
        CPB_TRY(codes[g].reserve(n * rb + 16));
        CPB_TRY(adj[g].reserve(size_t(n) * M * 4 + 16));
        // with rank pruning the candidate lists of ALL nodes are needed on every device
        CPB_TRY(cand[g].reserve((rank ? size_t(n) : size_t(e - b)) * k * 4 + 16));
        if (rank) CPB_TRY(kept[g].reserve(size_t(n) * M * 4 + 16));
        p_vec[g] = vec[g].as<unsigned char>(), p_codes[g] = codes[g].as<unsigned char>(), p_adj[g] = adj[g].as<unsigned char>();
        p_cand[g] = cand[g].as<unsigned char>(), p_kept[g] = kept[g].as<unsigned char>();
        float* mine = vec[g].as<float>() + b * dim;
        CPB_CUDA(cudaMemcpyAsync(mine, x + b * dim, (e - b) * dim * 4, cudaMemcpyHostToDevice, s->streams[g]));
        CPB_TRY(cphnsw_b200_encode_dev(s->h[g], mine, e - b, p_codes[g] + b * rb, nullptr, nullptr, s->streams[g]));
        CPB_CUDA(cudaStreamSynchronize(s->streams[g]));
        return 0;
    }));
    lap(kShardedEncode);
    CPB_TRY(exchange_blocks(s, p_codes, n, rb));
    lap(kShardedGatherCodes);
    // ---- kNN rows of the own block against all codes
    CPB_TRY(per_device(s, [&](int g) {
        uint64_t b, e;
        shard_range(n, g, G, &b, &e);
        uint32_t* out = !h0->prune ? adj[g].as<uint32_t>() + b * M : cand[g].as<uint32_t>() + (rank ? b * k : 0);
        CPB_TRY(cphnsw_b200_knn_graph_dev(s->h[g], p_codes[g], n, k, b, e, out, nullptr, s->streams[g]));
        CPB_CUDA(cudaStreamSynchronize(s->streams[g]));
        return cphnsw_b200_check_device_status(s->h[g]);
    }));
    lap(kShardedKnn);
    // ---- pruning of the own rows
    if (h0->prune && !rank) {
        CPB_TRY(per_device(s, [&](int g) {
            uint64_t b, e;
            shard_range(n, g, G, &b, &e);
            CPB_TRY(cphnsw_b200_select_neighbors_dev(s->h[g], p_codes[g], n, cand[g].as<uint32_t>(), k, b, e, M, h0->keep_pruned,
                                                     adj[g].as<uint32_t>() + b * M, s->streams[g]));
            CPB_CUDA(cudaStreamSynchronize(s->streams[g]));
            return 0;
        }));
    } else if (rank) {
        CPB_TRY(exchange_blocks(s, p_cand, n, size_t(k) * 4));
        CPB_TRY(per_device(s, [&](int g) {
            uint64_t b, e;
            shard_range(n, g, G, &b, &e);
            CPB_TRY(cphnsw_b200_rank_reorder_dev(s->h[g], cand[g].as<uint32_t>(), n, k, b, e, M, h0->rank_pruning_alpha,
                                                 kept[g].as<uint32_t>() + b * M, s->streams[g]));
            CPB_CUDA(cudaStreamSynchronize(s->streams[g]));
            return 0;
        }));
        CPB_TRY(exchange_blocks(s, p_kept, n, size_t(M) * 4));
        CPB_TRY(per_device(s, [&](int g) {
            uint64_t b, e;
            shard_range(n, g, G, &b, &e);
            CPB_TRY(cphnsw_b200_rank_merge_dev(s->h[g], kept[g].as<uint32_t>(), n, M, b, e, adj[g].as<uint32_t>() + b * M,
                                               s->streams[g]));
            CPB_CUDA(cudaStreamSynchronize(s->streams[g]));
            return 0;
        }));
    }
    lap(kShardedPrune);
    CPB_TRY(exchange_blocks(s, p_adj, n, size_t(M) * 4));
    CPB_TRY(exchange_blocks(s, p_vec, n, size_t(dim) * 4));
    lap(kShardedGatherAdjacency);
    CPB_TRY(per_device(s, [&](int g) {
        return cphnsw_b200_install_dev(s->h[g], vec[g].as<float>(), p_codes[g], adj[g].as<uint32_t>(), n, s->streams[g]);
    }));
    lap(kShardedInstall);
    return 0;
}

int cphnsw_b200_sharded_add_batch(cphnsw_b200_sharded* s, const float* x, uint64_t n) {
    if (!s) {
        set_error("null sharded index");
        return CPHNSW_B200_E_INVALID;
    }
    if (n == 0) return 0;
    if (cphnsw_b200_size(s->h[0]) == 0) return cphnsw_b200_sharded_add_batch_parallel(s, x, n);
    std::lock_guard<std::mutex> lock(s->mu);
    return per_device(s, [&](int g) { return cphnsw_b200_add_batch(s->h[g], x, n); });
}

// mode 0 search, 1 search_and_rerank, 2 search_multiprobe (arg = num_probes), 3 brute force, 4 calibrated (arg = rerank_k)
int cphnsw_b200_sharded_search(cphnsw_b200_sharded* s, int mode, const float* q, uint64_t nq, uint32_t k, uint32_t ef,
                               uint32_t arg, uint32_t* ids_out, float* dists_out, uint32_t* stats_out) {
    if (!s) {
        set_error("null sharded index");
        return CPHNSW_B200_E_INVALID;
    }
    if (mode < 0 || mode > 4) {
        set_error("sharded_search: unknown mode %d", mode);
        return CPHNSW_B200_E_INVALID;
    }
    if (nq == 0) return 0;
    const uint64_t dim = s->h[0]->dim;
    auto one = [&](int g, uint64_t b, uint64_t e) -> int {
        cphnsw_b200_index* h = s->h[g];
        const float* qq = q + b * dim;
        uint32_t* oi = ids_out + b * k;
        float* od = dists_out + b * k;
        uint32_t* os = stats_out ? stats_out + b * 2 : nullptr;
        switch (mode) {
            case 0: return cphnsw_b200_search_batch(h, qq, e - b, k, ef, oi, od, os);
            case 1: return cphnsw_b200_search_and_rerank_batch(h, qq, e - b, k, ef, arg, oi, od, os);
            case 2: return cphnsw_b200_search_multiprobe_batch(h, qq, e - b, k, ef, arg, oi, od);
            case 3: return cphnsw_b200_brute_force_search_batch(h, qq, e - b, k, oi, od);
            default: return cphnsw_b200_search_calibrated_batch(h, qq, e - b, k, ef, arg, oi, od);
        }
    };
    if (!q || !ids_out || !dists_out) {
        set_error("search: query/output pointers must be non-null");
        return CPHNSW_B200_E_INVALID;
    }
    if (s->G == 1 || nq < uint64_t(s->G) * kNarrowQueries) {
        // a small batch goes to one replica whole; successive calls (from any thread) go round the replicas
        const int g = s->G == 1 ? 0 : int(s->next_replica.fetch_add(1) % uint32_t(s->G));
        return one(g, 0, nq);
    }
    return per_device(s, [&](int g) {
        uint64_t b, e;
        shard_range(nq, g, s->G, &b, &e);
        return one(g, b, e);
    });
}

}  // extern "C"
