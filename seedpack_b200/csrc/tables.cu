// IQ lattice tables: host-side construction and per-device installation.
//
// For each of the six lattices the quantisers need (a) the points as packed int8 coordinates,
// (b) a map from every code tuple to its point index, or to a neighbour list when the tuple is not
// a lattice point, and (c) the neighbour lists.  The construction follows iq2xs_init_impl /
// iq3xs_init_impl (ggml-quants.c:2854-3259, 3704-3903): for an off-lattice tuple, order all points
// by (squared distance, index) and keep those within the `nwant` smallest distinct distances.  Since
// the squared distance is a small integer, the order is produced by bucketing instead of sorting.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "quant_iq.cuh"

namespace sg {

#include "iq_grids.inc"

struct HostTable {
    int dim, bits, npoints, map_size, nwant;
    std::vector<uint64_t> grid64;     // dim == 8
    std::vector<uint32_t> grid32;     // dim == 4
    std::vector<int32_t> map;
    std::vector<uint16_t> nb;
};

static const struct { const uint16_t* packed; int n, dim, bits, map_size, nwant; } SPEC[6] = {
    {kGrid0, 256, 8, 2, 43692, 2},   // IQ2_XXS
    {kGrid1, 512, 8, 2, 43692, 2},   // IQ2_XS
    {kGrid2, 2048, 8, 2, 43692, 3},  // IQ1_S / IQ1_M
    {kGrid3, 1024, 8, 2, 43692, 1},  // IQ2_S
    {kGrid4, 256, 4, 3, 4096, 2},    // IQ3_XXS
    {kGrid5, 512, 4, 3, 4096, 3},    // IQ3_S
};

static void build_one(int which, HostTable& t) {
    const auto& s = SPEC[which];
    t.dim = s.dim; t.bits = s.bits; t.npoints = s.n; t.map_size = s.map_size; t.nwant = s.nwant;
    const int mask = (1 << s.bits) - 1;
    std::vector<int8_t> pts((size_t)s.n * s.dim);
    for (int k = 0; k < s.n; ++k)
        for (int i = 0; i < s.dim; ++i) pts[(size_t)k * s.dim + i] = (int8_t)(2 * ((s.packed[k] >> (s.bits * i)) & mask) + 1);
    if (s.dim == 8) { t.grid64.resize(s.n); memcpy(t.grid64.data(), pts.data(), pts.size()); }
    else            { t.grid32.resize(s.n); memcpy(t.grid32.data(), pts.data(), pts.size()); }
    t.map.assign(s.map_size, -1);
    for (int k = 0; k < s.n; ++k) t.map[s.packed[k]] = k;

    // pass 1: neighbour count per off-lattice tuple; pass 2: fill at prefix offsets
    const int maxd = s.dim * (2 * mask) * (2 * mask) + 1;
    std::vector<int> count(s.map_size, 0);
    auto scan = [&](int i, std::vector<int>& d2, std::vector<int>& hist, uint16_t* out) -> int {
        int8_t pos[8];
        for (int k = 0; k < s.dim; ++k) pos[k] = (int8_t)(2 * ((i >> (s.bits * k)) & mask) + 1);
        std::fill(hist.begin(), hist.end(), 0);
        for (int j = 0; j < s.n; ++j) {
            const int8_t* pg = &pts[(size_t)j * s.dim];
            int d = 0;
            for (int k = 0; k < s.dim; ++k) d += (pg[k] - pos[k]) * (pg[k] - pos[k]);
            d2[j] = d; ++hist[d];
        }
        // the nwant smallest distinct distances
        int levels = 0, limit = -1, n = 0;
        for (int d = 0; d < maxd && levels < s.nwant; ++d)
            if (hist[d]) { ++levels; limit = d; n += hist[d]; }
        if (out) {
            int o = 0;
            for (int d = 0; d <= limit; ++d) {
                if (!hist[d]) continue;
                for (int j = 0; j < s.n; ++j) if (d2[j] == d) out[o++] = (uint16_t)j;
            }
        }
        return n;
    };
    const unsigned nthreads = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
    auto parallel = [&](auto&& fn) {
        std::vector<std::thread> th;
        for (unsigned w = 0; w < nthreads; ++w)
            th.emplace_back([&, w] {
                std::vector<int> d2(s.n), hist(maxd);
                for (int i = (int)w; i < s.map_size; i += (int)nthreads) if (t.map[i] < 0) fn(i, d2, hist);
            });
        for (auto& x : th) x.join();
    };
    parallel([&](int i, std::vector<int>& d2, std::vector<int>& hist) { count[i] = scan(i, d2, hist, nullptr); });
    std::vector<int> offset(s.map_size, -1);
    int counter = 0;
    for (int i = 0; i < s.map_size; ++i) if (t.map[i] < 0) { offset[i] = counter; counter += 1 + count[i]; }
    t.nb.assign(counter, 0);
    parallel([&](int i, std::vector<int>& d2, std::vector<int>& hist) {
        t.nb[offset[i]] = (uint16_t)count[i];
        scan(i, d2, hist, &t.nb[offset[i] + 1]);
    });
    for (int i = 0; i < s.map_size; ++i) if (offset[i] >= 0) t.map[i] = -(offset[i] + 1);
}

static std::mutex g_mu;
static HostTable* g_host = nullptr;          // six tables, built once per process
static constexpr int MAX_DEV = 64;
static IqTables* g_dev[MAX_DEV] = {nullptr};
static const uint16_t* g_keys[MAX_DEV][6] = {{nullptr}};     // per lattice: one packed code tuple per point

static const HostTable* host_tables() {
    if (!g_host) {
        HostTable* h = new HostTable[6];
        for (int i = 0; i < 6; ++i) build_one(i, h[i]);
        g_host = h;
    }
    return g_host;
}

const IqTables* device_tables(int device) {
    if (device < 0 || device >= MAX_DEV) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    return g_dev[device];
}

bool tables_ready(int device) { return device_tables(device) != nullptr; }

// packed level tuple of every lattice point (2 bits x 8 or 3 bits x 4): what the QR coder calls grid keys
// (seedpack/qr.py:936-949)
const uint16_t* device_grid_keys(int device, int which) {
    if (device < 0 || device >= MAX_DEV || which < 0 || which >= 6) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    return g_keys[device][which];
}

}  // namespace sg

using namespace sg;

extern "C" int sg_tables_host(int which, int what, const void** h_ptr, size_t* h_bytes) {
    if (which < 0 || which >= 6 || what < 0 || what > 2 || !h_ptr || !h_bytes) return SG_ERR_ARG;
    std::lock_guard<std::mutex> lk(g_mu);
    const HostTable& t = host_tables()[which];
    if (what == 0) {
        if (t.dim == 8) { *h_ptr = t.grid64.data(); *h_bytes = t.grid64.size() * 8; }
        else            { *h_ptr = t.grid32.data(); *h_bytes = t.grid32.size() * 4; }
    } else if (what == 1) { *h_ptr = t.map.data(); *h_bytes = t.map.size() * 4; }
    else                  { *h_ptr = t.nb.data(); *h_bytes = t.nb.size() * 2; }
    return SG_OK;
}

extern "C" int sg_tables_install(int device, void* stream) {
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_dev[device]) return SG_OK;
    const HostTable* h = host_tables();
    cudaStream_t st = (cudaStream_t)stream;
    // one allocation holds every table, each part 256-byte aligned
    // part 4: the neighbour lists once more with every point index replaced by the point's packed levels (what a
    // search needs to measure a distance, and what it returns), padded so that vector reads may overrun a list
    constexpr size_t NBK_PAD = 64;
    size_t off = 0, offs[6][5];
    std::vector<uint16_t> nbk[6];
    for (int i = 0; i < 6; ++i) {
        nbk[i].assign(h[i].nb.size() + NBK_PAD, 0);
        for (size_t pos = 0; pos < h[i].nb.size();) {
            const size_t n = h[i].nb[pos];
            nbk[i][pos] = (uint16_t)n;
            for (size_t j = 1; j <= n; ++j) nbk[i][pos + j] = SPEC[i].packed[h[i].nb[pos + j]];
            pos += n + 1;
        }
        const size_t sz[5] = {h[i].dim == 8 ? h[i].grid64.size() * 8 : h[i].grid32.size() * 4, h[i].map.size() * 4, h[i].nb.size() * 2,
                              (size_t)SPEC[i].n * 2, nbk[i].size() * 2};
        for (int k = 0; k < 5; ++k) { offs[i][k] = off; off += (sz[k] + 255) / 256 * 256; }
    }
    uint8_t* base = nullptr;
    rc = cuda_ok(cudaMalloc(&base, off));
    if (rc != SG_OK) return rc;
    IqTables* t = new IqTables;
    for (int i = 0; i < 6 && rc == SG_OK; ++i) {
        const void* src[3] = {h[i].dim == 8 ? (const void*)h[i].grid64.data() : (const void*)h[i].grid32.data(), h[i].map.data(), h[i].nb.data()};
        const size_t sz[3] = {h[i].dim == 8 ? h[i].grid64.size() * 8 : h[i].grid32.size() * 4, h[i].map.size() * 4, h[i].nb.size() * 2};
        for (int k = 0; k < 3 && rc == SG_OK; ++k)
            rc = cuda_ok(cudaMemcpyAsync(base + offs[i][k], src[k], sz[k], cudaMemcpyHostToDevice, st));
        if (rc == SG_OK) rc = cuda_ok(cudaMemcpyAsync(base + offs[i][3], SPEC[i].packed, (size_t)SPEC[i].n * 2, cudaMemcpyHostToDevice, st));
        if (rc == SG_OK) rc = cuda_ok(cudaMemcpyAsync(base + offs[i][4], nbk[i].data(), nbk[i].size() * 2, cudaMemcpyHostToDevice, st));
        g_keys[device][i] = (const uint16_t*)(base + offs[i][3]);
        t->t[i].nbkeys = (const uint16_t*)(base + offs[i][4]);
        t->t[i].nb_size = (int)h[i].nb.size();
        t->t[i].map_size = SPEC[i].map_size;
        t->t[i].grid = base + offs[i][0];
        t->t[i].map = (const int*)(base + offs[i][1]);
        t->t[i].neighbours = (const uint16_t*)(base + offs[i][2]);
        t->t[i].keys = g_keys[device][i];
    }
    if (rc == SG_OK) rc = cuda_ok(cudaStreamSynchronize(st));
    if (rc != SG_OK) { cudaFree(base); delete t; for (int i = 0; i < 6; ++i) g_keys[device][i] = nullptr; return rc; }
    g_dev[device] = t;
    return SG_OK;
}
