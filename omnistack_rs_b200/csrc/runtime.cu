// Library life cycle, error reporting and the MT19937-derived Rademacher tables.
#include "common.cuh"
#include <mutex>
#include <string>
#include <vector>
#include <cstring>
#include <algorithm>

namespace omni {

static thread_local std::string g_last_error;
static std::mutex g_mutex;
static DeviceTables g_tables[kMaxDevices];
static std::vector<uint32_t> g_host_rows;     // [1024][64][4]
static std::vector<uint64_t> g_host_cols;     // [1024][128]

int32_t set_error(int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int32_t check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return OMNI_OK;
    return set_error(OMNI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// MT19937 (Matsumoto & Nishimura 1998) seeded with init_genrand(seed): the engine of
// torch's CPU generator.  torch.randint(0, 2, (64,128)) consumes one 32-bit output per
// element and keeps its lowest bit (kernels/quantize.py:410-414 in the reference).
namespace {
struct Mt19937 {
    uint32_t mt[624];
    int idx;
    explicit Mt19937(uint32_t seed) {
        mt[0] = seed;
        for (int i = 1; i < 624; ++i) mt[i] = 1812433253u * (mt[i - 1] ^ (mt[i - 1] >> 30)) + (uint32_t)i;
        idx = 624;
    }
    void refill() {
        for (int i = 0; i < 624; ++i) {
            uint32_t y = (mt[i] & 0x80000000u) | (mt[(i + 1) % 624] & 0x7fffffffu);
            mt[i] = mt[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
        }
        idx = 0;
    }
    uint32_t next() {
        if (idx >= 624) refill();
        uint32_t y = mt[idx++];
        y ^= y >> 11;
        y ^= (y << 7) & 0x9d2c5680u;
        y ^= (y << 15) & 0xefc60000u;
        y ^= y >> 18;
        return y;
    }
};

// G of one seed in both layouts: rows[64][4] (bit d of projection i -> word d/32, bit d%32) and
// cols[128] (bit i of entry d); both must be zero on entry.
void fill_seed(uint32_t seed, uint32_t* rows, uint64_t* cols) {
    Mt19937 gen(seed);
    for (int i = 0; i < kQjlDim; ++i)
        for (int d = 0; d < kHeadDim; ++d) {
            uint32_t bit = gen.next() & 1u;
            rows[i * 4 + (d >> 5)] |= bit << (d & 31);
            cols[d] |= (uint64_t)bit << i;
        }
}

void build_host_tables_locked() {
    if (!g_host_rows.empty()) return;
    g_host_rows.assign((size_t)kSeeds * kQjlDim * 4, 0u);
    g_host_cols.assign((size_t)kSeeds * kHeadDim, 0ull);
    for (int seed = 0; seed < kSeeds; ++seed)
        fill_seed((uint32_t)seed, &g_host_rows[(size_t)seed * kQjlDim * 4], &g_host_cols[(size_t)seed * kHeadDim]);
}

// Seeds at or above 1,024 (the row-seeded codec reaches them once its row key passes 1,023): one aligned block
// of 1,024 seeds at a time lives in a second pair of device tables, filled on demand from the host generator.
struct ExtBlock {
    uint32_t* rows = nullptr;      // device [1024][64][4]
    uint64_t* cols = nullptr;      // device [1024][128]
    int64_t block = -1;            // seeds [1024 * block, 1024 * block + 1024) are (partly) resident
    std::vector<uint8_t> have;     // which seeds of the block have been uploaded
};
ExtBlock g_ext[kMaxDevices];
}  // namespace

int32_t extended_tables_for_block(int64_t block, const std::vector<int>& slots, DeviceTables* out) {
    int dev = -1;
    OMNI_CUDA(cudaGetDevice(&dev));
    OMNI_REQUIRE(dev >= 0 && dev < kMaxDevices, OMNI_ERR_ARG, "device index %d out of range", dev);
    OMNI_REQUIRE(block >= 1 && block < (1ll << 22), OMNI_ERR_UNSUPPORTED, "row keys beyond 2^32 are not supported");
    std::lock_guard<std::mutex> lk(g_mutex);
    ExtBlock& e = g_ext[dev];
    if (!e.rows) {
        OMNI_CUDA(cudaMalloc(&e.rows, (size_t)kSeeds * kQjlDim * 4 * sizeof(uint32_t)));
        OMNI_CUDA(cudaMalloc(&e.cols, (size_t)kSeeds * kHeadDim * sizeof(uint64_t)));
    }
    bool synced = false;
    if (e.block != block) {
        // kernels of an earlier call may still read the previous block
        OMNI_CUDA(cudaDeviceSynchronize());
        synced = true;
        e.block = block;
        e.have.assign(kSeeds, 0);
    }
    std::vector<uint32_t> rows((size_t)kQjlDim * 4);
    std::vector<uint64_t> cols((size_t)kHeadDim);
    bool uploaded = false;
    for (int j : slots) {
        if (j < 0 || j >= kSeeds || e.have[j]) continue;
        if (!synced) { OMNI_CUDA(cudaDeviceSynchronize()); synced = true; }
        std::fill(rows.begin(), rows.end(), 0u);
        std::fill(cols.begin(), cols.end(), 0ull);
        fill_seed((uint32_t)(block * kSeeds + j), rows.data(), cols.data());
        OMNI_CUDA(cudaMemcpy(e.rows + (size_t)j * kQjlDim * 4, rows.data(), rows.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
        OMNI_CUDA(cudaMemcpy(e.cols + (size_t)j * kHeadDim, cols.data(), cols.size() * sizeof(uint64_t), cudaMemcpyHostToDevice));
        e.have[j] = 1;
        uploaded = true;
    }
    // copies from pageable memory may return before the data has landed, and a caller's non-blocking stream is not
    // ordered behind them: wait for the device before a kernel may use the tables
    if (uploaded) OMNI_CUDA(cudaDeviceSynchronize());
    out->rows = e.rows;
    out->cols = e.cols;
    return OMNI_OK;
}

const uint32_t* host_rows_table() {
    std::lock_guard<std::mutex> lk(g_mutex);
    build_host_tables_locked();
    return g_host_rows.data();
}

const DeviceTables* tables_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error(OMNI_ERR_CUDA, "cudaGetDevice failed or device index out of range");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_mutex);
    if (!g_tables[dev].rows) {
        set_error(OMNI_ERR_NOT_INIT, "omni_init(%d) has not been called", dev);
        return nullptr;
    }
    return &g_tables[dev];
}

}  // namespace omni

using namespace omni;

extern "C" int32_t omni_abi_version(void) { return 3; }

extern "C" const char* omni_last_error(void) { return g_last_error.c_str(); }

extern "C" int32_t omni_gtable_host(uint32_t* out, int32_t seed_begin, int32_t seed_count) {
    OMNI_REQUIRE(out != nullptr, OMNI_ERR_ARG, "omni_gtable_host: out is NULL");
    OMNI_REQUIRE(seed_begin >= 0 && seed_count >= 0 && seed_begin + seed_count <= kSeeds, OMNI_ERR_ARG,
                 "omni_gtable_host: seed range [%d, %d) outside [0, %d)", seed_begin, seed_begin + seed_count, kSeeds);
    const uint32_t* rows = host_rows_table();
    memcpy(out, rows + (size_t)seed_begin * kQjlDim * 4, (size_t)seed_count * kQjlDim * 4 * sizeof(uint32_t));
    return OMNI_OK;
}

extern "C" int32_t omni_init(int32_t device) {
    OMNI_REQUIRE(device >= 0 && device < kMaxDevices, OMNI_ERR_ARG, "omni_init: device %d out of range", device);
    int count = 0;
    OMNI_CUDA(cudaGetDeviceCount(&count));
    OMNI_REQUIRE(device < count, OMNI_ERR_ARG, "omni_init: device %d but only %d CUDA devices", device, count);
    std::lock_guard<std::mutex> lk(g_mutex);
    if (g_tables[device].rows) return OMNI_OK;
    build_host_tables_locked();
    int prev = 0;
    OMNI_CUDA(cudaGetDevice(&prev));
    OMNI_CUDA(cudaSetDevice(device));
    uint32_t* rows = nullptr;
    uint64_t* cols = nullptr;
    cudaError_t e = cudaMalloc(&rows, g_host_rows.size() * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&cols, g_host_cols.size() * sizeof(uint64_t));
    if (e == cudaSuccess) e = cudaMemcpy(rows, g_host_rows.data(), g_host_rows.size() * sizeof(uint32_t), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(cols, g_host_cols.data(), g_host_cols.size() * sizeof(uint64_t), cudaMemcpyHostToDevice);
    // pageable copies may return once staged; a non-blocking stream is not ordered behind them: wait for the device
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (rows) cudaFree(rows);
        if (cols) cudaFree(cols);
        cudaSetDevice(prev);
        return check_cuda(e, "omni_init: table upload");
    }
    g_tables[device].rows = rows;
    g_tables[device].cols = cols;
    OMNI_CUDA(cudaSetDevice(prev));
    return OMNI_OK;
}

extern "C" int32_t omni_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_mutex);
    int prev = 0;
    cudaGetDevice(&prev);
    for (int d = 0; d < kMaxDevices; ++d) {
        if (!g_tables[d].rows) continue;
        if (cudaSetDevice(d) == cudaSuccess) {
            cudaFree(g_tables[d].rows);
            cudaFree(g_tables[d].cols);
        }
        g_tables[d] = DeviceTables();
    }
    for (int d = 0; d < kMaxDevices; ++d) {
        if (!g_ext[d].rows && !g_ext[d].cols) continue;
        if (cudaSetDevice(d) == cudaSuccess) {
            cudaFree(g_ext[d].rows);
            cudaFree(g_ext[d].cols);
        }
        g_ext[d] = ExtBlock();
    }
    cudaSetDevice(prev);
    return OMNI_OK;
}
