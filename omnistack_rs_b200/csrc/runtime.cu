// Library life cycle, error reporting and the MT19937-derived Rademacher tables.
#include "common.cuh"
#include <mutex>
#include <string>
#include <vector>
#include <cstring>

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

void build_host_tables_locked() {
    if (!g_host_rows.empty()) return;
    g_host_rows.assign((size_t)kSeeds * kQjlDim * 4, 0u);
    g_host_cols.assign((size_t)kSeeds * kHeadDim, 0ull);
    for (int seed = 0; seed < kSeeds; ++seed) {
        Mt19937 gen((uint32_t)seed);
        uint32_t* rows = &g_host_rows[(size_t)seed * kQjlDim * 4];
        uint64_t* cols = &g_host_cols[(size_t)seed * kHeadDim];
        for (int i = 0; i < kQjlDim; ++i)
            for (int d = 0; d < kHeadDim; ++d) {
                uint32_t bit = gen.next() & 1u;
                rows[i * 4 + (d >> 5)] |= bit << (d & 31);
                cols[d] |= (uint64_t)bit << i;
            }
    }
}
}  // namespace

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

extern "C" int32_t omni_abi_version(void) { return 1; }

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
    cudaSetDevice(prev);
    return OMNI_OK;
}
