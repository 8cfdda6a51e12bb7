// Shared host/device helpers of the omni_b200 library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <vector>
#include "../../include/omni_b200.h"

namespace omni {

constexpr int kHeadDim = OMNI_HEAD_DIM;
constexpr int kQjlDim = OMNI_QJL_DIM;
constexpr int kNibBytes = OMNI_NIB_BYTES;
constexpr int kQjlBytes = OMNI_QJL_BYTES;
constexpr int kSeeds = OMNI_N_SEEDS;
constexpr int kMaxDevices = 16;
constexpr unsigned kFullMask = 0xffffffffu;

// fp32 value of 1/sqrt(128): the single multiply that ends the rotation.
#define OMNI_WHT_SCALE_BITS 0x3DB504F3u
// fp32 value of sqrt(2/pi)/128: the QJL reconstruction coefficient.
constexpr float kQjlCoef = (float)(0.7978845608028654 / 128.0);

// Per-device Rademacher tables (device memory owned by the library).
//   rows : [1024 seeds][64 projections][4 words]  bit d of projection i -> word d/32, bit d%32
//   cols : [1024 seeds][128 dims] uint64          bit i of entry d = G[i][d]
struct DeviceTables {
    uint32_t* rows = nullptr;
    uint64_t* cols = nullptr;
};

const DeviceTables* tables_for_current_device();   // nullptr (and error set) if not initialised
const uint32_t* host_rows_table();                 // host copy, built on first use
// Tables of the aligned seed block [1024 * block, 1024 * block + 1024), block >= 1, with at least the seeds
// 1024 * block + j for j in `slots` filled in (generated on the host and uploaded on demand; one block is resident
// per device at a time, and switching blocks synchronises the device).
int32_t extended_tables_for_block(int64_t block, const std::vector<int>& slots, DeviceTables* out);

int32_t set_error(int32_t code, const char* fmt, ...);
int32_t check_cuda(cudaError_t e, const char* what);

#define OMNI_CUDA(call)                                         \
    do {                                                        \
        int32_t _st = ::omni::check_cuda((call), #call);        \
        if (_st != OMNI_OK) return _st;                         \
    } while (0)

#define OMNI_REQUIRE(cond, code, ...)                           \
    do {                                                        \
        if (!(cond)) return ::omni::set_error((code), __VA_ARGS__); \
    } while (0)

// ---- device helpers ----------------------------------------------------------

// 128-point normalised Walsh-Hadamard transform of one row spread over a warp:
// lane l holds elements 4l..4l+3.  Stage order h = 1, 2, 4, ..., 64, every add and
// subtract rounded to fp32 on its own, one final multiply -- the reference order.
__device__ __forceinline__ void wht128_warp(float (&v)[4], int lane) {
    float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]);
    float a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a0, a2); v[2] = __fsub_rn(a0, a2);
    v[1] = __fadd_rn(a1, a3); v[3] = __fsub_rn(a1, a3);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool lower = (lane & m) != 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float o = __shfl_xor_sync(kFullMask, v[k], m);
            v[k] = lower ? __fsub_rn(o, v[k]) : __fadd_rn(v[k], o);
        }
    }
    const float s = __uint_as_float(OMNI_WHT_SCALE_BITS);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __fmul_rn(v[k], s);
}

// Load 4 consecutive elements of a row as fp32 (lane-owned quarter of a 16-float group).
template <int DT> struct Elem;
template <> struct Elem<OMNI_F32> {
    using T = float;
    static __device__ __forceinline__ void load4(const void* p, int64_t i, float (&v)[4]) {
        float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store4(void* p, int64_t i, const float (&v)[4]) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct Elem<OMNI_BF16> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ void load4(const void* p, int64_t i, float (&v)[4]) {
        uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
        v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
        v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store4(void* p, int64_t i, const float (&v)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&lo);
        t.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = t;
    }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Elem<OMNI_F16> {
    using T = __half;
    static __device__ __forceinline__ void load4(const void* p, int64_t i, float (&v)[4]) {
        uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p) + i);
        __half2 lo = *reinterpret_cast<__half2*>(&t.x), hi = *reinterpret_cast<__half2*>(&t.y);
        float2 a = __half22float2(lo), b = __half22float2(hi);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store4(void* p, int64_t i, const float (&v)[4]) {
        __half2 lo = __floats2half2_rn(v[0], v[1]);
        __half2 hi = __floats2half2_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&lo);
        t.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p) + i) = t;
    }
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};

__device__ __forceinline__ int seed_of(int32_t user_id, int head) { return ((user_id & 1023) ^ head) & 1023; }

}  // namespace omni
