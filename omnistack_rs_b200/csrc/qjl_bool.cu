// Unpacked QJL residual coding (the reference's quantization/qjl.py: `RademacherQJL.encode` :78-104,
// `reconstruct` :106-135): one bool per projection instead of packed sign bytes, G chosen by an explicit seed.
//   encode:       signs[r][i] = (sum_d G[i][d] * e[r][d] >= 0),  norms[r] = ||e[r]||_2
//   reconstruct:  out[r][d]   = (sum_i b[r][i] * G[i][d]) * (norms[r] * sqrt(2/pi) / 128),  b = 2 * signs - 1
// A warp takes a row.  Projections are accumulated in fp64 (the exact sign; the reference's fp32 product can
// differ only where its own rounding order decides the bit); the reconstruction sum is an exact integer.
#include "common.cuh"

namespace omni {

constexpr int kQbWarps = 8;

__global__ void __launch_bounds__(kQbWarps * 32) qjl_encode_bool_kernel(const float* err, int64_t n_rows, const uint32_t* g_rows_seed,
                                                                       uint8_t* signs, float* norms) {
    __shared__ float row[kQbWarps][kHeadDim];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t r = (int64_t)blockIdx.x * kQbWarps + warp; r < n_rows; r += (int64_t)gridDim.x * kQbWarps) {
        const float4 v = *reinterpret_cast<const float4*>(err + r * kHeadDim + 4 * lane);
        *reinterpret_cast<float4*>(&row[warp][4 * lane]) = v;
        float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(kFullMask, ss, m);
        __syncwarp();
        // lane owns projections lane and lane + 32
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int i = lane + 32 * half;
            const uint4 gw = __ldg(reinterpret_cast<const uint4*>(g_rows_seed + i * 4));
            const uint32_t w[4] = {gw.x, gw.y, gw.z, gw.w};
            double acc = 0.0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll 8
                for (int k = 0; k < 32; ++k) {
                    const double e = (double)row[warp][32 * q + k];
                    acc += ((w[q] >> k) & 1u) ? e : -e;
                }
            }
            signs[r * kQjlDim + i] = acc >= 0.0 ? 1 : 0;
        }
        if (lane == 0) norms[r] = sqrtf(ss);
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kQbWarps * 32) qjl_reconstruct_bool_kernel(const uint8_t* signs, const float* norms, int64_t n_rows,
                                                                            const uint64_t* g_cols_seed, float* out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t r = (int64_t)blockIdx.x * kQbWarps + warp; r < n_rows; r += (int64_t)gridDim.x * kQbWarps) {
        const uint32_t lo = __ballot_sync(kFullMask, signs[r * kQjlDim + lane] != 0);
        const uint32_t hi = __ballot_sync(kFullMask, signs[r * kQjlDim + 32 + lane] != 0);
        const uint64_t sig = ((uint64_t)hi << 32) | lo;
        const float coef = __fmul_rn(norms[r], kQjlCoef);
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int sum = kQjlDim - 2 * __popcll(sig ^ __ldg(g_cols_seed + 4 * lane + k));   // matches minus mismatches
            v[k] = __fmul_rn((float)sum, coef);
        }
        *reinterpret_cast<float4*>(out + r * kHeadDim + 4 * lane) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

static int qb_grid(int64_t n_rows) {
    int64_t blocks = (n_rows + kQbWarps - 1) / kQbWarps;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace omni

using namespace omni;

extern "C" int32_t omni_qjl_encode_bool(const float* err, int64_t n_rows, int32_t seed, uint8_t* signs, float* norms, void* stream) {
    OMNI_REQUIRE(n_rows >= 0, OMNI_ERR_ARG, "omni_qjl_encode_bool: n_rows < 0");
    OMNI_REQUIRE(seed >= 0 && seed < kSeeds, OMNI_ERR_UNSUPPORTED, "omni_qjl_encode_bool: seed %d outside the %d-seed table", seed, kSeeds);
    if (n_rows == 0) return OMNI_OK;
    OMNI_REQUIRE(err && signs && norms && reinterpret_cast<uintptr_t>(err) % 16 == 0, OMNI_ERR_ARG,
                 "omni_qjl_encode_bool: NULL or misaligned buffer");
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    qjl_encode_bool_kernel<<<qb_grid(n_rows), kQbWarps * 32, 0, (cudaStream_t)stream>>>(
        err, n_rows, tb->rows + (size_t)seed * kQjlDim * 4, signs, norms);
    return check_cuda(cudaGetLastError(), "qjl_encode_bool_kernel launch");
}

extern "C" int32_t omni_qjl_reconstruct_bool(const uint8_t* signs, const float* norms, int64_t n_rows, int32_t seed, float* out,
                                             void* stream) {
    OMNI_REQUIRE(n_rows >= 0, OMNI_ERR_ARG, "omni_qjl_reconstruct_bool: n_rows < 0");
    OMNI_REQUIRE(seed >= 0 && seed < kSeeds, OMNI_ERR_UNSUPPORTED, "omni_qjl_reconstruct_bool: seed %d outside the %d-seed table", seed, kSeeds);
    if (n_rows == 0) return OMNI_OK;
    OMNI_REQUIRE(signs && norms && out && reinterpret_cast<uintptr_t>(out) % 16 == 0, OMNI_ERR_ARG,
                 "omni_qjl_reconstruct_bool: NULL or misaligned buffer");
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    qjl_reconstruct_bool_kernel<<<qb_grid(n_rows), kQbWarps * 32, 0, (cudaStream_t)stream>>>(
        signs, norms, n_rows, tb->cols + (size_t)seed * kHeadDim, out);
    return check_cuda(cudaGetLastError(), "qjl_reconstruct_bool_kernel launch");
}
