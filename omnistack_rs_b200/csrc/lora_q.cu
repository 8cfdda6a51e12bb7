// Per-user low-rank query update (the reference's LoRA-Q prologue).
//   q_eff[b,h,t,:] = q[b,h,t,:] + alpha * reshape((x[b,t,:] A[idx_b]^T) B[idx_b]^T)[h,:],  idx_b >= 0
//   q_eff[b] = q[b] exactly                                                                  idx_b <  0
// One CTA per (user, token): the rank-sized down projection is reduced by warps over the hidden
// axis, then every thread produces output elements with `rank` fused multiply-adds.  fp32 throughout.
#include "common.cuh"

namespace omni {

constexpr int kLoraThreads = 256;
constexpr int kLoraMaxRank = 128;

template <int DT>
__global__ void __launch_bounds__(kLoraThreads) lora_q_kernel(const void* q, const float* x, const float* la, const float* lb,
                                                             const int32_t* idx, float alpha, int Hq, int T, int hidden,
                                                             int rank, float* out) {
    __shared__ float down[kLoraMaxRank];
    const int b = blockIdx.x / T, t = blockIdx.x % T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int32_t li = idx[b];
    if (li >= 0) {
        const float* xr = x + ((int64_t)b * T + t) * hidden;
        const float* a = la + (int64_t)li * rank * hidden;
        for (int r = warp; r < rank; r += kLoraThreads / 32) {
            float acc = 0.f;
            for (int k = lane; k < hidden; k += 32) acc = fmaf(xr[k], a[(int64_t)r * hidden + k], acc);
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) acc += __shfl_xor_sync(kFullMask, acc, m);
            if (lane == 0) down[r] = acc;
        }
    }
    __syncthreads();
    const float* bm = li >= 0 ? lb + (int64_t)li * Hq * kHeadDim * rank : nullptr;
    for (int o = threadIdx.x; o < Hq * kHeadDim; o += kLoraThreads) {
        const int h = o / kHeadDim, d = o % kHeadDim;
        const int64_t qi = (((int64_t)b * Hq + h) * T + t) * kHeadDim + d;
        float qv;
        if (DT == OMNI_F32) qv = reinterpret_cast<const float*>(q)[qi];
        else if (DT == OMNI_BF16) qv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[qi]);
        else qv = __half2float(reinterpret_cast<const __half*>(q)[qi]);
        if (bm) {
            float up = 0.f;
            const float* br = bm + (int64_t)o * rank;
            for (int r = 0; r < rank; ++r) up = fmaf(down[r], br[r], up);
            qv = fmaf(up, alpha, qv);
        }
        out[qi] = qv;
    }
}

}  // namespace omni

using namespace omni;

extern "C" int32_t omni_lora_q(const void* q, int32_t q_dtype, const float* x, const float* lora_a, const float* lora_b,
                               const int32_t* lora_indices, float lora_alpha, int64_t B, int32_t Hq, int32_t T,
                               int32_t hidden, int32_t rank, float* out, void* stream) {
    OMNI_REQUIRE(B >= 0 && Hq > 0 && T >= 0 && hidden > 0 && rank > 0, OMNI_ERR_ARG, "omni_lora_q: bad extent");
    OMNI_REQUIRE(rank <= kLoraMaxRank, OMNI_ERR_UNSUPPORTED, "omni_lora_q: rank %d exceeds %d", rank, kLoraMaxRank);
    if (B == 0 || T == 0) return OMNI_OK;
    OMNI_REQUIRE(q && x && lora_a && lora_b && lora_indices && out, OMNI_ERR_ARG, "omni_lora_q: NULL buffer");
    OMNI_REQUIRE(B * T <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED, "omni_lora_q: too many (user, token) pairs");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)(B * T);
    switch (q_dtype) {
        case OMNI_F32:  lora_q_kernel<OMNI_F32><<<grid, kLoraThreads, 0, st>>>(q, x, lora_a, lora_b, lora_indices, lora_alpha, Hq, T, hidden, rank, out); break;
        case OMNI_BF16: lora_q_kernel<OMNI_BF16><<<grid, kLoraThreads, 0, st>>>(q, x, lora_a, lora_b, lora_indices, lora_alpha, Hq, T, hidden, rank, out); break;
        case OMNI_F16:  lora_q_kernel<OMNI_F16><<<grid, kLoraThreads, 0, st>>>(q, x, lora_a, lora_b, lora_indices, lora_alpha, Hq, T, hidden, rank, out); break;
        default: return set_error(OMNI_ERR_ARG, "omni_lora_q: unknown dtype code %d", q_dtype);
    }
    return check_cuda(cudaGetLastError(), "lora_q_kernel launch");
}
