// Per-user low-rank query update (the reference's LoRA-Q prologue).
//   q_eff[b,h,t,:] = q[b,h,t,:] + alpha * reshape((x[b,t,:] A[idx_b]^T) B[idx_b]^T)[h,:],  idx_b >= 0
//   q_eff[b] = q[b] exactly                                                                  idx_b <  0
// An index at or past the number of adapters leaves the row unchanged too and raises the status word to
// OMNI_STATUS_BAD_INDEX, so the host needs no synchronising range check before the launch.
// The attention kernels apply the same update inside their prologues (LoraFold in qattn.cuh); this kernel serves
// omni_lora_q and the calls whose attention kernel takes no folded update.
// One CTA of 1024 threads per (user, token).  Down projection: the warps take the `rank` rows of A in turn and
// reduce over the hidden axis (lora_down_row, shared with the folded form so that both agree bit for bit).  Up
// projection: a thread owns output elements o, o + 1024, ... and reads its rows of B as 16-byte vectors; those
// loads do not depend on the down projection and are issued before the barrier that publishes it.  fp32 throughout.
#include "common.cuh"
#include "qattn.cuh"

namespace omni {

constexpr int kLoraThreads = 1024;
constexpr int kLoraWarps = kLoraThreads / 32;
constexpr int kLoraMaxRank = 128;

template <int DT>
__device__ __forceinline__ float load_q(const void* q, int64_t i) {
    if (DT == OMNI_F32) return reinterpret_cast<const float*>(q)[i];
    if (DT == OMNI_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[i]);
    return __half2float(reinterpret_cast<const __half*>(q)[i]);
}

template <int DT>
__global__ void __launch_bounds__(kLoraThreads) lora_q_kernel(const void* q, const float* x, const float* la, const float* lb,
                                                             const int32_t* idx, int n_adapters, float alpha, int Hq, int T,
                                                             int hidden, int rank, float* out, int32_t* status) {
    __shared__ float down[kLoraMaxRank];
    const int b = blockIdx.x / T, t = blockIdx.x % T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_out = Hq * kHeadDim;
    int32_t li = idx[b];
    if (li >= n_adapters) {
        if (status && threadIdx.x == 0) atomicMax(status, OMNI_STATUS_BAD_INDEX);
        li = -1;
    }
    if (li < 0) {                                           // no adapter: q passes through bit for bit
        for (int o = threadIdx.x; o < n_out; o += kLoraThreads) {
            const int64_t qi = (((int64_t)b * Hq + o / kHeadDim) * T + t) * kHeadDim + o % kHeadDim;
            out[qi] = load_q<DT>(q, qi);
        }
        return;
    }
    const float* xr = x + ((int64_t)b * T + t) * hidden;
    const float* a = la + (int64_t)li * rank * hidden;
    for (int r = warp; r < rank; r += kLoraWarps) {
        const float acc = lora_down_row(xr, a + (int64_t)r * hidden, hidden, lane);
        if (lane == 0) down[r] = acc;
    }
    const float* bm = lb + (int64_t)li * n_out * rank;
    const bool vec = (rank % 4 == 0) && ((reinterpret_cast<uintptr_t>(lb) & 15) == 0);
    for (int o0 = 0; o0 < n_out; o0 += kLoraThreads) {
        const int o = o0 + threadIdx.x;
        const bool live = o < n_out;
        const int64_t qi = live ? (((int64_t)b * Hq + o / kHeadDim) * T + t) * kHeadDim + o % kHeadDim : 0;
        float qv = live ? load_q<DT>(q, qi) : 0.f;
        const float* br = bm + (int64_t)(live ? o : 0) * rank;
        float4 first = make_float4(0.f, 0.f, 0.f, 0.f);
        if (vec && live) first = *reinterpret_cast<const float4*>(br);   // in flight across the barrier below
        if (o0 == 0) __syncthreads();
        if (!live) continue;
        float up = 0.f;
        if (vec) {
            up = fmaf(down[0], first.x, up); up = fmaf(down[1], first.y, up);
            up = fmaf(down[2], first.z, up); up = fmaf(down[3], first.w, up);
            for (int r = 4; r < rank; r += 4) {
                const float4 w = *reinterpret_cast<const float4*>(br + r);
                up = fmaf(down[r], w.x, up); up = fmaf(down[r + 1], w.y, up);
                up = fmaf(down[r + 2], w.z, up); up = fmaf(down[r + 3], w.w, up);
            }
        } else {
            for (int r = 0; r < rank; ++r) up = fmaf(down[r], br[r], up);
        }
        out[qi] = fmaf(up, alpha, qv);
    }
}

}  // namespace omni

using namespace omni;

extern "C" int32_t omni_lora_q(const void* q, int32_t q_dtype, const float* x, const float* lora_a, const float* lora_b,
                               const int32_t* lora_indices, int32_t n_adapters, float lora_alpha, int64_t B, int32_t Hq,
                               int32_t T, int32_t hidden, int32_t rank, float* out, int32_t* status_word, void* stream) {
    OMNI_REQUIRE(B >= 0 && Hq > 0 && T >= 0 && hidden > 0 && rank > 0 && n_adapters >= 0, OMNI_ERR_ARG, "omni_lora_q: bad extent");
    OMNI_REQUIRE(rank <= kLoraMaxRank, OMNI_ERR_UNSUPPORTED, "omni_lora_q: rank %d exceeds %d", rank, kLoraMaxRank);
    if (B == 0 || T == 0) return OMNI_OK;
    OMNI_REQUIRE(q && x && lora_a && lora_b && lora_indices && out, OMNI_ERR_ARG, "omni_lora_q: NULL buffer");
    OMNI_REQUIRE(B * T <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED, "omni_lora_q: too many (user, token) pairs");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)(B * T);
    switch (q_dtype) {
        case OMNI_F32:  lora_q_kernel<OMNI_F32><<<grid, kLoraThreads, 0, st>>>(q, x, lora_a, lora_b, lora_indices, n_adapters, lora_alpha, Hq, T, hidden, rank, out, status_word); break;
        case OMNI_BF16: lora_q_kernel<OMNI_BF16><<<grid, kLoraThreads, 0, st>>>(q, x, lora_a, lora_b, lora_indices, n_adapters, lora_alpha, Hq, T, hidden, rank, out, status_word); break;
        case OMNI_F16:  lora_q_kernel<OMNI_F16><<<grid, kLoraThreads, 0, st>>>(q, x, lora_a, lora_b, lora_indices, n_adapters, lora_alpha, Hq, T, hidden, rank, out, status_word); break;
        default: return set_error(OMNI_ERR_ARG, "omni_lora_q: unknown dtype code %d", q_dtype);
    }
    return check_cuda(cudaGetLastError(), "lora_q_kernel launch");
}
