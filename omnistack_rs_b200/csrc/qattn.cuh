// Declarations shared by the decode-attention translation units.
#pragma once
#include "common.cuh"

namespace omni {

struct AttnArgs {
    const void* q; int q_dtype;
    const uint8_t* k_nib; const uint8_t* k_qjl; const float* k_norms; const uint8_t* v_nib;
    const float* codebooks; int cb_per_head;
    const int32_t* user_ids; int32_t user_id;
    const int32_t* seq_lens; const int32_t* cache_slots;
    int64_t B; int Hq, Hkv, T; int64_t S; int64_t ks_b, ks_h;
    float scale; int with_qjl, rotate_q, unrotate_out; int n_splits;
    float* ws; float* out; const uint32_t* g_rows;
    int32_t* status;           // device word set non-zero when a bounded wait expires (may be null)
    uint32_t* work_counter;    // kWorkCounterBytes of device memory behind the split-K partials: one ticket counter
                               // per kv head for the tensor-core kernel (null: items are assigned statically)
    int v_paired;              // V nibble rows are stored pair-wise (see omni_v_pair_groups): within every group of eight
                               // keys that lies completely below the user's length, the rows of keys (0,3), (1,2), (4,7),
                               // (5,6) hold the even-d / odd-d nibbles of both keys instead of one key's 128 nibbles each
    uint32_t* qprep;           // tensor-core kernel, split-K calls: device scratch for the prepared query operands of every
                               // (user, kv head, tile of 8 query columns), kPrepBytesPerUnit each (null: every work item
                               // builds its own)
    int only_if_wide;          // lane-per-key kernel: 1 = run only when the codebooks are outside the fp16 table's
                               // range (it then completes a call whose tensor-core launch stood down), 0 = always
};

// The tensor-core kernel dequantises through a table of fp16 centroid pairs.  fp16 rounds a centroid by at most
// 2^-9 = 1.95e-3 while |c| < 8 (1e-3 below 4, where Lloyd-Max codebooks of rotated unit-variance data lie) and by
// up to 3.9e-3 from 8 on, which a 3e-3 output budget cannot absorb; codebooks with a centroid of magnitude 8 or
// more, infinite or NaN ("wide") are served by the fp32 lane-per-key kernel instead.  Both kernels evaluate this
// same predicate on the device (over every codebook of the call), so the choice needs no host copy and cannot go
// stale.
constexpr float kFp16CentroidLimit = 8.0f;
__device__ __forceinline__ bool centroid_is_wide(float c) { return !(fabsf(c) < kFp16CentroidLimit); }

// Factor the fp16 centroid tables are built with.  fp16 spacing relative to the value is smallest just below a power
// of two, so the codebook is scaled to put its largest magnitude there (2.73 -> 3.996 for the Lloyd-Max codebook of
// unit-variance data: the largest centroids round by 6.7e-4 instead of 9.8e-4; 4.6 -> 7.99: 1.1e-3 instead of
// 1.95e-3).  The factor is taken back out of the scores through the query scale and out of the output row at the end.
__device__ __forceinline__ float lut_scale_of(const float* cb) {
    float m = 0.f;
#pragma unroll
    for (int c = 0; c < 16; ++c) m = fmaxf(m, fabsf(__ldg(cb + c)));
    if (!(m > 1e-30f) || !(m < kFp16CentroidLimit)) return 1.f;
    return exp2f(ceilf(log2f(m))) * (1.f - 1.f / 1024.f) / m;
}

constexpr int kWsStride = 132;     // floats per split-K partial: 128 accumulators, max, sum, 2 pad
constexpr size_t kWorkCounterBytes = 4096;   // kSeeds (the most kv heads a call may have) 32-bit counters
constexpr size_t kPrepBytesPerUnit = 32 * 4 * 32;   // prepared query operands of one work item: 32 words per lane

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, m));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(kFullMask, v, m);
    return v;
}

// Tensor-core kernel (qattn_mma.cu): shapes it covers, and its launcher.
bool mma_eligible(const AttnArgs& a);
int32_t launch_mma(const AttnArgs& a, cudaStream_t st);
// tcgen05 kernel (qattn_umma.cu): kv heads with many query columns, V rows in the reference layout.
bool umma_eligible(const AttnArgs& a);
int32_t launch_umma(const AttnArgs& a, cudaStream_t st);
// One-warp kernel that lets a bounded mbarrier wait run out on purpose (nothing arrives on its barrier).
int32_t launch_wait_probe(uint32_t limit, int32_t* status, cudaStream_t st);

}  // namespace omni
