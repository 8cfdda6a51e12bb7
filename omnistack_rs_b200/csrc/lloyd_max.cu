// Lloyd-Max fit of the 16-level codebooks on the GPU (the reference's offline calibration,
// quantization/codebook.py:64-108 `LloydMaxCalibrator.fit`, :148-172 `calibrate_per_group`).
//
// The reference assigns every sample to its nearest centroid (first-index argmin of |x - c| in fp32) and
// replaces each centroid by the mean of its samples, up to 300 times.  With the samples SORTED the cell of
// centroid c is a contiguous range of the array, so one iteration needs only the 15 cell boundaries (a binary
// search each, with the reference's own fp32 comparison as the predicate) and the range sums, which come from
// an fp64 prefix-sum array as a difference.  An iteration therefore costs 15 x log2(n) loads instead of a pass
// over n x 16 distances, and the whole loop (initialisation, iterations, convergence test, final sort) runs in
// one launch with one warp per group, without a host round trip.
//
// Means are formed in fp64 from the prefix sums and rounded to fp32 once; the reference sums in fp32 in an
// order its tensor library chooses, so codebooks agree with it to a few fp32 ulps, not bit for bit.
#include "common.cuh"

namespace omni {

constexpr int kScanThreads = 256;
constexpr int kScanPerThread = 32;
constexpr int kScanChunk = kScanThreads * kScanPerThread;   // samples per CTA of the prefix-sum kernels
constexpr int kLevels = 16;

__device__ __forceinline__ double warp_inclusive_scan(double v, int lane) {
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const double o = __shfl_up_sync(kFullMask, v, m);
        if (lane >= m) v += o;
    }
    return v;
}

// Inclusive scan of one value per thread over a CTA of kScanThreads; returns the CTA total through *total.
__device__ __forceinline__ double block_inclusive_scan(double v, double* total) {
    __shared__ double warp_tot[kScanThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_inclusive_scan(v, lane);
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    double before = 0.0, all = 0.0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
        if (w < warp) before += warp_tot[w];
        all += warp_tot[w];
    }
    __syncthreads();
    *total = all;
    return v + before;
}

// Pass 1: the fp64 sum of every chunk of kScanChunk samples.
__global__ void __launch_bounds__(kScanThreads) chunk_sums_kernel(const float* x, int64_t n, double* chunk_sum) {
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    double s = 0.0;
    for (int j = 0; j < kScanPerThread; ++j) {
        const int64_t i = base + (int64_t)j * kScanThreads + threadIdx.x;     // coalesced
        if (i < n) s += (double)x[i];
    }
    double total;
    block_inclusive_scan(s, &total);
    if (threadIdx.x == 0) chunk_sum[blockIdx.x] = total;
}

// Pass 2: exclusive scan of the chunk sums in place (one CTA; each thread owns a contiguous run).
__global__ void __launch_bounds__(kScanThreads) scan_chunk_sums_kernel(double* chunk_sum, int64_t n_chunks) {
    const int64_t per = (n_chunks + kScanThreads - 1) / kScanThreads;
    const int64_t lo = (int64_t)threadIdx.x * per;
    const int64_t hi = lo + per < n_chunks ? lo + per : n_chunks;
    double s = 0.0;
    for (int64_t i = lo; i < hi; ++i) s += chunk_sum[i];
    double total;
    const double incl = block_inclusive_scan(s, &total);
    double run = incl - s;
    for (int64_t i = lo; i < hi; ++i) {
        const double v = chunk_sum[i];
        chunk_sum[i] = run;
        run += v;
    }
}

// Pass 3: prefix[i] = sum of x[0..i) for i in [0, n]; a thread owns kScanPerThread consecutive samples.
__global__ void __launch_bounds__(kScanThreads) write_prefix_kernel(const float* x, int64_t n, const double* chunk_off,
                                                                   double* prefix) {
    const int64_t first = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanPerThread;
    float v[kScanPerThread];
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        v[j] = first + j < n ? x[first + j] : 0.f;
        s += (double)v[j];
    }
    double total;
    double run = chunk_off[blockIdx.x] + block_inclusive_scan(s, &total) - s;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        if (first + j <= n) prefix[first + j] = run;
        run += (double)v[j];
    }
}

// The reference's assignment: index of the first smallest |x - c| over the 16 centroids, in fp32.
__device__ __forceinline__ int nearest_level(float x, const float* cent) {
    float best = fabsf(x - cent[0]);
    int idx = 0;
#pragma unroll
    for (int k = 1; k < kLevels; ++k) {
        const float d = fabsf(x - cent[k]);
        if (d < best) { best = d; idx = k; }
    }
    return idx;
}

// One warp per group.  Lane c < 16 owns centroid c and the upper boundary of its cell.
__global__ void __launch_bounds__(32) lloyd_max_kernel(const float* sorted, const double* prefix, const int64_t* group_off,
                                                      int max_iters, double tol, float* codebooks, int32_t* iters_out) {
    __shared__ float cent[kLevels];
    __shared__ long long bound[kLevels + 1];
    const int g = blockIdx.x, lane = threadIdx.x;
    const int64_t lo = group_off[g], hi = group_off[g + 1], n = hi - lo;
    const int64_t per = n / kLevels;
    // equal-mass initialisation: the mean of each sixteenth of the sorted sample
    if (lane < kLevels) {
        const int64_t a = lo + lane * per, b = a + per;
        cent[lane] = (float)((prefix[b] - prefix[a]) / (double)per);
    }
    if (lane == 0) bound[0] = lo;
    __syncwarp();
    int steps = 0;
    for (int64_t span = n; span > 0; span >>= 1) ++steps;      // enough halvings for a range of n + 1 positions
    int it = 0;
    for (; it < max_iters; ++it) {
        // boundary of cell c: the first position whose sample is assigned to a level above c (monotone in x
        // because the centroids are in ascending order)
        if (lane < kLevels) {
            int64_t a = lo, b = hi;                              // answer in [a, b]
            if (lane < kLevels - 1) {
                for (int s = 0; s < steps && a < b; ++s) {
                    const int64_t mid = a + ((b - a) >> 1);
                    if (nearest_level(sorted[mid], cent) > lane) b = mid; else a = mid + 1;
                }
            } else {
                a = hi;
            }
            bound[lane + 1] = a;
        }
        __syncwarp();
        float mine = 0.f, moved = 0.f;
        if (lane < kLevels) {
            const int64_t a = bound[lane], b = bound[lane + 1];
            mine = cent[lane];
            if (b > a) {                                         // an empty cell keeps its centroid
                const float fresh = (float)((prefix[b] - prefix[a]) / (double)(b - a));
                moved = fabsf(fresh - mine);
                mine = fresh;
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) moved = fmaxf(moved, __shfl_xor_sync(kFullMask, moved, m));
        __syncwarp();
        if (lane < kLevels) cent[lane] = mine;
        __syncwarp();
        if ((double)moved < tol) { ++it; break; }
    }
    if (lane == 0) {
        for (int i = 1; i < kLevels; ++i) {                      // ascending order for the codec's search
            const float v = cent[i];
            int j = i - 1;
            while (j >= 0 && cent[j] > v) { cent[j + 1] = cent[j]; --j; }
            cent[j + 1] = v;
        }
        if (iters_out) iters_out[g] = it;
    }
    __syncwarp();
    if (lane < kLevels) codebooks[(int64_t)g * kLevels + lane] = cent[lane];
}

static int64_t n_chunks_of(int64_t n) { return (n + 1 + kScanChunk - 1) / kScanChunk; }
static size_t prefix_bytes(int64_t n) { return (((size_t)(n + 1) * sizeof(double)) + 255) & ~(size_t)255; }

}  // namespace omni

using namespace omni;

extern "C" size_t omni_lloyd_max_workspace_bytes(int64_t n_total) {
    if (n_total <= 0) return 0;
    return prefix_bytes(n_total) + (size_t)n_chunks_of(n_total) * sizeof(double);
}

extern "C" int32_t omni_lloyd_max_fit(const float* sorted, int64_t n_total, const int64_t* group_offsets, int32_t n_groups,
                                      int32_t max_iters, double tol, void* workspace, size_t workspace_bytes,
                                      float* codebooks, int32_t* iters_out, void* stream) {
    OMNI_REQUIRE(n_groups >= 0 && n_total >= 0 && max_iters >= 0, OMNI_ERR_ARG, "omni_lloyd_max_fit: bad extent");
    if (n_groups == 0) return OMNI_OK;
    OMNI_REQUIRE(sorted && group_offsets && codebooks && workspace, OMNI_ERR_ARG, "omni_lloyd_max_fit: NULL buffer");
    OMNI_REQUIRE(n_total >= (int64_t)n_groups * kLevels, OMNI_ERR_ARG,
                 "omni_lloyd_max_fit: every group needs at least %d samples", kLevels);
    OMNI_REQUIRE(workspace_bytes >= omni_lloyd_max_workspace_bytes(n_total) && reinterpret_cast<uintptr_t>(workspace) % 8 == 0, OMNI_ERR_ARG,
                 "omni_lloyd_max_fit: workspace of %zu bytes needed, got %zu", omni_lloyd_max_workspace_bytes(n_total),
                 workspace_bytes);
    const int64_t chunks = n_chunks_of(n_total);
    OMNI_REQUIRE(chunks <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED, "omni_lloyd_max_fit: too many samples for one grid");
    cudaStream_t st = (cudaStream_t)stream;
    double* prefix = (double*)workspace;
    double* chunk_sum = (double*)((char*)workspace + prefix_bytes(n_total));
    chunk_sums_kernel<<<(unsigned)chunks, kScanThreads, 0, st>>>(sorted, n_total, chunk_sum);
    scan_chunk_sums_kernel<<<1, kScanThreads, 0, st>>>(chunk_sum, chunks);
    write_prefix_kernel<<<(unsigned)chunks, kScanThreads, 0, st>>>(sorted, n_total, chunk_sum, prefix);
    lloyd_max_kernel<<<(unsigned)n_groups, 32, 0, st>>>(sorted, prefix, group_offsets, max_iters, tol, codebooks, iters_out);
    return check_cuda(cudaGetLastError(), "lloyd_max kernels launch");
}
