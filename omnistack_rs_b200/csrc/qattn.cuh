// Declarations shared by the decode-attention translation units.
#pragma once
#include "common.cuh"

namespace omni {

// Per-user low-rank query update applied where a kernel loads its query rows (x == nullptr: none):
//   q_eff[b,h,t,:] = q[b,h,t,:] + alpha * reshape((x[b,t,:] A[idx_b]^T) B[idx_b]^T)[h,:]   for 0 <= idx_b < n_adapters,
//   q_eff[b] = q[b] bit for bit otherwise (an index at or past n_adapters also raises OMNI_STATUS_BAD_INDEX).
struct LoraFold {
    const float* x;            // (B, T, hidden)
    const float* a;            // (n_adapters, rank, hidden)
    const float* b;            // (n_adapters, Hq * 128, rank)
    const int32_t* idx;        // (B,)
    int n_adapters, hidden, rank;
    float alpha;
};
constexpr int kLoraFoldMaxRank = 128;

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
    LoraFold lora;             // query update folded into the prologue (warp-level and lane-per-key kernels)
    int2* user_order;          // warp-level kernel, split-K calls with per-user lengths: (user, clamped length) pairs with
                               // the longest caches first, written by the preparation launch; work items are numbered in
                               // this order, so the tickets hand out the long items first and the short ones fill the
                               // end of the launch (null: users in index order)
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
// Split-K workspace: partial states | ticket counters (kWorkCounterBytes) | user order | prepared query operands.
constexpr int64_t kMaxOrderedUsers = 16384;          // one CTA sorts them in the preparation launch
inline size_t user_order_bytes(int64_t B) { return B <= kMaxOrderedUsers ? (((size_t)B * 8) + 255) & ~(size_t)255 : 0; }
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

// One element of the down projection by one warp: the dot product of a token's hidden state and a row of A, the
// same value in every lane.  The separate update kernel (lora_q.cu) uses this function too, so the folded and the
// separate update agree bit for bit.
__device__ __forceinline__ float lora_down_row(const float* xr, const float* ar, int hidden, int lane) {
    const bool vec = (hidden % 128 == 0) && ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(ar)) & 15) == 0;
    float acc = 0.f;
    if (vec) {
        for (int k = 4 * lane; k < hidden; k += 128) {
            const float4 xv = __ldg(reinterpret_cast<const float4*>(xr + k));
            const float4 av = __ldg(reinterpret_cast<const float4*>(ar + k));
            acc = fmaf(xv.x, av.x, acc); acc = fmaf(xv.y, av.y, acc);
            acc = fmaf(xv.z, av.z, acc); acc = fmaf(xv.w, av.w, acc);
        }
    } else {
        for (int k = lane; k < hidden; k += 32) acc = fmaf(__ldg(xr + k), __ldg(ar + k), acc);
    }
    return warp_sum(acc);
}

// Down projection of the update for user b, token tq, by one warp: element r of x[b,tq,:] A^T ends in lane r & 31,
// register d[r >> 5].  Returns the user's adapter index, or -1 when the query stays as it is.
__device__ __forceinline__ int lora_down(const LoraFold& L, int64_t b, int T, int tq, int lane, float (&d)[4], int32_t* status) {
    d[0] = 0.f; d[1] = 0.f; d[2] = 0.f; d[3] = 0.f;
    int32_t li = __ldg(L.idx + b);
    if (li >= L.n_adapters) {
        if (status && lane == 0) atomicMax(status, OMNI_STATUS_BAD_INDEX);
        li = -1;
    }
    if (li < 0) return -1;
    const float* xr = L.x + (b * T + tq) * (int64_t)L.hidden;
    const float* am = L.a + (int64_t)li * L.rank * L.hidden;
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        if (32 * rr >= L.rank) break;
        const int nr = L.rank - 32 * rr < 32 ? L.rank - 32 * rr : 32;
#pragma unroll 8
        for (int r = 0; r < nr; ++r) {
            const float acc = lora_down_row(xr, am + (int64_t)(32 * rr + r) * L.hidden, L.hidden, lane);
            if (lane == r) d[rr] = acc;
        }
    }
    return li;
}

// Up projection for NC query rows at once: row c takes the four outputs whose rows of B start at br[c] (`rank`
// floats apart); `d` as lora_down left it.  The loads of all NC rows are independent, so more rows per call means
// more of them in flight.  Every lane of the warp calls this together.
template <int NC>
__device__ __forceinline__ void lora_up_rows(const LoraFold& L, const float* const (&br)[NC], const float (&d)[4], float (&up)[NC][4]) {
    const bool vec = (L.rank % 4 == 0) && (reinterpret_cast<uintptr_t>(L.b) & 15) == 0;
#pragma unroll
    for (int c = 0; c < NC; ++c) { up[c][0] = 0.f; up[c][1] = 0.f; up[c][2] = 0.f; up[c][3] = 0.f; }
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        if (32 * rr >= L.rank) break;
        const int nr = L.rank - 32 * rr < 32 ? L.rank - 32 * rr : 32;
        if (vec) {
#pragma unroll 4
            for (int r = 0; r < nr; r += 4) {
                float dv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) dv[j] = __shfl_sync(kFullMask, d[rr], r + j);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 w = __ldg(reinterpret_cast<const float4*>(br[c] + (int64_t)i * L.rank + 32 * rr + r));
                        up[c][i] = fmaf(dv[0], w.x, up[c][i]); up[c][i] = fmaf(dv[1], w.y, up[c][i]);
                        up[c][i] = fmaf(dv[2], w.z, up[c][i]); up[c][i] = fmaf(dv[3], w.w, up[c][i]);
                    }
                }
            }
        } else {
            for (int r = 0; r < nr; ++r) {
                const float dv = __shfl_sync(kFullMask, d[rr], r);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) up[c][i] = fmaf(dv, __ldg(br[c] + (int64_t)i * L.rank + 32 * rr + r), up[c][i]);
                }
            }
        }
    }
}

// The update of one query row (lane-per-key kernel): both steps, then q += alpha * up.
static __device__ __noinline__ void lora_fold_row(const LoraFold L, int64_t b, int T, int tq, int n_out, int o, int lane,
                                                  int32_t* status, float (&qv)[4]) {
    float d[4];
    const int adapter = lora_down(L, b, T, tq, lane, d, status);
    if (adapter < 0) return;
    const float* const br[1] = {L.b + ((int64_t)adapter * n_out + o) * L.rank};
    float up[1][4];
    lora_up_rows<1>(L, br, d, up);
#pragma unroll
    for (int i = 0; i < 4; ++i) qv[i] = fmaf(up[0][i], L.alpha, qv[i]);
}

// The common small case with every extent known at compile time, so that the loads of a step are all issued before
// the first of them is used (a warp working alone has nothing else to hide their latency): one token per user,
// hidden == 128, RANK <= 32 adapter rows, 16-byte aligned x / A / B.  Same operations in the same order as the general
// code below, hence the same bits.
template <int RANK>
__device__ __forceinline__ void lora_tile_small(const LoraFold& L, int adapter, int64_t b, int Hq, int hkv, int Gq, int col0,
                                                int ncols, int lane, float* rows) {
    constexpr int NC = RANK <= 16 ? 2 : 1;                       // columns per batch of loads
    const float4 xv = __ldg(reinterpret_cast<const float4*>(L.x + b * 128) + lane);
    const float4* am = reinterpret_cast<const float4*>(L.a + (int64_t)adapter * RANK * 128) + lane;
    float acc[RANK];
#pragma unroll
    for (int r = 0; r < RANK; ++r) {
        const float4 av = __ldg(am + r * 32);
        float v = 0.f;
        v = fmaf(xv.x, av.x, v); v = fmaf(xv.y, av.y, v); v = fmaf(xv.z, av.z, v); v = fmaf(xv.w, av.w, v);
        acc[r] = v;
    }
    float d = 0.f;
#pragma unroll
    for (int r = 0; r < RANK; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == r) d = v;
    }
    const float* bm = L.b + (int64_t)adapter * Hq * kHeadDim * RANK;
    for (int c = 0; c < ncols; c += NC) {
        float4 w[NC][4][RANK / 4];
        int col[NC];
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            col[n] = c + n < ncols ? c + n : ncols - 1;          // an odd tail repeats the last column
            const float4* br = reinterpret_cast<const float4*>(bm + ((int64_t)(hkv * Gq + col0 + col[n]) * kHeadDim + 4 * lane) * RANK);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int r4 = 0; r4 < RANK / 4; ++r4) w[n][i][r4] = __ldg(br + i * (RANK / 4) + r4);
            }
        }
        float up[NC][4];
#pragma unroll
        for (int n = 0; n < NC; ++n) { up[n][0] = 0.f; up[n][1] = 0.f; up[n][2] = 0.f; up[n][3] = 0.f; }
#pragma unroll
        for (int r4 = 0; r4 < RANK / 4; ++r4) {
            const float d0 = __shfl_sync(kFullMask, d, 4 * r4), d1 = __shfl_sync(kFullMask, d, 4 * r4 + 1);
            const float d2 = __shfl_sync(kFullMask, d, 4 * r4 + 2), d3 = __shfl_sync(kFullMask, d, 4 * r4 + 3);
#pragma unroll
            for (int n = 0; n < NC; ++n) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = up[n][i];
                    v = fmaf(d0, w[n][i][r4].x, v); v = fmaf(d1, w[n][i][r4].y, v);
                    v = fmaf(d2, w[n][i][r4].z, v); v = fmaf(d3, w[n][i][r4].w, v);
                    up[n][i] = v;
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NC; ++n)
            *reinterpret_cast<float4*>(rows + col[n] * 128 + 4 * lane) = make_float4(up[n][0], up[n][1], up[n][2], up[n][3]);
    }
}

// The update of a tile of query columns (warp-level kernel): the up projections of columns col0 .. col0 + ncols - 1
// of kv head hkv (column = (q head in group, token)) are left in `rows`, 128 floats per column, lane l holding
// elements 4l .. 4l+3 of each; the caller adds alpha times them to the query rows.  Returns false when the user has
// no adapter (rows untouched).  Kept out of line: the callers' main loops are register-bound, and this code inlined
// into them changed their allocation.
static __device__ __noinline__ bool lora_fold_tile(const LoraFold L, int64_t b, int T, int Hq, int hkv, int Gq, int col0, int ncols,
                                                   int lane, int32_t* status, float* rows) {
    if (T == 1 && L.hidden == 128 && (L.rank == 8 || L.rank == 16 || L.rank == 32) &&
        ((reinterpret_cast<uintptr_t>(L.x) | reinterpret_cast<uintptr_t>(L.a) | reinterpret_cast<uintptr_t>(L.b)) & 15) == 0) {
        int32_t li = __ldg(L.idx + b);
        if (li >= L.n_adapters) {
            if (status && lane == 0) atomicMax(status, OMNI_STATUS_BAD_INDEX);
            li = -1;
        }
        if (li < 0) return false;
        if (L.rank == 16) lora_tile_small<16>(L, li, b, Hq, hkv, Gq, col0, ncols, lane, rows);
        else if (L.rank == 8) lora_tile_small<8>(L, li, b, Hq, hkv, Gq, col0, ncols, lane, rows);
        else lora_tile_small<32>(L, li, b, Hq, hkv, Gq, col0, ncols, lane, rows);
        return true;
    }
    float d[4];
    int token = col0 % T;
    const int adapter = lora_down(L, b, T, token, lane, d, status);
    if (adapter < 0) return false;
    const float* bm = L.b + (int64_t)adapter * Hq * kHeadDim * L.rank;
    for (int c = 0; c < ncols; ++c) {
        const int cg = col0 + c;
        if (cg % T != token) {
            token = cg % T;
            lora_down(L, b, T, token, lane, d, nullptr);
        }
        const float* const br[1] = {bm + ((int64_t)(hkv * Gq + cg / T) * kHeadDim + 4 * lane) * L.rank};
        float up[1][4];
        lora_up_rows<1>(L, br, d, up);
        *reinterpret_cast<float4*>(rows + c * 128 + 4 * lane) = make_float4(up[0][0], up[0][1], up[0][2], up[0][3]);
    }
    return true;
}

// Tensor-core kernel (qattn_mma.cu): shapes it covers, and its launcher.
bool mma_eligible(const AttnArgs& a);
int32_t launch_mma(const AttnArgs& a, cudaStream_t st);
int32_t launch_mma_lora(const AttnArgs& a, cudaStream_t st);   // qattn_mma_lora.cu: the same kernels with a.lora applied
// tcgen05 kernel (qattn_umma.cu): kv heads with many query columns.
bool umma_eligible(const AttnArgs& a);
int32_t launch_umma(const AttnArgs& a, cudaStream_t st);
// One-warp kernel that lets a bounded mbarrier wait run out on purpose (nothing arrives on its barrier).
int32_t launch_wait_probe(uint32_t limit, int32_t* status, cudaStream_t st);

}  // namespace omni
