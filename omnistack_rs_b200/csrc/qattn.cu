// Fused attention over the packed INT4 + QJL cache: the general CUDA-core kernel (small calls and the calls that
// fold the rotation into q / out), the split-K merge, kernel selection and the C entry points.  The tensor-core
// kernel that serves every larger call is in qattn_mma.cu.
//
// Work unit: one warp per (user, query head, query token, key split).  Lane l walks
// keys l, l+32, ... of its split with a private online-softmax state (max, sum, 128
// accumulators); nothing crosses lanes until the final merge.  K and V are dequantised
// in registers by a 16-entry codebook lookup in shared memory (16 words occupy 16
// distinct banks, so any access pattern is conflict-free).  The QJL part of K is
// applied as a score correction  norm * c * sum_i s_i (q . g_i)  with the 64 values
// (q . g_i) computed once per work unit -- the same algebra as the reference kernel
// (kernels/fused_attention.py:198-213, 260-276) but with G seeded per (user, kv head)
// exactly as the codec does (kernels/quantize.py:583), which is what the reference's
// CPU path (kernels/fused_attention.py:435-466) computes.
#include "qattn.cuh"
#include <mutex>
#include <cstdlib>

namespace omni {

constexpr int kAttnWarps = 4;

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" :: "l"(p)); }

template <int DT>
__global__ void __launch_bounds__(kAttnWarps * 32) qattn_lane_per_key_kernel(AttnArgs a) {
    __shared__ __align__(16) float q_s[kAttnWarps][kHeadDim];
    __shared__ __align__(16) float qg_s[kAttnWarps][kQjlDim];
    __shared__ float cb_s[kAttnWarps][16];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    if (a.only_if_wide) {
        // launched behind the tensor-core kernel: that kernel served the call unless some centroid is outside the
        // range of its fp16 table (same test there), in which case it stood down and this one does the work in fp32
        const int n_cb = a.cb_per_head ? a.Hkv * 16 : 16;
        bool wide = false;
        for (int i = threadIdx.x; i < n_cb; i += blockDim.x) wide = wide || centroid_is_wide(__ldg(a.codebooks + i));
        if (!__syncthreads_or(wide)) return;
    }
    const int64_t n_work = a.B * a.Hq * a.T * a.n_splits;
    for (int64_t work = (int64_t)blockIdx.x * kAttnWarps + wib; work < n_work; work += (int64_t)gridDim.x * kAttnWarps) {
    const int split = (int)(work % a.n_splits);
    int64_t rest = work / a.n_splits;
    const int64_t qrow = rest;                       // index into q / out: ((b*Hq + hq)*T + tq)
    rest /= a.T;
    const int hq = (int)(rest % a.Hq);
    const int64_t b = rest / a.Hq;
    const int hkv = hq / (a.Hq / a.Hkv);

    // ---- prologue: query, codebook, q . g_i ------------------------------------
    float qv[4];
    Elem<DT>::load4(a.q, qrow * kHeadDim + 4 * lane, qv);
    if (a.lora.x) {                                   // per-user low-rank update of the query row
        lora_fold_row(a.lora, b, a.T, (int)(qrow % a.T), a.Hq * kHeadDim, hq * kHeadDim + 4 * lane, lane, a.status, qv);
    }
    if (a.rotate_q) wht128_warp(qv, lane);
    *reinterpret_cast<float4*>(&q_s[wib][4 * lane]) = make_float4(qv[0], qv[1], qv[2], qv[3]);
    {
        const float c = __ldg(a.codebooks + (a.cb_per_head ? hkv * 16 : 0) + (lane & 15));
        if (lane < 16) cb_s[wib][lane] = c;
        // an infinite or NaN centroid has no meaningful attention result: say so through the status word
        if (__any_sync(kFullMask, !isfinite(c)) && lane == 0 && a.status) atomicExch(a.status, OMNI_STATUS_BAD_CODEBOOK);
    }
    __syncwarp();
    if (a.with_qjl) {
        const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
        const uint4* grow = reinterpret_cast<const uint4*>(a.g_rows) + (size_t)seed_of(uid, hkv) * kQjlDim;
        const uint4 g0 = __ldg(grow + lane), g1 = __ldg(grow + lane + 32);
        const uint32_t w0[4] = {g0.x, g0.y, g0.z, g0.w};
        const uint32_t w1[4] = {g1.x, g1.y, g1.z, g1.w};
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll 8
            for (int j = 0; j < 32; ++j) {
                const float qd = q_s[wib][w * 32 + j];
                acc0 += ((w0[w] >> j) & 1u) ? qd : -qd;
                acc1 += ((w1[w] >> j) & 1u) ? qd : -qd;
            }
        }
        const float cs = kQjlCoef * a.scale;
        qg_s[wib][lane] = acc0 * cs;
        qg_s[wib][lane + 32] = acc1 * cs;
    }
    __syncwarp();

    // ---- key range of this split -----------------------------------------------
    int64_t len = a.seq_lens ? (int64_t)a.seq_lens[b] : a.S;
    len = len < 0 ? 0 : (len > a.S ? a.S : len);
    int64_t per = (len + a.n_splits - 1) / a.n_splits;
    per = (per + 31) / 32 * 32;
    const int64_t s0 = (int64_t)split * per;
    const int64_t s1 = (s0 + per < len) ? s0 + per : len;
    const int64_t slot = a.cache_slots ? (int64_t)a.cache_slots[b] : b;
    const int64_t base_row = slot * a.ks_b + (int64_t)hkv * a.ks_h;

    float m = -INFINITY, l = 0.f;
    float O[kHeadDim];
#pragma unroll
    for (int d = 0; d < kHeadDim; ++d) O[d] = 0.f;
    const float* qs = q_s[wib];
    const float* cbs = cb_s[wib];

    for (int64_t k = s0 + lane; k < s1; k += 32) {
        const int64_t row = base_row + k;
        const uint4* kp = reinterpret_cast<const uint4*>(a.k_nib + row * kNibBytes);
        // This key's sign bytes, norm and V row are needed one after the other further down: on a cold cache that is
        // three memory latencies in a row, so they are requested now, together with the K and V rows of the lane's
        // next key (a V row in the pair layout lies in this key's row and its partner's: the same 512-byte group).
        prefetch_l2(a.v_nib + row * kNibBytes);
        if (a.v_paired && k < (len & ~(int64_t)7)) prefetch_l2(a.v_nib + (base_row + (k ^ 3)) * kNibBytes);
        if (a.with_qjl) { prefetch_l2(a.k_qjl + row * kQjlBytes); prefetch_l2(a.k_norms + row); }
        if (k + 32 < s1) { prefetch_l2(a.k_nib + (row + 32) * kNibBytes); prefetch_l2(a.v_nib + (row + 32) * kNibBytes); }
        float dot = 0.f;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
            const uint4 wv = __ldg(kp + c4);
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const float4 qa = *reinterpret_cast<const float4*>(qs + c4 * 32 + wi * 8);
                const float4 qb = *reinterpret_cast<const float4*>(qs + c4 * 32 + wi * 8 + 4);
                const uint32_t w = ww[wi];
                dot = fmaf(qa.x, cbs[w & 15], dot);
                dot = fmaf(qa.y, cbs[(w >> 4) & 15], dot);
                dot = fmaf(qa.z, cbs[(w >> 8) & 15], dot);
                dot = fmaf(qa.w, cbs[(w >> 12) & 15], dot);
                dot = fmaf(qb.x, cbs[(w >> 16) & 15], dot);
                dot = fmaf(qb.y, cbs[(w >> 20) & 15], dot);
                dot = fmaf(qb.z, cbs[(w >> 24) & 15], dot);
                dot = fmaf(qb.w, cbs[(w >> 28) & 15], dot);
            }
        }
        float score = dot * a.scale;
        if (a.with_qjl) {
            const uint2 sb = __ldg(reinterpret_cast<const uint2*>(a.k_qjl + row * kQjlBytes));
            const float nrm = __ldg(a.k_norms + row);
            float corr = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float g0 = qg_s[wib][i], g1 = qg_s[wib][i + 32];
                corr += ((sb.x >> i) & 1u) ? g0 : -g0;
                corr += ((sb.y >> i) & 1u) ? g1 : -g1;
            }
            score = fmaf(nrm, corr, score);
        }
        const float m_new = fmaxf(m, score);
        const float p = expf(score - m_new);
        if (m_new > m) {
            const float alpha = expf(m - m_new);
            l *= alpha;
#pragma unroll
            for (int d = 0; d < kHeadDim; ++d) O[d] *= alpha;
            m = m_new;
        }
        l += p;
        if (a.v_paired && k < (len & ~(int64_t)7)) {
            // pair layout: this key's even-d nibbles sit in the row of the pair's first key, its odd-d nibbles in
            // the row of the second (pairs (0,3), (1,2), (4,7), (5,6) of a group of eight: partner = key ^ 3), in
            // the low nibbles when this key is the first of the pair, else in the high ones
            const int64_t first = (k & 2) ? (k ^ 3) : k;
            const int sh = (k & 2) ? 4 : 0;
            const uint4* xp = reinterpret_cast<const uint4*>(a.v_nib + (base_row + first) * kNibBytes);
            const uint4* yp = reinterpret_cast<const uint4*>(a.v_nib + (base_row + (first ^ 3)) * kNibBytes);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const uint4 xv = __ldg(xp + c4), yv = __ldg(yp + c4);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int d = c4 * 32 + wi * 8 + 2 * i;
                        O[d] = fmaf(p, cbs[(xw[wi] >> (8 * i + sh)) & 15], O[d]);
                        O[d + 1] = fmaf(p, cbs[(yw[wi] >> (8 * i + sh)) & 15], O[d + 1]);
                    }
                }
            }
        } else {
            const uint4* vp = reinterpret_cast<const uint4*>(a.v_nib + row * kNibBytes);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const uint4 wv = __ldg(vp + c4);
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    const uint32_t w = ww[wi];
#pragma unroll
                    for (int n = 0; n < 8; ++n)
                        O[c4 * 32 + wi * 8 + n] = fmaf(p, cbs[(w >> (4 * n)) & 15], O[c4 * 32 + wi * 8 + n]);
                }
            }
        }
    }

    // ---- merge the 32 lane states ------------------------------------------------
    const float m_w = warp_max(m);
    const float f = (m == -INFINITY) ? 0.f : expf(m - m_w);
    const float l_w = warp_sum(l * f);
#pragma unroll
    for (int d = 0; d < kHeadDim; ++d) O[d] *= f;
    // butterfly reduce-scatter: afterwards O[0..3] hold dims 4*lane .. 4*lane+3
#pragma unroll
    for (int half = 64, mk = 16; half >= 4; half >>= 1, mk >>= 1) {
        const bool upper = (lane & mk) != 0;
#pragma unroll
        for (int j = 0; j < half; ++j) {
            const float send = upper ? O[j] : O[j + half];
            const float keep = upper ? O[j + half] : O[j];
            O[j] = keep + __shfl_xor_sync(kFullMask, send, mk);
        }
    }
    if (a.n_splits == 1) {
        float o[4];
        const float inv = l_w > 0.f ? 1.f / l_w : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = O[k] * inv;
        if (a.unrotate_out) wht128_warp(o, lane);
        *reinterpret_cast<float4*>(a.out + qrow * kHeadDim + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
        float* w = a.ws + work * kWsStride;
        *reinterpret_cast<float4*>(w + 4 * lane) = make_float4(O[0], O[1], O[2], O[3]);
        if (lane == 0) { w[128] = m_w; w[129] = l_w; }
    }
    __syncwarp();                      // the next unit overwrites this warp's query row in shared memory
    }
}

// Merge the per-split partial states of one (user, head, token).  A CTA per output row; its warps take the splits
// round-robin, kCombineUnroll at a time with independent loads (a call with few rows and hundreds of splits is
// bound by load latency, not by bytes), each keeping a running (max, sum, 128 accumulators) state; the warps' states
// are merged through shared memory.  Lane l owns dims 4l .. 4l+3.
constexpr int kCombineWarps = 4;
constexpr int kCombineUnroll = 4;

__device__ __forceinline__ void merge_state(float& m, float& l, float (&o)[4], float ms, float ls, const float4& v) {
    const float mn = fmaxf(m, ms);
    const float fo = (m == -INFINITY) ? 0.f : expf(m - mn);
    const float fs = (ms == -INFINITY) ? 0.f : expf(ms - mn);
    l = l * fo + ls * fs;
    o[0] = o[0] * fo + v.x * fs; o[1] = o[1] * fo + v.y * fs; o[2] = o[2] * fo + v.z * fs; o[3] = o[3] * fo + v.w * fs;
    m = mn;
}

__global__ void __launch_bounds__(kCombineWarps * 32) qattn_combine_kernel(const float* ws, float* out, int64_t n_rows,
                                                                          int n_splits, int unrotate_out) {
    __shared__ float m_s[kCombineWarps], l_s[kCombineWarps];
    __shared__ __align__(16) float o_s[kCombineWarps][kHeadDim];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t r = blockIdx.x;
    const float* w = ws + r * n_splits * kWsStride;
    float m = -INFINITY, l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s0 = warp; s0 < n_splits; s0 += kCombineWarps * kCombineUnroll) {
        float ms[kCombineUnroll], ls[kCombineUnroll];
        float4 v[kCombineUnroll];
#pragma unroll
        for (int u = 0; u < kCombineUnroll; ++u) {
            const int s = s0 + u * kCombineWarps;
            const bool have = s < n_splits;
            const float* p = w + (int64_t)(have ? s : s0) * kWsStride;
            ms[u] = have ? p[128] : -INFINITY;
            ls[u] = p[129];
            v[u] = *reinterpret_cast<const float4*>(p + 4 * lane);
        }
#pragma unroll
        for (int u = 0; u < kCombineUnroll; ++u) merge_state(m, l, o, ms[u], ls[u], v[u]);
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
    *reinterpret_cast<float4*>(&o_s[warp][4 * lane]) = make_float4(o[0], o[1], o[2], o[3]);
    __syncthreads();
    if (warp != 0) return;
    m = -INFINITY; l = 0.f;
    o[0] = o[1] = o[2] = o[3] = 0.f;
#pragma unroll
    for (int k = 0; k < kCombineWarps; ++k)
        merge_state(m, l, o, m_s[k], l_s[k], *reinterpret_cast<const float4*>(&o_s[k][4 * lane]));
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] *= inv;
    if (unrotate_out) wht128_warp(o, lane);
    *reinterpret_cast<float4*>(out + r * kHeadDim + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
}


// Pair layout of V nibble rows.  In the tensor-core kernel the V operand of the P.V product pairs two KEYS per
// register, so its table index is (nibble of key a) | (nibble of key b) << 4; a cache that stores exactly those bytes
// saves the shift-and-merge per lookup.  Within a group of eight consecutive keys the pairs are (0,3), (1,2), (4,7),
// (5,6); the row of the pair's first key receives the even-d nibbles of both keys (byte j = code[a][2j] |
// code[b][2j] << 4), the row of the second key the odd-d nibbles.  The transform is its own inverse.  One warp
// converts one group: lane = (pair, 8-byte column).
__global__ void __launch_bounds__(256) v_pair_groups_kernel(uint8_t* v_nib, int64_t B, int H, int64_t ks_b, int64_t ks_h,
                                                            const int64_t* lens_before, int64_t len_before,
                                                            const int64_t* lens_after, int64_t len_after, int64_t max_groups) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * 8;
    const int64_t units = B * H * max_groups;
    for (int64_t u = warp; u < units; u += n_warps) {
        const int64_t gi = u % max_groups, bh = u / max_groups;
        const int h = (int)(bh % H);
        const int64_t b = bh / H;
        const int64_t g0 = (lens_before ? lens_before[b] : len_before) >> 3, g1 = (lens_after ? lens_after[b] : len_after) >> 3;
        const int64_t grp = g0 + gi;                    // groups [g0, g1) became complete with this append
        if (grp >= g1) continue;
        const int pair = lane >> 3, col = lane & 7;
        const int ra = (pair & 1) + 4 * (pair >> 1), rb = ra ^ 3;            // rows 0,1,4,5 and their partners 3,2,7,6
        uint8_t* base = v_nib + (b * ks_b + (int64_t)h * ks_h + grp * 8) * kNibBytes + 8 * col;
        uint2* pa = reinterpret_cast<uint2*>(base + ra * kNibBytes);
        uint2* pb = reinterpret_cast<uint2*>(base + rb * kNibBytes);
        const uint2 A = *pa, Bv = *pb;
        uint2 x, y;
        x.x = (A.x & 0x0F0F0F0Fu) | ((Bv.x << 4) & 0xF0F0F0F0u);  y.x = ((A.x >> 4) & 0x0F0F0F0Fu) | (Bv.x & 0xF0F0F0F0u);
        x.y = (A.y & 0x0F0F0F0Fu) | ((Bv.y << 4) & 0xF0F0F0F0u);  y.y = ((A.y >> 4) & 0x0F0F0F0Fu) | (Bv.y & 0xF0F0F0F0u);
        *pa = x;
        *pb = y;
    }
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// the part of a split-K workspace no call can do without: partial states and the ticket counters behind them
static size_t partials_and_counter_bytes(int64_t B, int32_t Hq, int32_t T, int32_t n_splits) {
    if (n_splits <= 1 || B <= 0 || Hq <= 0 || T <= 0) return 0;
    return (size_t)B * Hq * T * n_splits * kWsStride * sizeof(float) + kWorkCounterBytes;
}

static int32_t validate(const AttnArgs& a, size_t ws_bytes) {
    OMNI_REQUIRE(a.B >= 0 && a.Hq > 0 && a.Hkv > 0 && a.T >= 0 && a.S >= 0, OMNI_ERR_ARG, "qattn: bad extent");
    OMNI_REQUIRE(a.Hq % a.Hkv == 0, OMNI_ERR_ARG, "qattn: Hq=%d is not a multiple of Hkv=%d", a.Hq, a.Hkv);
    OMNI_REQUIRE(a.Hkv <= kSeeds, OMNI_ERR_UNSUPPORTED, "qattn: Hkv=%d exceeds %d", a.Hkv, kSeeds);
    OMNI_REQUIRE(a.n_splits >= 1 && a.n_splits <= 1024, OMNI_ERR_ARG, "qattn: n_splits=%d outside [1,1024]", a.n_splits);
    if (a.B == 0 || a.T == 0) return OMNI_OK;
    OMNI_REQUIRE(a.q && a.out && a.codebooks, OMNI_ERR_ARG, "qattn: NULL q/out/codebooks");
    OMNI_REQUIRE(a.S == 0 || (a.k_nib && a.v_nib && (!a.with_qjl || (a.k_qjl && a.k_norms))), OMNI_ERR_ARG,
                 "qattn: NULL cache buffer");
    OMNI_REQUIRE(aligned(a.q, a.q_dtype == OMNI_F32 ? 16 : 8) && aligned(a.out, 16), OMNI_ERR_ARG, "qattn: q/out misaligned");
    OMNI_REQUIRE(aligned(a.k_nib, 16) && aligned(a.v_nib, 16) && aligned(a.k_qjl, 8) && aligned(a.k_norms, 4),
                 OMNI_ERR_ARG, "qattn: cache arrays must be 16-byte (nibbles) / 8-byte (sign bytes) aligned");
    if (a.n_splits > 1) {
        const size_t need = partials_and_counter_bytes(a.B, a.Hq, a.T, a.n_splits);
        OMNI_REQUIRE(a.ws && aligned(a.ws, 16) && ws_bytes >= need, OMNI_ERR_ARG,
                     "qattn: workspace of %zu bytes needed for %d splits, got %zu", need, a.n_splits, ws_bytes);
    }
    return OMNI_OK;
}

enum KernelChoice { kAuto = 0, kLanePerKey = 1, kMma = 2, kUmma = 3 };

// OMNI_QATTN_KERNEL=lane|mma|umma forces one kernel where it covers the call (tests and profiling); default: by shape.
static KernelChoice kernel_choice_from_env() {
    const char* e = getenv("OMNI_QATTN_KERNEL");
    if (!e) return kAuto;
    if (e[0] == 'l') return kLanePerKey;
    if (e[0] == 'm') return kMma;
    if (e[0] == 'u') return kUmma;
    return kAuto;
}

// Query columns per kv head from which the tcgen05 kernel is taken: it dequantises a key once for up to 128 columns,
// the warp-level kernel once per eight (measured, 64 users x 2,048 keys: 48 columns = six tiles 0.246 vs 0.235 ms,
// 56 columns = seven tiles 0.247 vs 0.303 ms, 128 columns 0.259 vs 0.546 ms).
constexpr int64_t kUmmaMinColumns = 49;

// Which tensor-core kernel serves a call, if any (otherwise the lane-per-key kernel does).
// Measured crossover: the warp-level kernel wins from 128 keys on, and for shorter caches once the lane-per-key
// kernel would need more than about a thousand warps.
static void choose_kernels(const AttnArgs& a, bool* use_umma, bool* use_mma) {
    const KernelChoice choice = kernel_choice_from_env();
    const int64_t cols = (int64_t)(a.Hq / a.Hkv) * a.T;
    *use_umma = umma_eligible(a) && (choice == kUmma || (choice == kAuto && cols >= kUmmaMinColumns && a.S >= 128));
    *use_mma = !*use_umma && mma_eligible(a) &&
               (choice == kMma || ((choice == kAuto || choice == kUmma) && (a.S >= 128 || a.B * a.Hq * a.T >= 1024)));
}

static int32_t launch(const AttnArgs& a, cudaStream_t st, size_t ws_bytes) {
    if (a.B == 0 || a.T == 0) return OMNI_OK;
    bool use_umma, use_mma;
    choose_kernels(a, &use_umma, &use_mma);
    OMNI_REQUIRE(!(use_umma && a.lora.x), OMNI_ERR_UNSUPPORTED, "qattn: the tcgen05 kernel takes no folded query update");
    if (use_umma) {
        const int32_t rc = launch_umma(a, st);
        if (rc != OMNI_OK) return rc;
    }
    if (use_mma) {
        AttnArgs m = a;
        if (a.n_splits > 1) {    // the ticket counters sit behind the partial states, the prepared query operands behind those
            const size_t partial_floats = (size_t)a.B * a.Hq * a.T * a.n_splits * kWsStride;
            m.work_counter = reinterpret_cast<uint32_t*>(a.ws + partial_floats);
            // OMNI_QATTN_PREP=0 keeps every work item building its own operands (tests and profiling)
            const char* prep_env = getenv("OMNI_QATTN_PREP");
            // Preparing the operands in a launch of its own pays once warps serve several items each (throughput);
            // a call whose items all run at once would only see the extra launch on its critical path (latency).
            const int64_t n_items = a.B * a.Hkv * (((int64_t)(a.Hq / a.Hkv) * a.T + 7) / 8) * a.n_splits;
            const bool many = n_items >= 2 * 148 * 12 || (prep_env && prep_env[0] == '1');
            if (many && !(prep_env && prep_env[0] == '0') && ws_bytes >= omni_qattn_workspace_bytes(a.B, a.Hq, a.T, a.n_splits)) {
                char* behind = reinterpret_cast<char*>(a.ws + partial_floats) + kWorkCounterBytes;
                m.qprep = reinterpret_cast<uint32_t*>(behind + user_order_bytes(a.B));
                // users of different lengths: the preparation launch also sorts them, longest first
                // (OMNI_QATTN_ORDER=0 keeps index order: tests and profiling)
                const char* order_env = getenv("OMNI_QATTN_ORDER");
                const bool one_col = (int64_t)(a.Hq / a.Hkv) * a.T == 1;          // those kernel variants keep index order
                if (a.seq_lens && !one_col && a.B > 1 && a.B <= kMaxOrderedUsers && !(order_env && order_env[0] == '0'))
                    m.user_order = reinterpret_cast<int2*>(behind);
            }
        }
        const int32_t rc = launch_mma(m, st);
        if (rc != OMNI_OK) return rc;
    }
    {
        // The lane-per-key kernel: the call's only kernel for small shapes; behind the tensor-core kernel it is a
        // stand-by that returns at once unless the codebooks are outside the fp16 table's range (decided on the
        // device by both kernels with the same test), so a persistent-size grid suffices there.
        AttnArgs l = a;
        l.only_if_wide = (use_mma || use_umma) ? 1 : 0;
        const int64_t n_work = a.B * a.Hq * a.T * a.n_splits;
        int64_t blocks = (n_work + kAttnWarps - 1) / kAttnWarps;
        const int64_t cap = (use_mma || use_umma) ? 148 * 8 : 148 * 64;
        if (blocks > cap) blocks = cap;
        switch (a.q_dtype) {
            case OMNI_F32:  qattn_lane_per_key_kernel<OMNI_F32><<<(unsigned)blocks, kAttnWarps * 32, 0, st>>>(l); break;
            case OMNI_BF16: qattn_lane_per_key_kernel<OMNI_BF16><<<(unsigned)blocks, kAttnWarps * 32, 0, st>>>(l); break;
            case OMNI_F16:  qattn_lane_per_key_kernel<OMNI_F16><<<(unsigned)blocks, kAttnWarps * 32, 0, st>>>(l); break;
            default: return set_error(OMNI_ERR_ARG, "qattn: unknown q dtype code %d", a.q_dtype);
        }
        OMNI_CUDA(cudaGetLastError());
    }
    if (a.n_splits > 1) {
        const int64_t rows = a.B * a.Hq * a.T;
        OMNI_REQUIRE(rows <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED, "qattn: %lld output rows exceed one grid", (long long)rows);
        qattn_combine_kernel<<<(unsigned)rows, kCombineWarps * 32, 0, st>>>(a.ws, a.out, rows, a.n_splits, a.unrotate_out);
        OMNI_CUDA(cudaGetLastError());
    }
    return OMNI_OK;
}

// Device-side address of a host buffer the GPU can access directly (page-locked by the CUDA allocator or registered),
// or null for pageable memory.
static const void* device_alias_of(const void* host) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        cudaGetLastError();                         // pageable memory is not an error for the caller
        return nullptr;
    }
    return (attr.type == cudaMemoryTypeHost && attr.devicePointer) ? attr.devicePointer : nullptr;
}

// Two internal streams + events per device for the host-buffer step.
struct HostStepStreams { cudaStream_t s[2] = {nullptr, nullptr}; bool ready = false; };
static HostStepStreams g_hs[kMaxDevices];
static std::mutex g_hs_mutex;


// ---- allocation-free variant ---------------------------------------------------------
// Split-K scratch and a private copy of the Rademacher rows live in file-scope device
// arrays, so the entry point below needs no device allocation at all.  The names of
// these arrays are host-side handles, not device addresses: the address a kernel can use
// comes from cudaGetSymbolAddress, taken once per device with that device current.
constexpr size_t kStaticScratchBytes = 32u << 20;                       // 32 MiB of split-K partials
constexpr size_t kStaticRowsWords = (size_t)kSeeds * kQjlDim * 4;        // 1 MiB of G rows
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];
static __device__ __align__(256) uint32_t g_static_rows[kStaticRowsWords];
static __device__ __align__(256) int32_t g_static_status[64];                   // word 0: the entry point's status word

struct StaticArrays { float* scratch = nullptr; uint32_t* rows = nullptr; int32_t* status = nullptr; };
static StaticArrays g_static[kMaxDevices];
static std::mutex g_static_mutex;

// First use on the current device: resolve both symbol addresses and fill the G rows.
static int32_t static_arrays_for_current_device(StaticArrays* out) {
    int dev = -1;
    OMNI_CUDA(cudaGetDevice(&dev));
    OMNI_REQUIRE(dev >= 0 && dev < kMaxDevices, OMNI_ERR_ARG, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_mutex);
    if (!g_static[dev].scratch) {
        float* scratch = nullptr;
        uint32_t* rows = nullptr;
        OMNI_CUDA(cudaGetSymbolAddress((void**)&scratch, g_static_scratch));
        int32_t* status = nullptr;
        OMNI_CUDA(cudaGetSymbolAddress((void**)&rows, g_static_rows));
        OMNI_CUDA(cudaGetSymbolAddress((void**)&status, g_static_status));
        OMNI_CUDA(cudaMemcpy(rows, host_rows_table(), kStaticRowsWords * sizeof(uint32_t), cudaMemcpyHostToDevice));
        // The copy above comes from pageable host memory on the legacy stream: it may return once the data is staged,
        // and a non-blocking stream of the caller has no ordering with the legacy stream at all.  Wait for the device
        // before the table is published, so the first kernel on any stream reads complete rows.
        OMNI_CUDA(cudaDeviceSynchronize());
        g_static[dev].rows = rows;
        g_static[dev].status = status;
        g_static[dev].scratch = scratch;
    }
    *out = g_static[dev];
    return OMNI_OK;
}

}  // namespace omni

using namespace omni;

extern "C" size_t omni_qattn_workspace_bytes(int64_t B, int32_t Hq, int32_t T, int32_t n_splits) {
    if (n_splits <= 1 || B <= 0 || Hq <= 0 || T <= 0) return 0;
    // partial states, ticket counters, the users' processing order, and room for the prepared query operands of every (user, kv head, tile of 8
    // query columns): at most Hq * ceil((T + 7) / 8) such tiles per user whatever the head grouping
    return partials_and_counter_bytes(B, Hq, T, n_splits) + user_order_bytes(B) +
           (size_t)B * Hq * ((T + 7 + 7) / 8) * kPrepBytesPerUnit;
}

extern "C" int32_t omni_qattn_decode(const void* q, int32_t q_dtype,
                                     const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                     const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                     const int32_t* user_ids, int32_t user_id,
                                     const int32_t* seq_lens, const int32_t* cache_slots,
                                     int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                     int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl,
                                     int32_t rotate_q, int32_t unrotate_out, int32_t v_paired, int32_t n_splits,
                                     void* workspace, size_t workspace_bytes, float* out,
                                     int32_t* status_word, void* stream) {
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    AttnArgs a{q, q_dtype, k_nib, k_qjl, k_norms, v_nib, codebooks, cb_per_head, user_ids, user_id, seq_lens,
               cache_slots, B, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, rotate_q, unrotate_out, n_splits,
               (float*)workspace, out, tb->rows, status_word, nullptr, v_paired};
    int32_t st = validate(a, workspace_bytes);
    if (st != OMNI_OK) return st;
    return launch(a, (cudaStream_t)stream, workspace_bytes);
}

static size_t lora_q_bytes(int64_t B, int32_t Hq, int32_t T) {
    if (B <= 0 || Hq <= 0 || T <= 0) return 0;
    return (((size_t)B * Hq * T * kHeadDim * sizeof(float)) + 255) & ~(size_t)255;
}

extern "C" size_t omni_qattn_lora_workspace_bytes(int64_t B, int32_t Hq, int32_t T, int32_t n_splits) {
    return lora_q_bytes(B, Hq, T) + omni_qattn_workspace_bytes(B, Hq, T, n_splits);
}

extern "C" int32_t omni_qattn_decode_lora(const void* q, int32_t q_dtype,
                                          const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                          const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                          const int32_t* user_ids, int32_t user_id,
                                          const int32_t* seq_lens, const int32_t* cache_slots,
                                          int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                          int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl,
                                          int32_t rotate_q, int32_t unrotate_out, int32_t v_paired, int32_t n_splits,
                                          void* workspace, size_t workspace_bytes, float* out,
                                          int32_t* status_word, void* stream, const omni_lora_t* lora) {
    if (!lora)
        return omni_qattn_decode(q, q_dtype, k_nib, k_qjl, k_norms, v_nib, codebooks, cb_per_head, user_ids, user_id,
                                 seq_lens, cache_slots, B, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, rotate_q,
                                 unrotate_out, v_paired, n_splits, workspace, workspace_bytes, out, status_word, stream);
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    const size_t qb = lora_q_bytes(B, Hq, T);
    OMNI_REQUIRE(B == 0 || T == 0 || (workspace && workspace_bytes >= qb), OMNI_ERR_ARG,
                 "qattn_decode_lora: the workspace must hold omni_qattn_lora_workspace_bytes(...) = %zu bytes, got %zu",
                 omni_qattn_lora_workspace_bytes(B, Hq, T, n_splits), workspace_bytes);
    float* q_eff = (float*)workspace;
    AttnArgs a{q_eff, OMNI_F32, k_nib, k_qjl, k_norms, v_nib, codebooks, cb_per_head, user_ids, user_id, seq_lens,
               cache_slots, B, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, rotate_q, unrotate_out, n_splits,
               (float*)((char*)workspace + qb), out, tb->rows, status_word, nullptr, v_paired};
    int32_t st = validate(a, workspace_bytes - (B == 0 || T == 0 ? 0 : qb));
    if (st != OMNI_OK) return st;
    OMNI_REQUIRE(q, OMNI_ERR_ARG, "qattn_decode_lora: NULL q");
    // The update runs inside the attention kernels' prologues (one launch less, no q_eff round trip) wherever the
    // kernel that serves the call loads its query rows itself; OMNI_LORA_FOLD=0 keeps the separate launch.
    // Folded, every work item of a user repeats the down projection, and a lane-per-key warp would repeat it for
    // one query row each: the fold is taken for the warp-level kernel and small adapters (measured on the reference
    // benchmark's shape, rank 16 / hidden 128), the separate launch otherwise.  OMNI_LORA_FOLD=1 folds wherever the
    // serving kernel can, OMNI_LORA_FOLD=0 never.
    const char* fold_env = getenv("OMNI_LORA_FOLD");
    bool use_umma = false, use_mma = false;
    if (B > 0 && T > 0) choose_kernels(a, &use_umma, &use_mma);
    const bool fold = (fold_env && fold_env[0] == '1') ? !use_umma
                    : (fold_env && fold_env[0] == '0') ? false
                    : (use_mma && lora->rank <= 32 && (int64_t)lora->rank * lora->hidden <= 8192);
    if (fold && B > 0 && T > 0) {
        OMNI_REQUIRE(lora->hidden > 0 && lora->rank > 0 && lora->n_adapters >= 0, OMNI_ERR_ARG, "qattn_decode_lora: bad extent");
        OMNI_REQUIRE(lora->rank <= kLoraFoldMaxRank, OMNI_ERR_UNSUPPORTED, "qattn_decode_lora: rank %d exceeds %d", lora->rank, kLoraFoldMaxRank);
        OMNI_REQUIRE(lora->x && lora->lora_a && lora->lora_b && lora->lora_indices, OMNI_ERR_ARG, "qattn_decode_lora: NULL adapter buffer");
        a.q = q;
        a.q_dtype = q_dtype;
        a.lora = LoraFold{lora->x, lora->lora_a, lora->lora_b, lora->lora_indices, lora->n_adapters, lora->hidden, lora->rank, lora->alpha};
        st = validate(a, workspace_bytes - qb);
        if (st != OMNI_OK) return st;
        return launch(a, (cudaStream_t)stream, workspace_bytes - qb);
    }
    st = omni_lora_q(q, q_dtype, lora->x, lora->lora_a, lora->lora_b, lora->lora_indices, lora->n_adapters, lora->alpha,
                     B, Hq, T, lora->hidden, lora->rank, q_eff, status_word, stream);
    if (st != OMNI_OK) return st;
    return launch(a, (cudaStream_t)stream, workspace_bytes - (B == 0 || T == 0 ? 0 : qb));
}

extern "C" int32_t omni_qattn_decode_host(const void* q_host, int32_t q_dtype, void* q_stage,
                                          const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                          const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                          const int32_t* user_ids, int32_t user_id,
                                          const int32_t* seq_lens, const int32_t* cache_slots,
                                          int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                          int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl, int32_t v_paired,
                                          float* out_stage, float* out_host, int32_t n_chunks,
                                          int32_t n_splits, void* workspace, size_t workspace_bytes,
                                          int32_t* status_word) {
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    OMNI_REQUIRE(q_host && out_host, OMNI_ERR_ARG, "qattn_decode_host: NULL host buffer");
    OMNI_REQUIRE(n_chunks >= 1, OMNI_ERR_ARG, "qattn_decode_host: n_chunks < 1");
    // Host buffers the device can address itself (page-locked or registered memory under unified addressing) need no
    // staging: the kernels read the queries and write the rows across PCIe as they go, which overlaps the transfer
    // with the attention work completely (measured on the 16,384-user shard: 34.6 ms against 34.5 ms with everything
    // resident, where the staged two-stream pipeline takes 36.9 ms).  Pageable buffers take the staged pipeline;
    // OMNI_HOST_STEP=staged forces it.
    const void* q_alias = device_alias_of(q_host);
    float* out_alias = static_cast<float*>(const_cast<void*>(device_alias_of(out_host)));
    const char* mode_env = getenv("OMNI_HOST_STEP");
    const bool direct = q_alias && out_alias && !(mode_env && mode_env[0] == 's');
    OMNI_REQUIRE(direct || (q_stage && out_stage), OMNI_ERR_ARG,
                 "qattn_decode_host: staging buffers are required unless both host buffers are page-locked");
    int dev = 0;
    OMNI_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(g_hs_mutex);
        if (!g_hs[dev].ready) {
            OMNI_CUDA(cudaStreamCreateWithFlags(&g_hs[dev].s[0], cudaStreamNonBlocking));
            OMNI_CUDA(cudaStreamCreateWithFlags(&g_hs[dev].s[1], cudaStreamNonBlocking));
            g_hs[dev].ready = true;
        }
    }
    const size_t qsz = q_dtype == OMNI_F32 ? 4 : 2;
    // direct mode: one launch over all users when the workspace allows it (no copies to pipeline), else launch by chunk
    if (direct && (n_splits == 1 || workspace_bytes >= partials_and_counter_bytes(B, Hq, T, n_splits))) n_chunks = 1;
    const int64_t per = (B + n_chunks - 1) / n_chunks;
    // chunks alternate between two streams, so split-K needs one workspace slice per stream
    const size_t ws_chunk = omni_qattn_workspace_bytes(per, Hq, T, n_splits);
    OMNI_REQUIRE(n_splits >= 1, OMNI_ERR_ARG, "qattn_decode_host: n_splits < 1");
    const size_t ws_need = n_chunks == 1 ? partials_and_counter_bytes(B, Hq, T, n_splits) : 2 * ws_chunk;
    OMNI_REQUIRE(n_splits == 1 || (workspace && workspace_bytes >= ws_need), OMNI_ERR_ARG,
                 "qattn_decode_host: %d splits need a workspace of %zu bytes (one slice per stream in use), got %zu",
                 n_splits, ws_need, workspace_bytes);
    const size_t ws_slice = n_chunks == 1 ? workspace_bytes : ws_chunk;
    int c = 0;
    for (int64_t b0 = 0; b0 < B; b0 += per, ++c) {
        const int64_t nb = (b0 + per <= B) ? per : B - b0;
        cudaStream_t st = g_hs[dev].s[c & 1];
        const size_t qoff = (size_t)b0 * Hq * T * kHeadDim;
        if (!direct)
            OMNI_CUDA(cudaMemcpyAsync((char*)q_stage + qoff * qsz, (const char*)q_host + qoff * qsz,
                                      (size_t)nb * Hq * T * kHeadDim * qsz, cudaMemcpyHostToDevice, st));
        // without a slot table user b reads cache block b: shift the cache base for the chunk
        const int64_t row0 = cache_slots ? 0 : b0 * ks_b;
        AttnArgs a{(direct ? (const char*)q_alias : (const char*)q_stage) + qoff * qsz, q_dtype,
                   k_nib + row0 * kNibBytes, k_qjl ? k_qjl + row0 * kQjlBytes : nullptr,
                   k_norms ? k_norms + row0 : nullptr, v_nib + row0 * kNibBytes,
                   codebooks, cb_per_head, user_ids ? user_ids + b0 : nullptr, user_id,
                   seq_lens ? seq_lens + b0 : nullptr, cache_slots ? cache_slots + b0 : nullptr,
                   nb, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, 0, 0, n_splits,
                   n_splits > 1 ? reinterpret_cast<float*>((char*)workspace + (size_t)(c & 1) * ws_chunk) : nullptr,
                   (direct ? out_alias : out_stage) + qoff, tb->rows, status_word, nullptr, v_paired};
        int32_t stc = validate(a, ws_slice);
        if (stc == OMNI_OK) stc = launch(a, st, ws_slice);
        if (stc != OMNI_OK) { cudaStreamSynchronize(g_hs[dev].s[0]); cudaStreamSynchronize(g_hs[dev].s[1]); return stc; }
        if (!direct)
            OMNI_CUDA(cudaMemcpyAsync(out_host + qoff, out_stage + qoff, (size_t)nb * Hq * T * kHeadDim * sizeof(float),
                                      cudaMemcpyDeviceToHost, st));
    }
    OMNI_CUDA(cudaStreamSynchronize(g_hs[dev].s[0]));
    OMNI_CUDA(cudaStreamSynchronize(g_hs[dev].s[1]));
    return OMNI_OK;
}

extern "C" int32_t omni_v_pair_groups(uint8_t* v_nib, int64_t B, int32_t H, int64_t S, int64_t ks_b, int64_t ks_h,
                                      const int64_t* lens_before, int64_t len_before,
                                      const int64_t* lens_after, int64_t len_after, void* stream) {
    OMNI_REQUIRE(B >= 0 && H >= 0 && S >= 0, OMNI_ERR_ARG, "omni_v_pair_groups: negative extent");
    OMNI_REQUIRE((lens_before == nullptr) == (lens_after == nullptr), OMNI_ERR_ARG,
                 "omni_v_pair_groups: give both length arrays or neither");
    if (!lens_before) {
        OMNI_REQUIRE(0 <= len_before && len_before <= len_after && len_after <= S, OMNI_ERR_ARG,
                     "omni_v_pair_groups: lengths %lld -> %lld outside [0, %lld]", (long long)len_before, (long long)len_after, (long long)S);
    }
    const int64_t max_groups = lens_before ? (S >> 3) : ((len_after >> 3) - (len_before >> 3));
    if (B == 0 || H == 0 || max_groups <= 0) return OMNI_OK;
    OMNI_REQUIRE(v_nib && aligned(v_nib, 8), OMNI_ERR_ARG, "omni_v_pair_groups: NULL or misaligned nibble array");
    int64_t blocks = (B * H * max_groups + 7) / 8;
    if (blocks > 148 * 32) blocks = 148 * 32;
    v_pair_groups_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(v_nib, B, H, ks_b, ks_h, lens_before, len_before,
                                                                           lens_after, len_after, max_groups);
    return check_cuda(cudaGetLastError(), "v_pair_groups_kernel launch");
}

extern "C" size_t omni_qattn_noalloc_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int32_t omni_qattn_decode_noalloc(const void* q, int32_t q_dtype,
                                             const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                             const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                             const int32_t* user_ids, int32_t user_id,
                                             const int32_t* seq_lens, const int32_t* cache_slots,
                                             int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                             int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl,
                                             int32_t rotate_q, int32_t unrotate_out, int32_t v_paired, int32_t n_splits,
                                             float* out, void* stream) {
    // partial states and ticket counters only: the built-in scratch leaves out the prepared query operands that a
    // caller-provided workspace has room for (every work item builds its own here)
    const size_t need = partials_and_counter_bytes(B, Hq, T, n_splits);
    OMNI_REQUIRE(need <= kStaticScratchBytes, OMNI_ERR_UNSUPPORTED,
                 "omni_qattn_decode_noalloc: B*Hq*T*n_splits = %lld partial states need %zu bytes of scratch but the "
                 "built-in array holds %zu; lower n_splits or use omni_qattn_decode with a caller-provided workspace",
                 (long long)(B * Hq * T * n_splits), need, kStaticScratchBytes);
    StaticArrays arr;
    int32_t st = static_arrays_for_current_device(&arr);
    if (st != OMNI_OK) return st;
    AttnArgs a{q, q_dtype, k_nib, k_qjl, k_norms, v_nib, codebooks, cb_per_head, user_ids, user_id, seq_lens,
               cache_slots, B, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, rotate_q, unrotate_out, n_splits,
               arr.scratch, out, arr.rows, arr.status, nullptr, v_paired};
    st = validate(a, kStaticScratchBytes);
    if (st != OMNI_OK) return st;
    return launch(a, (cudaStream_t)stream, need);
}

extern "C" int32_t omni_qattn_noalloc_status(int32_t* value_out, int32_t clear) {
    OMNI_REQUIRE(value_out != nullptr, OMNI_ERR_ARG, "omni_qattn_noalloc_status: value_out is NULL");
    StaticArrays arr;
    int32_t st = static_arrays_for_current_device(&arr);
    if (st != OMNI_OK) return st;
    OMNI_CUDA(cudaDeviceSynchronize());
    OMNI_CUDA(cudaMemcpy(value_out, arr.status, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (clear && *value_out != 0) OMNI_CUDA(cudaMemset(arr.status, 0, sizeof(int32_t)));
    return OMNI_OK;
}

extern "C" int32_t omni_diag_bounded_wait(int32_t poll_limit, int32_t* status_word, void* stream) {
    OMNI_REQUIRE(poll_limit >= 1 && poll_limit <= (1 << 20), OMNI_ERR_ARG,
                 "omni_diag_bounded_wait: poll_limit %d outside [1, 2^20]", poll_limit);
    OMNI_REQUIRE(status_word != nullptr, OMNI_ERR_ARG, "omni_diag_bounded_wait: status_word is NULL");
    return launch_wait_probe((uint32_t)poll_limit, status_word, (cudaStream_t)stream);
}
