// Fused decode / short-prefill attention over the packed INT4 + QJL cache.
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
#include "common.cuh"
#include <mutex>
#include <cstdlib>

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
};

constexpr int kAttnWarps = 4;
constexpr int kWsStride = 132;     // floats per partial: 128 accumulators, max, sum, 2 pad

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

template <int DT>
__global__ void __launch_bounds__(kAttnWarps * 32) qattn_lane_per_key_kernel(AttnArgs a) {
    __shared__ __align__(16) float q_s[kAttnWarps][kHeadDim];
    __shared__ __align__(16) float qg_s[kAttnWarps][kQjlDim];
    __shared__ float cb_s[kAttnWarps][16];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int64_t work = (int64_t)blockIdx.x * kAttnWarps + wib;
    const int64_t n_work = a.B * a.Hq * a.T * a.n_splits;
    if (work >= n_work) return;
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
    if (a.rotate_q) wht128_warp(qv, lane);
    *reinterpret_cast<float4*>(&q_s[wib][4 * lane]) = make_float4(qv[0], qv[1], qv[2], qv[3]);
    if (lane < 16) cb_s[wib][lane] = __ldg(a.codebooks + (a.cb_per_head ? hkv * 16 : 0) + lane);
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
}

// Merge the per-split partial states of one (user, head, token): warp per output row.
__global__ void __launch_bounds__(kAttnWarps * 32) qattn_combine_kernel(const float* ws, float* out, int64_t n_rows,
                                                                        int n_splits, int unrotate_out) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * kAttnWarps + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const float* w = ws + r * n_splits * kWsStride;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, w[s * kWsStride + 128]);
    float l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_splits; ++s) {
        const float ms = w[s * kWsStride + 128];
        const float f = (ms == -INFINITY) ? 0.f : expf(ms - m);
        l += w[s * kWsStride + 129] * f;
        const float4 v = *reinterpret_cast<const float4*>(w + s * kWsStride + 4 * lane);
        o[0] = fmaf(v.x, f, o[0]); o[1] = fmaf(v.y, f, o[1]); o[2] = fmaf(v.z, f, o[2]); o[3] = fmaf(v.w, f, o[3]);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] *= inv;
    if (unrotate_out) wht128_warp(o, lane);
    *reinterpret_cast<float4*>(out + r * kHeadDim + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
}


// =====================================================================================
// Tensor-core decode kernel (mma.sync m16n8k16, fp16 operands, fp32 accumulate).
//
// One warp owns one (user, kv head, key split) and all query columns of that kv head
// (a column = one (query head of the group, query token); at most 8).  Keys are taken 16
// at a time.  Everything is computed transposed so that the key axis is the MMA "M":
//     S^T[key, col]  = sum_d  K^[key, d] * q[col, d]         (8 MMAs, A = dequantised K)
//                    + norm[key] * sum_i s_i[key] * (q.g_i)[col]   (4 MMAs, A = +-1)
//     O^T[d,  col]  += sum_key V^[key, d] * P[key, col]       (8 MMAs, A = dequantised V^T)
// A fragments come straight from the packed bytes: a 256-entry table maps a byte to the
// half2 (cb[low nibble], cb[high nibble]); it is replicated per lane so that every lookup
// is bank-conflict free, and placed on a 64 KiB boundary of the shared window so that one
// PRMT forms the complete address (byte -> bits 8..15).  The contraction index of each MMA
// is a permutation of d (or of the projections) chosen so that each thread reads 16
// contiguous bytes of a key row.  For V the two nibbles of a pair come from two different
// keys; the index byte is formed with one shift and one LOP3 per four lookups.
// Packed bytes go global -> registers (no shared-memory staging: shared-memory bandwidth
// is what the table lookups need), double-buffered one 16-key block ahead.
// =====================================================================================
#ifndef OMNI_MMA_WARPS
#define OMNI_MMA_WARPS 12
#endif
constexpr int kMmaWarps = OMNI_MMA_WARPS;
constexpr int kLutSpan = 65536;                 // 256 entries x 256 B (32 lanes x 4 B used per entry)
constexpr int kWarpScratchBytes = 512 + 8 * 64 * 4;
// Dynamic shared memory: the two tables start at the first 64 KiB boundary of the shared
// window (offset up to 65535 from the start of the allocation); the warp scratch sits in
// front of them when that gap is large enough, otherwise behind them.
constexpr int kScratchAllBytes = kMmaWarps * kWarpScratchBytes;
constexpr int kMmaSmemBytes = (kLutSpan + 2 * kLutSpan) > (2 * kScratchAllBytes + 2 * kLutSpan)
                                  ? (kLutSpan + 2 * kLutSpan) : (2 * kScratchAllBytes + 2 * kLutSpan);
static_assert(kMmaSmemBytes <= 227 * 1024, "decode kernel exceeds the shared memory of one SM");
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first MMA of a chain: D = A*B with a zero addend (no accumulator registers to clear)
__device__ __forceinline__ void mma_f16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
#ifdef OMNI_LDG_L1ALLOC
#define OMNI_LDG "ld.global.nc"
#else
#define OMNI_LDG "ld.global.nc.L1::no_allocate"
#endif
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile(OMNI_LDG ".v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 v;
    asm volatile(OMNI_LDG ".v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream2(const void* p) {
    uint16_t v;
    asm volatile(OMNI_LDG ".u16 %0, [%1];\n" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldg_stream_f32(const void* p) {
    float v;
    asm volatile(OMNI_LDG ".f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// table lookup: byte `which` of w selects the entry; lut_lane has zero bits 8..15
template <int WHICH>
__device__ __forceinline__ uint32_t lut_at(uint32_t lut_lane, uint32_t w) {
    const uint32_t addr = __byte_perm(w, lut_lane, 0x7604 | (WHICH << 4));
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));   // read-only table: free to be scheduled early
    return v;
}
// sign-table lookup: byte WHICH of the 16 sign bits selects four half2 of +-1.0
// (bits 0,1 | 2,3 | 4,5 | 6,7 of that byte); sgn_lane has zero bits 8..15
template <int WHICH>
__device__ __forceinline__ uint4 sgn_at(uint32_t sgn_lane, uint32_t s) {
    const uint32_t addr = __byte_perm(s, sgn_lane, 0x7604 | (WHICH << 4));
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__host__ __device__ constexpr uint32_t sign_half2(uint32_t bit0, uint32_t bit1) {
    return 0x3C003C00u ^ (bit0 ? 0u : 0x8000u) ^ (bit1 ? 0u : 0x80000000u);
}

struct KeyBlock {           // packed bytes of one 16-key block as this thread needs them
    // Score-tile row r of the MMA holds key rho(r): rho(g) = (g>>1) + 4*(g&1) for r < 8, rho(r) = rho(r-8)+8.
    // With this order the transposed weights pair keys (t, t+4) and (t+8, t+12), so that each V load
    // instruction reads four consecutive rows.
    uint4 ka, kb;           // K nibbles: keys rho(g) and rho(g)+8, bytes 16t..16t+15
    uint2 v0, v1, v2, v3;   // V nibbles: keys t, t+4, t+8, t+12, bytes 8g..8g+7
    uint32_t sa, sb;        // K sign bits: keys rho(g), rho(g)+8, bits 16t..16t+15
    float na, nb;           // K residual norms: keys rho(g), rho(g)+8
};

// Per-thread cursors into the packed arrays, positioned at the next block to load.
struct Cursors {
    const uint8_t* pk;      // k_nib + row(rho(g))*64 + 16t
    const uint8_t* pv;      // v_nib + row(t)*64 + 8g
    const uint8_t* ps;      // k_qjl + row(rho(g))*8 + 2t
    const float* pn;        // k_norms + row(rho(g))
    const uint8_t* pf;      // L2 prefetch cursor of this lane (lanes 0-3: K nibbles, V nibbles, signs, norms)
    const uint8_t* pf_end;  // end of this work unit's rows in that array: prefetches never reach past it
    uint32_t pf_bytes;      // bytes per 16-key block behind pf (multiple of 16), 0 for the other lanes
};

constexpr int kPrefetchBlocks = 4;   // 16-key blocks between the L2 prefetch and the register loads

// Bulk L2 prefetch (issued by the TMA unit): `bytes` (multiple of 16) from a 16-byte aligned address.
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(p), "r"(bytes) : "memory");
}
// Block step j: the lane that owns stream (j mod 4) prefetches that stream for four blocks at once,
// so every stream is refreshed every fourth block and stays kPrefetchBlocks..kPrefetchBlocks+3 ahead.
__device__ __forceinline__ void prefetch_step(Cursors& c, int j, int lane) {
    if (lane == (j & 3) && c.pf_bytes) {
        const uint32_t room = (uint32_t)(c.pf_end - c.pf) & ~15u;
        const uint32_t want = 4u * c.pf_bytes + 16u;                            // 16 extra: starts are rounded down
        const uint32_t n = room < want ? room : want;
        if (n) prefetch_l2_bulk(c.pf, n);
        c.pf += 4u * c.pf_bytes;
    }
}

// full block: every row exists, fixed offsets from the cursors
template <bool QJL>
__device__ __forceinline__ void load_full_block(KeyBlock& kb, Cursors& c) {
    kb.ka = ldg_stream16(c.pk);
    kb.kb = ldg_stream16(c.pk + 8 * kNibBytes);
    kb.v0 = ldg_stream8(c.pv);
    kb.v1 = ldg_stream8(c.pv + 4 * kNibBytes);
    kb.v2 = ldg_stream8(c.pv + 8 * kNibBytes);
    kb.v3 = ldg_stream8(c.pv + 12 * kNibBytes);
    if (QJL) {
        kb.sa = ldg_stream2(c.ps);
        kb.sb = ldg_stream2(c.ps + 8 * kQjlBytes);
        kb.na = ldg_stream_f32(c.pn);
        kb.nb = ldg_stream_f32(c.pn + 8);
    }
    c.pk += 16 * kNibBytes; c.pv += 16 * kNibBytes; c.ps += 16 * kQjlBytes; c.pn += 16;
}

// last, partial block: rows past the end are clamped to the last valid key (their scores are masked)
template <bool QJL>
__device__ __forceinline__ void load_tail_block(KeyBlock& kb, const Cursors& c, int nvalid, int kl, int t) {
    const int last = nvalid - 1;
    const int dg = min(kl, last) - kl, dg8 = min(kl + 8, last) - kl;
    kb.ka = ldg_stream16(c.pk + dg * kNibBytes);
    kb.kb = ldg_stream16(c.pk + dg8 * kNibBytes);
    const int d0 = min(t, last) - t, d1 = min(t + 4, last) - t;
    const int d2 = min(t + 8, last) - t, d3 = min(t + 12, last) - t;
    kb.v0 = ldg_stream8(c.pv + d0 * kNibBytes);
    kb.v1 = ldg_stream8(c.pv + d1 * kNibBytes);
    kb.v2 = ldg_stream8(c.pv + d2 * kNibBytes);
    kb.v3 = ldg_stream8(c.pv + d3 * kNibBytes);
    if (QJL) {
        kb.sa = ldg_stream2(c.ps + dg * kQjlBytes);
        kb.sb = ldg_stream2(c.ps + dg8 * kQjlBytes);
        kb.na = ldg_stream_f32(c.pn + dg);
        kb.nb = ldg_stream_f32(c.pn + dg8);
    }
}

struct WarpState {
    float O[8][4];          // O^T accumulators: [m-tile][c-fragment]
    float m0, m1, l0, l1;   // running max (log2 units) and partial sums for columns 2t, 2t+1
};

constexpr float kLazyMaxSlack = 6.f;   // log2 units a score may exceed the reference maximum before it is raised


template <bool QJL, bool TAIL>
__device__ __forceinline__ void process_key_block(const KeyBlock& kb, WarpState& st, const uint32_t (&qB)[8][2],
                                                  const uint32_t (&gB)[4][2], float post0, float post1,
                                                  uint32_t lut_lane, uint32_t sgn_lane, int nvalid, int kl) {
    // two independent accumulator chains per product so consecutive MMAs do not wait on each other
    float cd[4], ce[4];
    {
        const uint32_t wa[4] = {kb.ka.x, kb.ka.y, kb.ka.z, kb.ka.w};
        const uint32_t wb[4] = {kb.kb.x, kb.kb.y, kb.kb.z, kb.kb.w};
        // k-step 2w: bytes 0,1 of word w; k-step 2w+1: bytes 2,3
        mma_f16_first(cd, lut_at<0>(lut_lane, wa[0]), lut_at<0>(lut_lane, wb[0]),
                          lut_at<1>(lut_lane, wa[0]), lut_at<1>(lut_lane, wb[0]), qB[0][0], qB[0][1]);
        mma_f16_first(ce, lut_at<2>(lut_lane, wa[0]), lut_at<2>(lut_lane, wb[0]),
                          lut_at<3>(lut_lane, wa[0]), lut_at<3>(lut_lane, wb[0]), qB[1][0], qB[1][1]);
#pragma unroll
        for (int w = 1; w < 4; ++w) {
            mma_f16(cd, lut_at<0>(lut_lane, wa[w]), lut_at<0>(lut_lane, wb[w]),
                        lut_at<1>(lut_lane, wa[w]), lut_at<1>(lut_lane, wb[w]), qB[2 * w][0], qB[2 * w][1]);
            mma_f16(ce, lut_at<2>(lut_lane, wa[w]), lut_at<2>(lut_lane, wb[w]),
                        lut_at<3>(lut_lane, wa[w]), lut_at<3>(lut_lane, wb[w]), qB[2 * w + 1][0], qB[2 * w + 1][1]);
        }
    }
    float s00, s01, s80, s81;           // scores of keys rho(g) / rho(g)+8 for columns 2t / 2t+1, log2 units
    if (QJL) {
        float cq[4], cr[4];
        const uint4 a_lo = sgn_at<0>(sgn_lane, kb.sa), a_hi = sgn_at<1>(sgn_lane, kb.sa);   // key g
        const uint4 b_lo = sgn_at<0>(sgn_lane, kb.sb), b_hi = sgn_at<1>(sgn_lane, kb.sb);   // key g+8
        mma_f16_first(cq, a_lo.x, b_lo.x, a_lo.y, b_lo.y, gB[0][0], gB[0][1]);
        mma_f16_first(cr, a_lo.z, b_lo.z, a_lo.w, b_lo.w, gB[1][0], gB[1][1]);
        mma_f16(cq, a_hi.x, b_hi.x, a_hi.y, b_hi.y, gB[2][0], gB[2][1]);
        mma_f16(cr, a_hi.z, b_hi.z, a_hi.w, b_hi.w, gB[3][0], gB[3][1]);
        s00 = post0 * fmaf(kb.na, cq[0] + cr[0], cd[0] + ce[0]);
        s01 = post1 * fmaf(kb.na, cq[1] + cr[1], cd[1] + ce[1]);
        s80 = post0 * fmaf(kb.nb, cq[2] + cr[2], cd[2] + ce[2]);
        s81 = post1 * fmaf(kb.nb, cq[3] + cr[3], cd[3] + ce[3]);
    } else {
        s00 = post0 * (cd[0] + ce[0]); s01 = post1 * (cd[1] + ce[1]);
        s80 = post0 * (cd[2] + ce[2]); s81 = post1 * (cd[3] + ce[3]);
    }
    if (TAIL) {
        if (kl >= nvalid) { s00 = -INFINITY; s01 = -INFINITY; }
        if (kl + 8 >= nvalid) { s80 = -INFINITY; s81 = -INFINITY; }
    }
    // Lazy running maximum: the reference point m of a column is raised only when some score
    // exceeds it by more than kLazyMaxSlack, so the cross-lane reduction and the rescale of the
    // accumulators run on few blocks; in between, weights are at most 2^kLazyMaxSlack.
    const bool exceed = (fmaxf(s00, s80) > st.m0 + kLazyMaxSlack) || (fmaxf(s01, s81) > st.m1 + kLazyMaxSlack);
    if (__any_sync(kFullMask, exceed)) {
        float mx0 = fmaxf(s00, s80), mx1 = fmaxf(s01, s81);
#pragma unroll
        for (int m = 4; m <= 16; m <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, m));
            mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, m));
        }
        const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
        const float al0 = ex2_approx(st.m0 - mn0), al1 = ex2_approx(st.m1 - mn1);
        st.l0 *= al0; st.l1 *= al1;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            st.O[mt][0] *= al0; st.O[mt][1] *= al1; st.O[mt][2] *= al0; st.O[mt][3] *= al1;
        }
        st.m0 = mn0; st.m1 = mn1;
    }
    const float p00 = ex2_approx(s00 - st.m0), p01 = ex2_approx(s01 - st.m1);
    const float p80 = ex2_approx(s80 - st.m0), p81 = ex2_approx(s81 - st.m1);
    st.l0 += p00 + p80;
    st.l1 += p01 + p81;
    // P^T as the B operand: transpose the two 8x8 (key x column) blocks across the warp
    const uint32_t pb0 = movmatrix_trans(pack_half2(p00, p01));
    const uint32_t pb1 = movmatrix_trans(pack_half2(p80, p81));
    // V: index byte = nibble of key A | nibble of key B << 4
    {
        const uint32_t A[2] = {kb.v0.x, kb.v0.y}, B[2] = {kb.v1.x, kb.v1.y};
        const uint32_t C[2] = {kb.v2.x, kb.v2.y}, D[2] = {kb.v3.x, kb.v3.y};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t x01 = (A[h] & 0x0F0F0F0Fu) | ((B[h] << 4) & 0xF0F0F0F0u);
            const uint32_t y01 = ((A[h] >> 4) & 0x0F0F0F0Fu) | (B[h] & 0xF0F0F0F0u);
            const uint32_t x23 = (C[h] & 0x0F0F0F0Fu) | ((D[h] << 4) & 0xF0F0F0F0u);
            const uint32_t y23 = ((C[h] >> 4) & 0x0F0F0F0Fu) | (D[h] & 0xF0F0F0F0u);
            mma_f16(st.O[4 * h + 0], lut_at<0>(lut_lane, x01), lut_at<0>(lut_lane, y01),
                                     lut_at<0>(lut_lane, x23), lut_at<0>(lut_lane, y23), pb0, pb1);
            mma_f16(st.O[4 * h + 1], lut_at<1>(lut_lane, x01), lut_at<1>(lut_lane, y01),
                                     lut_at<1>(lut_lane, x23), lut_at<1>(lut_lane, y23), pb0, pb1);
            mma_f16(st.O[4 * h + 2], lut_at<2>(lut_lane, x01), lut_at<2>(lut_lane, y01),
                                     lut_at<2>(lut_lane, x23), lut_at<2>(lut_lane, y23), pb0, pb1);
            mma_f16(st.O[4 * h + 3], lut_at<3>(lut_lane, x01), lut_at<3>(lut_lane, y01),
                                     lut_at<3>(lut_lane, x23), lut_at<3>(lut_lane, y23), pb0, pb1);
        }
    }
}

template <int DT, bool QJL>
__global__ void __launch_bounds__(kMmaWarps * 32, 1) qattn_mma_kernel(AttnArgs a, int64_t n_items) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kl = (g >> 1) + 4 * (g & 1);        // key (within a 16-key block) of score-tile row g
    const bool head_in_item = (gridDim.y == 1 && a.Hkv > 1);   // shared codebook: a CTA serves all kv heads
    const int cb_head = blockIdx.y;
    // place the table on a 64 KiB boundary of the shared window, the warp scratch beside it
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t lut_off = (kLutSpan - (smem_base & (kLutSpan - 1))) & (kLutSpan - 1);
    constexpr uint32_t kScratchAll = kMmaWarps * kWarpScratchBytes;
    const uint32_t scratch_off = (lut_off >= kScratchAll) ? 0u : lut_off + 2 * kLutSpan;
    {
        const float* cb = a.codebooks + (a.cb_per_head ? cb_head * 16 : 0);
        uint32_t* lut = reinterpret_cast<uint32_t*>(smem + lut_off);
        for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
            const int byte = i >> 5, ln = i & 31;
            lut[byte * 64 + ln] = pack_half2(__ldg(cb + (byte & 15)), __ldg(cb + (byte >> 4)));
        }
        if (QJL) {   // sign table: entry b, 8 copies of 16 B: +-1.0 pairs for bits (0,1) (2,3) (4,5) (6,7) of b
            uint4* sgn = reinterpret_cast<uint4*>(smem + lut_off + kLutSpan);
            for (int i = threadIdx.x; i < 256 * 8; i += blockDim.x) {
                const uint32_t b = i >> 3;
                sgn[b * 16 + (i & 7)] = make_uint4(sign_half2(b & 1, b & 2), sign_half2(b & 4, b & 8),
                                                   sign_half2(b & 16, b & 32), sign_half2(b & 64, b & 128));
            }
        }
    }
    __syncthreads();
    const uint32_t lut_lane = smem_base + lut_off + 4 * lane;                     // bits 8..15 are zero
    const uint32_t sgn_lane = smem_base + lut_off + kLutSpan + 16 * (lane & 7);  // likewise
    float* qf = reinterpret_cast<float*>(smem + scratch_off + warp * kWarpScratchBytes);
    float* qg_s = qf + 128;                                          // [8][64]
    const int Gq = a.Hq / a.Hkv;
    const int ncols = Gq * a.T;
    const float qs = a.scale * kLog2e;

    for (int64_t item = (int64_t)blockIdx.x * kMmaWarps + warp; item < n_items;
         item += (int64_t)gridDim.x * kMmaWarps) {
        int64_t rest = item;
        int hkv = cb_head;
        if (head_in_item) { hkv = (int)(rest % a.Hkv); rest /= a.Hkv; }
        const int split = (int)(rest % a.n_splits);
        const int64_t b = rest / a.n_splits;

        // ---- prologue: B operands (scaled queries, q.g projections) ---------------------
        uint32_t qB[8][2], gB[4][2];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) { qB[kk][0] = 0u; qB[kk][1] = 0u; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) { gB[kk][0] = 0u; gB[kk][1] = 0u; }
        float post0 = 1.f, post1 = 1.f;
        uint4 g0 = make_uint4(0, 0, 0, 0), g1 = g0;
        if (QJL) {
            const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
            const uint4* grow = reinterpret_cast<const uint4*>(a.g_rows) + (size_t)seed_of(uid, hkv) * kQjlDim;
            g0 = __ldg(grow + lane); g1 = __ldg(grow + lane + 32);
        }
        for (int c = 0; c < ncols; ++c) {
            const int64_t qrow = (b * a.Hq + (int64_t)hkv * Gq + c / a.T) * a.T + (c % a.T);
            float qv[4];
            Elem<DT>::load4(a.q, qrow * kHeadDim + 4 * lane, qv);
            const float mx = warp_max(fmaxf(fmaxf(fabsf(qv[0]), fabsf(qv[1])), fmaxf(fabsf(qv[2]), fabsf(qv[3])))) * fabsf(qs);
            // keep the fp16 operands below 2^10 in magnitude; the power of two is re-applied to the scores
            float post = 1.f;
            if (mx > 1024.f) post = exp2f(ceilf(log2f(mx * (1.f / 1024.f))));
            const float f = qs / post;
            __syncwarp();
            *reinterpret_cast<float4*>(qf + 4 * lane) = make_float4(qv[0], qv[1], qv[2], qv[3]);
            __syncwarp();
            if (QJL) {
                const uint32_t w0[4] = {g0.x, g0.y, g0.z, g0.w}, w1[4] = {g1.x, g1.y, g1.z, g1.w};
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
#pragma unroll 8
                    for (int j = 0; j < 32; ++j) {
                        const float qd = qf[w * 32 + j];
                        acc0 += ((w0[w] >> j) & 1u) ? qd : -qd;
                        acc1 += ((w1[w] >> j) & 1u) ? qd : -qd;
                    }
                }
                qg_s[c * 64 + lane] = acc0 * (kQjlCoef * f);
                qg_s[c * 64 + lane + 32] = acc1 * (kQjlCoef * f);
            }
            if (g == c) {
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const float4 v = *reinterpret_cast<const float4*>(qf + 32 * t + 4 * kk);
                    qB[kk][0] = pack_half2(v.x * f, v.y * f);
                    qB[kk][1] = pack_half2(v.z * f, v.w * f);
                }
            }
            if (c == 2 * t) post0 = post;
            if (c == 2 * t + 1) post1 = post;
        }
        __syncwarp();
        if (QJL && g < ncols) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float4 v = *reinterpret_cast<const float4*>(qg_s + g * 64 + 16 * t + 4 * kk);
                gB[kk][0] = pack_half2(v.x, v.y);
                gB[kk][1] = pack_half2(v.z, v.w);
            }
        }

        // ---- key range of this split -----------------------------------------------------
        int64_t len = a.seq_lens ? (int64_t)a.seq_lens[b] : a.S;
        len = len < 0 ? 0 : (len > a.S ? a.S : len);
        int64_t per = (len + a.n_splits - 1) / a.n_splits;
        per = (per + 31) / 32 * 32;
        const int64_t s0 = (int64_t)split * per;
        const int64_t s1 = (s0 + per < len) ? s0 + per : len;
        const int64_t slot = a.cache_slots ? (int64_t)a.cache_slots[b] : b;
        const int64_t base_row = slot * a.ks_b + (int64_t)hkv * a.ks_h;

        WarpState st;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) { st.O[mt][0] = 0.f; st.O[mt][1] = 0.f; st.O[mt][2] = 0.f; st.O[mt][3] = 0.f; }
        st.m0 = -INFINITY; st.m1 = -INFINITY; st.l0 = 0.f; st.l1 = 0.f;

        if (s1 > s0) {
            const int64_t row0 = base_row + s0;
            const int64_t row_g = row0 + kl, row_v = row0 + t;
            Cursors cur;
            cur.pk = a.k_nib + row_g * kNibBytes + 16 * t;
            cur.pv = a.v_nib + row_v * kNibBytes + 8 * g;
            cur.ps = a.k_qjl + row_g * kQjlBytes + 2 * t;
            cur.pn = a.k_norms + row_g;
            const int nfull = (int)((s1 - s0) >> 4), rem = (int)((s1 - s0) & 15);
            // L2 prefetch streams: lane 0 K nibbles, 1 V nibbles, 2 sign bytes, 3 norms.  The sign and
            // norm rows need not start on a 16-byte boundary: round the start down and fetch 16 bytes more.
            cur.pf = nullptr; cur.pf_end = nullptr; cur.pf_bytes = 0;
            {
                const int64_t nrows = s1 - s0;
                if (lane == 0)             { cur.pf = a.k_nib + row0 * kNibBytes; cur.pf_bytes = 16 * kNibBytes; cur.pf_end = cur.pf + nrows * kNibBytes; }
                else if (lane == 1)        { cur.pf = a.v_nib + row0 * kNibBytes; cur.pf_bytes = 16 * kNibBytes; cur.pf_end = cur.pf + nrows * kNibBytes; }
                else if (QJL && lane == 2) { cur.pf = a.k_qjl + row0 * kQjlBytes; cur.pf_bytes = 16 * kQjlBytes; cur.pf_end = cur.pf + nrows * kQjlBytes; }
                else if (QJL && lane == 3) { cur.pf = reinterpret_cast<const uint8_t*>(a.k_norms + row0); cur.pf_bytes = 16 * 4; cur.pf_end = cur.pf + nrows * 4; }
            }
            if (cur.pf_bytes) {
                // the first blocks in one request, then one block per step
                cur.pf = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(cur.pf) & ~(uintptr_t)15);
                const uint32_t room = (uint32_t)(cur.pf_end - cur.pf) & ~15u;
                // stream s is refreshed at block steps j = s (mod 4): start it s blocks further ahead
                const uint32_t want = (kPrefetchBlocks + lane) * cur.pf_bytes + 16u;
                const uint32_t n = room < want ? room : want;
                if (n) prefetch_l2_bulk(cur.pf, n);
                cur.pf += (kPrefetchBlocks + lane) * cur.pf_bytes;
            }
            KeyBlock blk_a, blk_b;
            if (nfull > 0) load_full_block<QJL>(blk_a, cur);
            int j = 0;
            for (; j + 1 < nfull; j += 2) {            // blocks j (in blk_a) and j+1 are full
                load_full_block<QJL>(blk_b, cur);
                prefetch_step(cur, j, lane);
                process_key_block<QJL, false>(blk_a, st, qB, gB, post0, post1, lut_lane, sgn_lane, 16, kl);
                if (j + 2 < nfull) load_full_block<QJL>(blk_a, cur);
                prefetch_step(cur, j + 1, lane);
                process_key_block<QJL, false>(blk_b, st, qB, gB, post0, post1, lut_lane, sgn_lane, 16, kl);
            }
            if (j < nfull)                              // odd count: the last full block is already in blk_a
                process_key_block<QJL, false>(blk_a, st, qB, gB, post0, post1, lut_lane, sgn_lane, 16, kl);
            if (rem) {                                   // partial block: clamped loads, masked scores
                load_tail_block<QJL>(blk_b, cur, rem, kl, t);
                process_key_block<QJL, true>(blk_b, st, qB, gB, post0, post1, lut_lane, sgn_lane, rem, kl);
            }
        }

        // ---- epilogue ----------------------------------------------------------------------
#pragma unroll
        for (int m = 4; m <= 16; m <<= 1) {
            st.l0 += __shfl_xor_sync(kFullMask, st.l0, m);
            st.l1 += __shfl_xor_sync(kFullMask, st.l1, m);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = 2 * t + j;
            if (c >= ncols) continue;
            const int64_t qrow = (b * a.Hq + (int64_t)hkv * Gq + c / a.T) * a.T + (c % a.T);
            const float l = j ? st.l1 : st.l0;
            const float m = j ? st.m1 : st.m0;
            float* dst;
            float mul;
            if (a.n_splits == 1) {
                dst = a.out + qrow * kHeadDim + 16 * g;
                mul = l > 0.f ? 1.f / l : 0.f;
            } else {
                float* w = a.ws + (qrow * a.n_splits + split) * kWsStride;
                dst = w + 16 * g;
                mul = 1.f;
                if (g == 0) { w[128] = m * 0.6931471805599453f; w[129] = l; }   // max back in natural-log units
            }
#pragma unroll
            for (int mp = 0; mp < 4; ++mp) {      // d = 16g + 4mp .. 16g + 4mp + 3  (m-tiles 2mp, 2mp+1)
                float4 v;
                v.x = st.O[2 * mp][j] * mul;     v.y = st.O[2 * mp][2 + j] * mul;
                v.z = st.O[2 * mp + 1][j] * mul; v.w = st.O[2 * mp + 1][2 + j] * mul;
                *reinterpret_cast<float4*>(dst + 4 * mp) = v;
            }
        }
    }
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

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
        const size_t need = omni_qattn_workspace_bytes(a.B, a.Hq, a.T, a.n_splits);
        OMNI_REQUIRE(a.ws && aligned(a.ws, 16) && ws_bytes >= need, OMNI_ERR_ARG,
                     "qattn: workspace of %zu bytes needed for %d splits, got %zu", need, a.n_splits, ws_bytes);
    }
    return OMNI_OK;
}

enum KernelChoice { kAuto = 0, kLanePerKey = 1, kMma = 2 };

// OMNI_QATTN_KERNEL=lane|mma forces one kernel (tests and profiling); default: by shape.
static KernelChoice kernel_choice_from_env() {
    const char* e = getenv("OMNI_QATTN_KERNEL");
    if (!e) return kAuto;
    if (e[0] == 'l') return kLanePerKey;
    if (e[0] == 'm') return kMma;
    return kAuto;
}

static bool mma_eligible(const AttnArgs& a) {
    const int cols = (a.Hq / a.Hkv) * a.T;
    return cols <= 8 && !a.rotate_q && !a.unrotate_out && a.Hkv <= 65535;
}

template <int DT>
static int32_t launch_mma(const AttnArgs& a, cudaStream_t st) {
    int dev = 0, sms = 148;
    OMNI_CUDA(cudaGetDevice(&dev));
    OMNI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // Persistent CTAs, one per SM.  With one shared codebook a CTA serves every kv head
    // (grid.y == 1, the head is part of the item index); with per-head codebooks a CTA is
    // bound to one head because its lookup table is built from that head's centroids.
    int64_t items, ctas;
    unsigned gy;
    if (a.cb_per_head) {
        items = a.B * a.n_splits;
        ctas = sms / a.Hkv > 0 ? sms / a.Hkv : 1;
        gy = (unsigned)a.Hkv;
    } else {
        items = a.B * a.n_splits * a.Hkv;
        ctas = sms;
        gy = 1;
    }
    const int64_t need = (items + kMmaWarps - 1) / kMmaWarps;
    if (ctas > need) ctas = need;
    dim3 grid((unsigned)ctas, gy);
    auto kern = a.with_qjl ? qattn_mma_kernel<DT, true> : qattn_mma_kernel<DT, false>;
    OMNI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmemBytes));
    kern<<<grid, kMmaWarps * 32, kMmaSmemBytes, st>>>(a, items);
    return check_cuda(cudaGetLastError(), "qattn_mma_kernel launch");
}

static int32_t launch(const AttnArgs& a, cudaStream_t st) {
    if (a.B == 0 || a.T == 0) return OMNI_OK;
    const KernelChoice choice = kernel_choice_from_env();
    const bool use_mma = mma_eligible(a) && (choice == kMma || (choice == kAuto && a.S >= 128));
    if (use_mma) {
        int32_t rc;
        switch (a.q_dtype) {
            case OMNI_F32:  rc = launch_mma<OMNI_F32>(a, st); break;
            case OMNI_BF16: rc = launch_mma<OMNI_BF16>(a, st); break;
            case OMNI_F16:  rc = launch_mma<OMNI_F16>(a, st); break;
            default: return set_error(OMNI_ERR_ARG, "qattn: unknown q dtype code %d", a.q_dtype);
        }
        if (rc != OMNI_OK) return rc;
    } else {
        const int64_t n_work = a.B * a.Hq * a.T * a.n_splits;
        const int64_t blocks = (n_work + kAttnWarps - 1) / kAttnWarps;
        OMNI_REQUIRE(blocks <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED, "qattn: %lld work units exceed one grid", (long long)n_work);
        switch (a.q_dtype) {
            case OMNI_F32:  qattn_lane_per_key_kernel<OMNI_F32><<<(unsigned)blocks, kAttnWarps * 32, 0, st>>>(a); break;
            case OMNI_BF16: qattn_lane_per_key_kernel<OMNI_BF16><<<(unsigned)blocks, kAttnWarps * 32, 0, st>>>(a); break;
            case OMNI_F16:  qattn_lane_per_key_kernel<OMNI_F16><<<(unsigned)blocks, kAttnWarps * 32, 0, st>>>(a); break;
            default: return set_error(OMNI_ERR_ARG, "qattn: unknown q dtype code %d", a.q_dtype);
        }
        OMNI_CUDA(cudaGetLastError());
    }
    if (a.n_splits > 1) {
        const int64_t rows = a.B * a.Hq * a.T;
        qattn_combine_kernel<<<(unsigned)((rows + kAttnWarps - 1) / kAttnWarps), kAttnWarps * 32, 0, st>>>(
            a.ws, a.out, rows, a.n_splits, a.unrotate_out);
        OMNI_CUDA(cudaGetLastError());
    }
    return OMNI_OK;
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

struct StaticArrays { float* scratch = nullptr; uint32_t* rows = nullptr; };
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
        OMNI_CUDA(cudaGetSymbolAddress((void**)&rows, g_static_rows));
        OMNI_CUDA(cudaMemcpy(rows, host_rows_table(), kStaticRowsWords * sizeof(uint32_t), cudaMemcpyHostToDevice));
        g_static[dev].rows = rows;
        g_static[dev].scratch = scratch;
    }
    *out = g_static[dev];
    return OMNI_OK;
}

}  // namespace omni

using namespace omni;

extern "C" size_t omni_qattn_workspace_bytes(int64_t B, int32_t Hq, int32_t T, int32_t n_splits) {
    if (n_splits <= 1 || B <= 0 || Hq <= 0 || T <= 0) return 0;
    return (size_t)B * Hq * T * n_splits * kWsStride * sizeof(float);
}

extern "C" int32_t omni_qattn_decode(const void* q, int32_t q_dtype,
                                     const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                     const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                     const int32_t* user_ids, int32_t user_id,
                                     const int32_t* seq_lens, const int32_t* cache_slots,
                                     int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                     int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl,
                                     int32_t rotate_q, int32_t unrotate_out, int32_t n_splits,
                                     void* workspace, size_t workspace_bytes, float* out,
                                     int32_t* status_word, void* stream) {
    (void)status_word;   // this kernel has no device-side waits
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    AttnArgs a{q, q_dtype, k_nib, k_qjl, k_norms, v_nib, codebooks, cb_per_head, user_ids, user_id, seq_lens,
               cache_slots, B, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, rotate_q, unrotate_out, n_splits,
               (float*)workspace, out, tb->rows};
    int32_t st = validate(a, workspace_bytes);
    if (st != OMNI_OK) return st;
    return launch(a, (cudaStream_t)stream);
}

extern "C" int32_t omni_qattn_decode_host(const void* q_host, int32_t q_dtype, void* q_stage,
                                          const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                          const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                          const int32_t* user_ids, int32_t user_id,
                                          const int32_t* seq_lens, const int32_t* cache_slots,
                                          int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                          int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl,
                                          float* out_stage, float* out_host, int32_t n_chunks) {
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    OMNI_REQUIRE(q_host && q_stage && out_stage && out_host, OMNI_ERR_ARG, "qattn_decode_host: NULL buffer");
    OMNI_REQUIRE(n_chunks >= 1, OMNI_ERR_ARG, "qattn_decode_host: n_chunks < 1");
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
    const int64_t per = (B + n_chunks - 1) / n_chunks;
    int c = 0;
    for (int64_t b0 = 0; b0 < B; b0 += per, ++c) {
        const int64_t nb = (b0 + per <= B) ? per : B - b0;
        cudaStream_t st = g_hs[dev].s[c & 1];
        const size_t qoff = (size_t)b0 * Hq * T * kHeadDim;
        OMNI_CUDA(cudaMemcpyAsync((char*)q_stage + qoff * qsz, (const char*)q_host + qoff * qsz,
                                  (size_t)nb * Hq * T * kHeadDim * qsz, cudaMemcpyHostToDevice, st));
        // without a slot table user b reads cache block b: shift the cache base for the chunk
        const int64_t row0 = cache_slots ? 0 : b0 * ks_b;
        AttnArgs a{(const char*)q_stage + qoff * qsz, q_dtype,
                   k_nib + row0 * kNibBytes, k_qjl ? k_qjl + row0 * kQjlBytes : nullptr,
                   k_norms ? k_norms + row0 : nullptr, v_nib + row0 * kNibBytes,
                   codebooks, cb_per_head, user_ids ? user_ids + b0 : nullptr, user_id,
                   seq_lens ? seq_lens + b0 : nullptr, cache_slots ? cache_slots + b0 : nullptr,
                   nb, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, 0, 0, 1, nullptr, out_stage + qoff, tb->rows};
        int32_t stc = validate(a, 0);
        if (stc == OMNI_OK) stc = launch(a, st);
        if (stc != OMNI_OK) { cudaStreamSynchronize(g_hs[dev].s[0]); cudaStreamSynchronize(g_hs[dev].s[1]); return stc; }
        OMNI_CUDA(cudaMemcpyAsync(out_host + qoff, out_stage + qoff, (size_t)nb * Hq * T * kHeadDim * sizeof(float),
                                  cudaMemcpyDeviceToHost, st));
    }
    OMNI_CUDA(cudaStreamSynchronize(g_hs[dev].s[0]));
    OMNI_CUDA(cudaStreamSynchronize(g_hs[dev].s[1]));
    return OMNI_OK;
}

extern "C" size_t omni_qattn_noalloc_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int32_t omni_qattn_decode_noalloc(const void* q, int32_t q_dtype,
                                             const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                             const uint8_t* v_nib, const float* codebooks, int32_t cb_per_head,
                                             const int32_t* user_ids, int32_t user_id,
                                             const int32_t* seq_lens, const int32_t* cache_slots,
                                             int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                             int64_t ks_b, int64_t ks_h, float scale, int32_t with_qjl,
                                             int32_t rotate_q, int32_t unrotate_out, int32_t n_splits,
                                             float* out, void* stream) {
    const size_t need = omni_qattn_workspace_bytes(B, Hq, T, n_splits);
    OMNI_REQUIRE(need <= kStaticScratchBytes, OMNI_ERR_UNSUPPORTED,
                 "omni_qattn_decode_noalloc: B*Hq*T*n_splits = %lld partial states need %zu bytes of scratch but the "
                 "built-in array holds %zu; lower n_splits or use omni_qattn_decode with a caller-provided workspace",
                 (long long)(B * Hq * T * n_splits), need, kStaticScratchBytes);
    StaticArrays arr;
    int32_t st = static_arrays_for_current_device(&arr);
    if (st != OMNI_OK) return st;
    AttnArgs a{q, q_dtype, k_nib, k_qjl, k_norms, v_nib, codebooks, cb_per_head, user_ids, user_id, seq_lens,
               cache_slots, B, Hq, Hkv, T, S, ks_b, ks_h, scale, with_qjl, rotate_q, unrotate_out, n_splits,
               arr.scratch, out, arr.rows};
    st = validate(a, kStaticScratchBytes);
    if (st != OMNI_OK) return st;
    return launch(a, (cudaStream_t)stream);
}
