// Rotate + quantize with one THREAD per row and the 64 x 128 +-1 projections on the fifth-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory).  Included by codec_fast.cu, whose helpers it shares.
//
// The warp-cooperative kernel (fast_quantize_kernel) spreads a row over four lanes and pays for it in shuffles, ballots
// and selects: about 172 warp instructions per row.  Here a CTA of 128 threads takes 128 consecutive tokens of one
// (user, head); thread r owns row r from the load to the stores:
//   * rotation: all seven butterfly stages inside the thread, in the reference's stage order, one rounding per add or
//     subtract (packed f32x2 where the partner is 64 elements away), one multiply by float32(1/sqrt(128)), rounding to
//     the element type for 16-bit inputs;
//   * INT4 codes: the same exact search as the warp-cooperative kernel (grid cell + one exact threshold compare; binary
//     search or the defining scan for codebooks and values outside the proven range), chosen per thread;
//   * sign bits: the residual row is scaled by a power of two (times 1 - 2^-9) to 23-bit integers, one rounding each,
//     and split into three byte limbs that the thread stores as row r of three K-major int8 operand tiles in shared
//     memory.  One thread issues twelve tcgen05.mma (three limbs x four K steps of 32) against the +-1 matrix of the
//     (user, head), M = 128 rows, N = 64 projections, int32 accumulators in tensor memory.  Thread r reads its 64 x 3
//     sums back (tcgen05.ld), recombines them and takes the signs.  The integer sum differs from the exact scaled sum
//     by at most 64, so |sum| > 64 decides the sign rigorously; with 23-bit integers about one row in five thousand
//     has a projection inside that band, and those few are recomputed exactly in fp64 by the owning thread;
//   * packed outputs: 64 contiguous nibble bytes, 8 sign bytes and one norm per thread.
// The highest limb is stored with the +0x40 offset that the magic-number conversion leaves in it (so all three limbs are
// unsigned bytes); the offset contributes 2^22 * (row sum of G) to projection i, a constant per (seed, i) that is kept in
// shared memory and taken off again.
#pragma once

namespace omni {

constexpr int kTcThreads = 128;
constexpr uint32_t kTcLbo = 128;                      // K-major int8 tiles: bytes between the two 16-element K chunks of an MMA
constexpr uint32_t kTcSbo = (128 / 16) * 128;         // ... and between groups of 8 rows (8 core matrices of 128 B)
constexpr uint32_t kTcLimbBytes = 128 * 128;          // one limb tile: 128 rows x 128 int8
constexpr uint32_t kTcGBytes = 64 * 128;              // the +-1 matrix: 64 projections x 128 int8
constexpr uint32_t kTcTmemCols = 256;                 // three accumulators of 64 columns (power of two allocation)
constexpr uint32_t kTcWaitLimit = 1u << 22;

__device__ __forceinline__ void tcq_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool tcq_mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kTcWaitLimit; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// D[tmem] (+)= A[smem desc] * B[smem desc], 8-bit integer operands, int32 accumulator
__device__ __forceinline__ void tcq_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ uint64_t tcq_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// kind::i8 instruction descriptor: unsigned A, signed B, int32 accumulator, both operands K-major
__host__ __device__ constexpr uint32_t tcq_idesc(int M, int N) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tcq_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tcq_sts16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// One row of 128 elements as fp32 registers.
template <int DT> struct Row128;
template <> struct Row128<OMNI_F32> {
    static __device__ __forceinline__ void load(const void* x, int64_t i, float (&y)[128]) {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(x) + i);
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const uint4 c = __ldg(p + k);
            y[4 * k] = __uint_as_float(c.x); y[4 * k + 1] = __uint_as_float(c.y);
            y[4 * k + 2] = __uint_as_float(c.z); y[4 * k + 3] = __uint_as_float(c.w);
        }
    }
};
template <> struct Row128<OMNI_BF16> {
    static __device__ __forceinline__ void load(const void* x, int64_t i, float (&y)[128]) {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + i);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const uint4 c = __ldg(p + k);
            const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                y[8 * k + 2 * j] = __uint_as_float(w[j] << 16);
                y[8 * k + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    }
};
template <> struct Row128<OMNI_F16> {
    static __device__ __forceinline__ void load(const void* x, int64_t i, float (&y)[128]) {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(x) + i);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const uint4 c = __ldg(p + k);
            const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                y[8 * k + 2 * j] = f.x; y[8 * k + 2 * j + 1] = f.y;
            }
        }
    }
};

// Normalised 128-point Walsh-Hadamard transform inside one thread: stage order h = 1 .. 64, one rounding per operation;
// elements i and i + 64 travel as a packed pair through the first six stages (u - v is fma(v, -1, u), which rounds like
// the subtraction), the last stage pairs them with each other.
__device__ __forceinline__ void rotate_row128(float (&y)[128]) {
#pragma unroll
    for (int hh = 1; hh < 64; hh <<= 1) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            if ((i & hh) == 0) {
                const float u0 = y[i], u1 = y[i + 64], v0 = y[i | hh], v1 = y[(i | hh) + 64];
                add2(y[i], y[i + 64], u0, u1, v0, v1);
                fma2(y[i | hh], y[(i | hh) + 64], v0, v1, -1.f, -1.f, u0, u1);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 64; ++i) {
        const float u = y[i], v = y[i + 64];
        y[i] = __fadd_rn(u, v);
        y[i + 64] = __fsub_rn(u, v);
    }
    const float sc = __uint_as_float(OMNI_WHT_SCALE_BITS);
#pragma unroll
    for (int i = 0; i < 64; ++i) mul2(y[i], y[i + 64], y[i], y[i + 64], sc, sc);
}

// Exact sign of projection `pi` of the residual row e (fp64 accumulation of fp32 values): true when the sum is >= 0.
__device__ __forceinline__ bool exact_projection_sign(const float (&e)[128], const uint32_t* grow, int pi) {
    double acc = 0.0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t gw = __ldg(grow + pi * 4 + w);
#pragma unroll
        for (int i = 0; i < 32; ++i) { const double ev = (double)e[32 * w + i]; acc += ((gw >> i) & 1u) ? ev : -ev; }
    }
    return acc >= 0.0;
}

template <int DT, bool ROTATE, bool SIGNS>
__global__ void __launch_bounds__(kTcThreads, 2) tc_quantize_kernel(FastQuantArgs a, int64_t n_items, int64_t tiles_per_head) {
    extern __shared__ __align__(1024) unsigned char tq_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_tabs = a.cb_per_head ? a.H : 1;
    // shared memory: [limb tiles 3 x 16 KB][G 8 KB][row-sum constants 64 x int][mbarrier, tmem slot][per-head tables]
    const uint32_t s_base = (uint32_t)__cvta_generic_to_shared(tq_smem);
    const uint32_t sA = s_base, sG = s_base + 3 * kTcLimbBytes;
    int* rowconst = reinterpret_cast<int*>(tq_smem + 3 * kTcLimbBytes + kTcGBytes);        // 64 - 2^22 * rowsum(G_i)
    const uint32_t bar = s_base + 3 * kTcLimbBytes + kTcGBytes + 256;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tq_smem + 3 * kTcLimbBytes + kTcGBytes + 256 + 16);
    HeadTables* tabs = reinterpret_cast<HeadTables*>(tq_smem + 3 * kTcLimbBytes + kTcGBytes + 512);

    for (int h = warp; h < n_tabs; h += kTcThreads / 32) build_head_tables(tabs[h], a.codebooks + h * 16, lane);
    uint32_t tmem = 0;
    if (SIGNS) {
        if (tid == 0) {
            tcq_mbar_init(bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        if (warp == 0) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                         :: "r"((uint32_t)__cvta_generic_to_shared(tmem_slot)), "r"(kTcTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    }
    __syncthreads();
    if (SIGNS) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        tmem = *tmem_slot;
    }
    const uint32_t t_lane = tmem + ((uint32_t)(32 * warp) << 16);
    uint32_t phase = 0;
    bool ok = true;
    int cur_seed = -1;

    for (int64_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const int64_t tile = item % tiles_per_head, bh = item / tiles_per_head;
        const int h = (int)(bh % a.H);
        const int64_t b = bh / a.H;
        const int64_t t0 = tile * kTcThreads, tr = t0 + tid;
        const bool active = tr < a.T;
        const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
        const int seed = seed_of(uid, h);
        const uint32_t* grow = a.g_rows + (size_t)seed * kQjlDim * 4;
        if (SIGNS && seed != cur_seed) {
            // the +-1 matrix of this (user, head) as the K-major B operand: thread i < 64 writes projection row i
            if (tid < kQjlDim) {
                int ones = 0;
                const uint32_t rowg = sG + (uint32_t)(tid >> 3) * kTcSbo + (uint32_t)(tid & 7) * 16;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t gw = __ldg(grow + tid * 4 + w);
                    ones += __popc(gw);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {            // 16 dims per 16-byte chunk
                        const uint32_t x = gw >> (16 * c);
                        tcq_sts16(rowg + (uint32_t)(2 * w + c) * kTcLbo, pm1_bytes<0>(x), pm1_bytes<4>(x),
                                  pm1_bytes<0>(x >> 8), pm1_bytes<4>(x >> 8));
                    }
                }
                // the highest limb carries +0x40: it adds 2^22 * sum_d g_id to projection i; the band test wants + 64
                rowconst[tid] = 64 - (2 * ones - kHeadDim) * (1 << 22);
            }
            cur_seed = seed;
        }
        const HeadTables& ht = tabs[a.cb_per_head ? h : 0];
        const int64_t in_row = b * a.xs_b + (int64_t)h * a.xs_h + (active ? tr : a.T - 1) * a.xs_t;
        const int64_t ro = b * a.os_b + (int64_t)h * a.os_h + (a.out_offsets ? a.out_offsets[b] : a.out_offset) + tr;

        float y[128];
        Row128<DT>::load(a.x, in_row, y);
        if (ROTATE) {
            rotate_row128(y);
#pragma unroll
            for (int i = 0; i < 128; i += 2) Row32<DT>::round_pair(y[i], y[i + 1]);
        }
        // ---- INT4 codes and residual (y becomes the residual) ------------------------------------------------
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 128; ++i) amax = fmaxf(amax, fabsf(y[i]));
        uint32_t codes[16];
#pragma unroll
        for (int w = 0; w < 16; ++w) codes[w] = 0u;
        if (!(amax <= ht.guard)) {
#pragma unroll
            for (int i = 0; i < 128; ++i) {
                const int c = code_by_scan(y[i], ht.cb);
                codes[i >> 3] |= (uint32_t)c << (4 * (i & 7));
                y[i] = __fsub_rn(y[i], ht.cb[c]);
            }
        } else if (ht.valid == 2) {
#pragma unroll
            for (int i = 0; i < 128; ++i) {
                int c = (y[i] >= ht.thr[8]) ? 8 : 0;
                c += (y[i] >= ht.thr[c + 4]) ? 4 : 0;
                c += (y[i] >= ht.thr[c + 2]) ? 2 : 0;
                c += (y[i] >= ht.thr[c + 1]) ? 1 : 0;
                codes[i >> 3] |= (uint32_t)c << (4 * (i & 7));
                y[i] = __fsub_rn(y[i], ht.cb[c]);
            }
        } else {
            const float inv32 = ht.inv32, off32 = ht.off32;
#pragma unroll
            for (int i = 0; i < 128; ++i) {
                const float2 rec = ht.cell2[cell_of(y[i], inv32, off32)];
                const int c = __float_as_int(rec.y) + (y[i] >= rec.x ? 1 : 0);
                codes[i >> 3] |= (uint32_t)c << (4 * (i & 7));
                y[i] = __fsub_rn(y[i], ht.cb[c]);
            }
        }
        if (active) {
            uint4* np = reinterpret_cast<uint4*>(a.nib + ro * kNibBytes);
#pragma unroll
            for (int k = 0; k < 4; ++k) np[k] = make_uint4(codes[4 * k], codes[4 * k + 1], codes[4 * k + 2], codes[4 * k + 3]);
        }
        if (!SIGNS) continue;

        // ---- residual norm and fixed-point scale ------------------------------------------------------------
        float ss, emax;
        {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, m0 = 0.f, m1 = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                fma2(s0, s1, y[i], y[i + 64], y[i], y[i + 64], s0, s1);
                fma2(s2, s3, y[i + 32], y[i + 96], y[i + 32], y[i + 96], s2, s3);
                m0 = fmaxf(m0, fmaxf(fabsf(y[i]), fabsf(y[i + 64])));
                m1 = fmaxf(m1, fmaxf(fabsf(y[i + 32]), fabsf(y[i + 96])));
            }
            ss = (s0 + s1) + (s2 + s3);
            emax = fmaxf(m0, m1);
        }
        const int E = (__float_as_uint(emax) >> 23) & 0xFF;
        // rows whose largest residual is 0 / tiny / inf, or that hold a NaN, cannot be scaled to integers
        const bool degenerate = (E < 24) || (E == 255) || !(ss < INFINITY);
        // scale = 2^(148-E) * (1 - 2^-9): emax * scale lies in [2^21 - 4096, 2^22 - 8192), so the rounded integers
        // stay inside the range in which adding 1.5 * 2^23 leaves them in the low 23 bits of the sum
        const float scale = degenerate ? 0.f : __uint_as_float(((uint32_t)(274 - E) << 23) | 0x7F8000u);
        {
            const uint32_t rowa = sA + (uint32_t)(tid >> 3) * kTcSbo + (uint32_t)(tid & 7) * 16;
#pragma unroll
            for (int c = 0; c < 8; ++c) {                        // 16 elements per 16-byte chunk and limb
                uint32_t l0[4], l1[4], l2[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t v[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) v[k] = __float_as_uint(fmaf(y[16 * c + 4 * q + k], scale, 12582912.f));
                    const uint32_t p01 = __byte_perm(v[0], v[1], 0x5140), p23 = __byte_perm(v[2], v[3], 0x5140);
                    l0[q] = __byte_perm(p01, p23, 0x5410);
                    l1[q] = __byte_perm(p01, p23, 0x7632);
                    l2[q] = __byte_perm(__byte_perm(v[0], v[1], 0x0062), __byte_perm(v[2], v[3], 0x0062), 0x5410);
                }
                tcq_sts16(rowa + (uint32_t)c * kTcLbo, l0[0], l0[1], l0[2], l0[3]);
                tcq_sts16(rowa + kTcLimbBytes + (uint32_t)c * kTcLbo, l1[0], l1[1], l1[2], l1[3]);
                tcq_sts16(rowa + 2 * kTcLimbBytes + (uint32_t)c * kTcLbo, l2[0], l2[1], l2[2], l2[3]);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int l = 0; l < 3; ++l)
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    tcq_mma_i8(tmem + 64 * l, tcq_desc(sA + l * kTcLimbBytes + ks * 2 * kTcLbo, kTcLbo, kTcSbo),
                               tcq_desc(sG + ks * 2 * kTcLbo, kTcLbo, kTcSbo), tcq_idesc(128, 64), ks > 0);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" :: "r"(bar) : "memory");
        }
        ok = __syncthreads_and(tcq_mbar_wait_bounded(bar, phase)) != 0;
        phase ^= 1u;
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

        // ---- signs: sum_i = (D2 * 256 + D1) * 256 + D0 - 2^22 * rowsum_i; u = sum + 64; sign = u >= 64, band = u <= 128 ----
        uint32_t bits_lo = 0u, bits_hi = 0u;
        bool any_band = false;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t d0[16], d1[16], d2[16];
            tcq_ld16(t_lane + 16 * ch, d0);
            tcq_ld16(t_lane + 64 + 16 * ch, d1);
            tcq_ld16(t_lane + 128 + 16 * ch, d2);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            uint32_t part = 0u;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int u = ((int)d2[i] * 256 + (int)d1[i]) * 256 + (int)d0[i] + rowconst[16 * ch + i];
                part |= (u >= 64 ? 1u : 0u) << i;
                any_band = any_band || ((uint32_t)u <= 128u);
            }
            if (ch < 2) bits_lo |= part << (16 * ch); else bits_hi |= part << (16 * (ch - 2));
        }
        if (emax == 0.f) { bits_lo = 0xffffffffu; bits_hi = 0xffffffffu; }         // zero residual: every projection is +0
        // (the tensor-memory loads are warp-wide: every lane of the warp takes this path when one of its rows needs it)
        const bool redo = emax != 0.f && (degenerate || any_band);
        if (__any_sync(kFullMask, redo)) {
            // which projections lie inside the band (all of them for a row that could not be scaled)
            uint32_t band_lo = 0u, band_hi = 0u;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t d0[16], d1[16], d2[16];
                tcq_ld16(t_lane + 16 * ch, d0);
                tcq_ld16(t_lane + 64 + 16 * ch, d1);
                tcq_ld16(t_lane + 128 + 16 * ch, d2);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                uint32_t part = 0u;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int u = ((int)d2[i] * 256 + (int)d1[i]) * 256 + (int)d0[i] + rowconst[16 * ch + i];
                    part |= ((uint32_t)u <= 128u ? 1u : 0u) << i;
                }
                if (ch < 2) band_lo |= part << (16 * ch); else band_hi |= part << (16 * (ch - 2));
            }
            if (degenerate) { band_lo = 0xffffffffu; band_hi = 0xffffffffu; }
            if (!redo) { band_lo = 0u; band_hi = 0u; }
            // exact recomputation in fp64 by the thread that owns the row
            while (band_lo | band_hi) {
                const bool low = band_lo != 0u;
                const int pi = low ? __ffs((int)band_lo) - 1 : 32 + __ffs((int)band_hi) - 1;
                if (low) band_lo &= band_lo - 1u; else band_hi &= band_hi - 1u;
                const bool pos = exact_projection_sign(y, grow, pi);
                const uint32_t m = 1u << (pi & 31);
                if (low) bits_lo = pos ? (bits_lo | m) : (bits_lo & ~m);
                else     bits_hi = pos ? (bits_hi | m) : (bits_hi & ~m);
            }
        }
        if (active) {
            *reinterpret_cast<uint2*>(a.qjl + ro * kQjlBytes) = make_uint2(bits_lo, bits_hi);
            a.norms[ro] = sqrtf(ss);
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();                                     // every thread has read its sums before the next tile's products
    }
    if (SIGNS) {
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        if (warp == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" :: "r"(tmem), "r"(kTcTmemCols) : "memory");
        }
    }
}

template <int DT>
static int32_t launch_tc_t(const FastQuantArgs& a, int rotate, cudaStream_t st) {
    int dev = 0, sms = 148;
    OMNI_CUDA(cudaGetDevice(&dev));
    OMNI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int n_tabs = a.cb_per_head ? a.H : 1;
    // at least 80 KB, so that no more than two CTAs share an SM: each holds half of its tensor memory
    size_t smem = 3 * kTcLimbBytes + kTcGBytes + 512 + sizeof(HeadTables) * n_tabs;
    if (smem < 80 * 1024) smem = 80 * 1024;
    const int64_t tiles = (a.T + kTcThreads - 1) / kTcThreads;
    const int64_t items = a.B * a.H * tiles;
    const bool signs = a.qjl != nullptr;
    auto kern = signs ? (rotate ? tc_quantize_kernel<DT, true, true> : tc_quantize_kernel<DT, false, true>)
                      : (rotate ? tc_quantize_kernel<DT, true, false> : tc_quantize_kernel<DT, false, false>);
    {
        static std::mutex mu;
        static std::vector<std::pair<const void*, int>> done;
        const void* key = reinterpret_cast<const void*>(kern);
        std::lock_guard<std::mutex> lk(mu);
        bool seen = false;
        for (const auto& p : done) seen = seen || (p.first == key && p.second == dev);
        if (!seen) {
            size_t smem_max = 3 * kTcLimbBytes + kTcGBytes + 512 + sizeof(HeadTables) * kFqMaxHeads;
            if (smem_max < 80 * 1024) smem_max = 80 * 1024;
            OMNI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
            done.emplace_back(key, dev);
        }
    }
    int64_t blocks = items < 2 * (int64_t)sms ? items : 2 * (int64_t)sms;
    kern<<<(unsigned)blocks, kTcThreads, smem, st>>>(a, items, tiles);
    return check_cuda(cudaGetLastError(), "tc_quantize_kernel launch");
}

}  // namespace omni
