// Decode / short-prefill attention over the packed INT4 + QJL cache on the fifth-generation tensor cores
// (tcgen05.mma with accumulators in tensor memory), for kv heads with MANY query columns.
//
// A column is one (query head of the group, query token).  The warp-level kernel (qattn_mma.cu) serves columns eight
// at a time and dequantises the keys again for every such tile; that is the right trade for decode, where a kv head
// has one to eight columns, and the wrong one for grouped queries over several tokens (speculative decoding, short
// prefill), where 32 to 128 columns share every key.  Here the keys of a 128-key tile are dequantised ONCE into
// shared memory and multiplied against up to 128 columns by two dense contractions:
//     S[col, key]  = sum_k  Q'[col, k] * K'[key, k]        k = 128 dims + 64 sign projections   (tcgen05.mma, SS)
//     O[col, d]   += sum_key P[col, key] * V^[key, d]                                            (tcgen05.mma, TS)
// Q' = [f q | f c (q.g)] and K' = [cb[code] | +-norm] in fp16, so the QJL score correction rides in the same product
// (c = sqrt(2/pi)/128, f = scale * log2(e) / post with a power-of-two post-scale that keeps fp16 operands below 2^10).
// S, P (fp16, the A operand of the second product) and O live in tensor memory; lane c of all three is column c, and
// the two threads (c, half 0) and (c, half 1) share it: each takes 64 of a tile's 128 keys in the softmax (they hand
// each other their partial maxima through shared memory; the running sum is merged once per work item) and 64 of the
// 128 output dims when O is rescaled or read out.
//
// One CTA of 256 threads per SM (two warps per scheduler: the phases below are latency-bound, not throughput-bound).
// Per tile: thread (k, 0) dequantises the K' row of key k (table lookups as in the warp-level kernel: byte -> half2 of
// two centroids, table replicated per lane; K-major core-matrix layout), thread (k, 1) its V^ row (MN-major); one
// thread issues the MMAs; completion comes back through mbarriers
// (tcgen05.commit), every wait on them bounded.  The q.g projections of the prologue are a tcgen05 product as well
// (Q against the +-1 matrix G expanded to fp16).  Operand layouts are the canonical no-swizzle forms: K-major
// ((8 rows x 16 B) core matrices, LBO between the two K chunks of an instruction, SBO between row groups) and
// MN-major (8 K-rows x 16 B core matrices, SBO between MN chunks, LBO between K groups).
//
// Covers: V rows in the reference or the pair layout, any S, ragged lengths, cache slots, split-K (static
// assignment), rotation folding.  Wide codebooks (a centroid of magnitude 8 or
// more) make the grid stand down exactly like the warp-level kernel; the fp32 kernel launched behind it takes over.
#include "qattn.cuh"
#include <mutex>
#include <utility>
#include <vector>

namespace omni {

constexpr int kUTile = 128;                    // keys per tile = columns per work item (at most) = tensor-memory lanes
constexpr int kUThreads = 256;                 // threads per CTA: two per column / key, thread (x = tid & 127, half = tid >> 7)
constexpr int kUKdim = 192;                    // contraction length of the score product: 128 dims + 64 projections
constexpr uint32_t kULbo = 128;                // K-major operands: bytes between the two 8-element K chunks of an MMA
constexpr uint32_t kUSbo = (kUKdim / 8) * 128; // ... and between groups of 8 rows (24 core matrices of 128 B)
constexpr uint32_t kUQBytes = 128 * kUKdim * 2;
constexpr uint32_t kUKBytes = 128 * kUKdim * 2;
constexpr uint32_t kUVSbo = 128;               // MN-major V^: bytes between chunks of 8 dims
constexpr uint32_t kUVLbo = 16 * 128;          // ... and between groups of 8 keys
constexpr uint32_t kUVBytes = 128 * 128 * 2;
constexpr uint32_t kUSignTabBytes = 256 * 16;  // byte of 8 sign bits -> four words of fp16 sign masks
constexpr uint32_t kUXchBytes = 2 * kUTile * 4;  // one float per thread: values the two threads of a column hand each other
constexpr uint32_t kUSmallBytes = kUSignTabBytes + 256 + kUXchBytes + kUTile * 4;
constexpr int kULutSpan = 65536;
constexpr int kUSmemBytes = 227 * 1024;
constexpr uint32_t kUTmemCols = 512;
constexpr uint32_t kUColS = 0, kUColP = 128, kUColO = 256;     // tensor-memory columns of S (128), P (64), O (128)
constexpr uint32_t kUWaitLimit = 1u << 22;
constexpr float kULog2e = 1.4426950408889634f;
constexpr float kUSlack = 6.f;

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ void u_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool u_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool u_mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kUWaitLimit; ++i)
        if (u_mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void u_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" :: "r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                    "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                    "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                    "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                 : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
                 :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                    "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}
// shared-memory matrix descriptor, no swizzle: start address, leading / stride byte offsets (all in 16-byte units)
__device__ __forceinline__ uint64_t u_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// instruction descriptor, kind::f16: fp16 A and B, fp32 accumulator, A K-major, B K-major or MN-major
__host__ __device__ constexpr uint32_t u_idesc(int M, int N, bool b_mn_major) {
    return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ uint4 u_ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float u_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t u_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <int WHICH>
__device__ __forceinline__ uint32_t u_lut(uint32_t lut_lane, uint32_t w) {
    const uint32_t addr = __byte_perm(w, lut_lane, 0x7604 | (WHICH << 4));
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void u_sts16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 u_lds16_const(uint32_t addr) {        // tables that do not change while they are read
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 u_lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// eight centroids of one packed word as a 16-byte chunk of fp16
__device__ __forceinline__ void u_dequant_store(uint32_t dst, uint32_t lut_lane, uint32_t w) {
    u_sts16(dst, u_lut<0>(lut_lane, w), u_lut<1>(lut_lane, w), u_lut<2>(lut_lane, w), u_lut<3>(lut_lane, w));
}
// A whole 64-byte row (16 packed words -> 16 chunks `stride` bytes apart) in two batches of 32 table lookups followed by
// their 8 stores: a store cannot be moved above a load of the same memory space, so lookups written chunk by chunk
// would each wait out the table's latency before the next chunk's could be issued.
__device__ __forceinline__ void u_dequant_row(uint32_t dst, uint32_t stride, uint32_t lut_lane, const uint4 (&nw)[4]) {
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {
        const uint32_t w[8] = {nw[2 * hb].x, nw[2 * hb].y, nw[2 * hb].z, nw[2 * hb].w,
                               nw[2 * hb + 1].x, nw[2 * hb + 1].y, nw[2 * hb + 1].z, nw[2 * hb + 1].w};
        uint32_t l[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            l[i][0] = u_lut<0>(lut_lane, w[i]); l[i][1] = u_lut<1>(lut_lane, w[i]);
            l[i][2] = u_lut<2>(lut_lane, w[i]); l[i][3] = u_lut<3>(lut_lane, w[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) u_sts16(dst + (uint32_t)(8 * hb + i) * stride, l[i][0], l[i][1], l[i][2], l[i][3]);
    }
}
// in-thread normalised 128-point Walsh-Hadamard transform (stage order h = 1 .. 64, one rounding per operation)
__device__ __forceinline__ void u_wht128(float (&v)[128]) {
#pragma unroll
    for (int h = 1; h < 128; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i | h];
                v[i] = __fadd_rn(a, b);
                v[i | h] = __fsub_rn(a, b);
            }
        }
    }
    const float s = __uint_as_float(OMNI_WHT_SCALE_BITS);
#pragma unroll
    for (int i = 0; i < 128; ++i) v[i] = __fmul_rn(v[i], s);
}

template <int DT>
__global__ void __launch_bounds__(kUThreads, 1) qattn_umma_kernel(AttnArgs a, int64_t n_items) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int x = tid & (kUTile - 1), half = tid >> 7;             // column / key of this thread, and which half of the work
    {   // a codebook the fp16 tables cannot hold to the error budget: the grid stands down (see qattn.cuh)
        const int n_cb = a.cb_per_head ? a.Hkv * 16 : 16;
        bool wide = false;
        for (int i = tid; i < n_cb; i += kUThreads) wide = wide || centroid_is_wide(__ldg(a.codebooks + i));
        if (__syncthreads_or(wide)) return;
    }
    // ---- shared memory carve-up: the lookup table takes the 64 KiB at the first 64 KiB boundary of the window, the
    //      operand tiles go in front of it or behind it, wherever each fits -------------------------------------------
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t lut_off = (kULutSpan - (smem_base & (kULutSpan - 1))) & (kULutSpan - 1);
    uint32_t front = 0, back = lut_off + kULutSpan;
    auto place = [&](uint32_t bytes) -> uint32_t {
        uint32_t at;
        if (front + bytes <= lut_off) { at = front; front += bytes; }
        else { at = back; back += bytes; }
        return at;
    };
    const uint32_t off_q = place(kUQBytes), off_k = place(kUKBytes), off_v = place(kUVBytes), off_small = place(kUSmallBytes);
    if (back > (uint32_t)kUSmemBytes) {            // cannot happen for the window bases the hardware uses; say so and leave
        if (tid == 0 && a.status) atomicExch(a.status, OMNI_ERR_DEVICE_WAIT);
        return;
    }
    const uint32_t sQ = smem_base + off_q, sK = smem_base + off_k, sV = smem_base + off_v;
    const uint32_t sSign = smem_base + off_small;                       // sign-mask table
    const uint32_t bar_s = sSign + kUSignTabBytes, bar_o = bar_s + 8;   // mbarriers
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_small + kUSignTabBytes + 16);
    float* xch = reinterpret_cast<float*>(smem + off_small + kUSignTabBytes + 256);          // [256] per-thread hand-over
    float* post_s = xch + kUThreads;                                                          // [128] per-column post-scale
    const uint32_t lut_lane = smem_base + lut_off + 4 * lane;

    // sign-mask table: byte b -> words p = 0..3 with bit 15 / 31 set where bit 2p / 2p+1 of b is CLEAR (a clear bit
    // means -1: xor with a positive fp16 pair flips those halves)
    for (int b = tid; b < 256; b += kUThreads) {
        uint32_t w[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) w[p] = ((((~b) >> (2 * p)) & 1u) << 15) | ((((~b) >> (2 * p + 1)) & 1u) << 31);
        u_sts16(sSign + 16 * b, w[0], w[1], w[2], w[3]);
    }
    if (tid == 0) {
        u_mbar_init(bar_s, 1);
        u_mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     :: "r"((uint32_t)__cvta_generic_to_shared(tmem_slot)), "r"(kUTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_lane = tmem + ((uint32_t)(32 * (warp & 3)) << 16); // this warp's 32 lanes: lane x = column x
    uint32_t ph_s = 0, ph_o = 0;                                        // parities of the next completions
    bool ok = true;                                                     // false once a bounded wait has expired

    const int Gq = a.Hq / a.Hkv;
    const int ncols_all = Gq * a.T;
    const int n_ctiles = (ncols_all + kUTile - 1) / kUTile;
    const float qs = a.scale * kULog2e;
    const int ksteps = a.with_qjl ? kUKdim / 16 : 128 / 16;
    int lut_head = -1;
    float lut_scale = 1.f;                          // the centroid tables hold cb * lut_scale (see lut_scale_of)

    for (int64_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        int64_t rest = item;
        const int col0 = kUTile * (int)(rest % n_ctiles);
        rest /= n_ctiles;
        const int ncols = ncols_all - col0 < kUTile ? ncols_all - col0 : kUTile;
        const int hkv = (int)(rest % a.Hkv);
        rest /= a.Hkv;
        const int split = (int)(rest % a.n_splits);
        const int64_t b = rest / a.n_splits;
        int64_t len = a.seq_lens ? (int64_t)a.seq_lens[b] : a.S;
        len = len < 0 ? 0 : (len > a.S ? a.S : len);
        int64_t per = (len + a.n_splits - 1) / a.n_splits;
        per = (per + 31) / 32 * 32;
        const int64_t s0 = (int64_t)split * per;
        const int64_t s1 = (s0 + per < len) ? s0 + per : len;
        const int64_t slot = a.cache_slots ? (int64_t)a.cache_slots[b] : b;
        const int64_t row0 = slot * a.ks_b + (int64_t)hkv * a.ks_h + s0;
        const int nkeys = s1 > s0 ? (int)(s1 - s0) : 0;
        const int64_t paired_limit = (len & ~(int64_t)7) - s0;      // pair layout: key offsets of this split below this
        const bool col_on = x < ncols;
        const int cg = col0 + (col_on ? x : 0);
        const int64_t qrow = (b * a.Hq + (int64_t)hkv * Gq + cg / a.T) * a.T + (cg % a.T);

        // ---- lookup table of this head's centroids (rebuilt only when the head's codebook changes) -----------------
        const int want_head = a.cb_per_head ? hkv : 0;
        if (want_head != lut_head) {
            __syncthreads();
            const float* cb = a.codebooks + want_head * 16;
            lut_scale = lut_scale_of(cb);
            uint32_t* lut = reinterpret_cast<uint32_t*>(smem + lut_off);
            for (int i = tid; i < 256 * 8; i += kUThreads) {
                const int byte = i >> 3, quad = i & 7;
                const uint32_t v = u_half2(__ldg(cb + (byte & 15)) * lut_scale, __ldg(cb + (byte >> 4)) * lut_scale);
                *reinterpret_cast<uint4*>(lut + byte * 64 + 4 * quad) = make_uint4(v, v, v, v);
            }
            lut_head = want_head;
            __syncthreads();
        }

        // ---- prologue: row x of Q' (zeros for unused columns), built by the column's first thread -----------------------
        float post = 1.f;
        if (half == 0) {
            float qv[128];
            if (col_on) {
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    float t4[4];
                    Elem<DT>::load4(a.q, qrow * kHeadDim + 4 * k, t4);
                    qv[4 * k] = t4[0]; qv[4 * k + 1] = t4[1]; qv[4 * k + 2] = t4[2]; qv[4 * k + 3] = t4[3];
                }
                if (a.rotate_q) u_wht128(qv);
            } else {
#pragma unroll
                for (int k = 0; k < 128; ++k) qv[k] = 0.f;
            }
            float amax = 0.f;
#pragma unroll
            for (int k = 0; k < 128; ++k) amax = fmaxf(amax, fabsf(qv[k]));
            const float mx = amax * fabsf(qs) / lut_scale;
            if (mx > 1024.f) post = exp2f(ceilf(log2f(mx * (1.f / 1024.f))));
            const float f = qs / post / lut_scale;          // score operands: the table's factor taken back out
            const uint32_t rowq = sQ + (uint32_t)(x >> 3) * kUSbo + (uint32_t)(x & 7) * 16;
#pragma unroll
            for (int kc = 0; kc < 16; ++kc)
                u_sts16(rowq + kc * kULbo, u_half2(qv[8 * kc] * f, qv[8 * kc + 1] * f), u_half2(qv[8 * kc + 2] * f, qv[8 * kc + 3] * f),
                        u_half2(qv[8 * kc + 4] * f, qv[8 * kc + 5] * f), u_half2(qv[8 * kc + 6] * f, qv[8 * kc + 7] * f));
            post_s[x] = post;
        }
        __syncthreads();                                  // Q' rows and post-scales are complete
        post = post_s[x];
        if (a.with_qjl) {
            // G of this (user, kv head) as +-1 fp16, K-major [64 projections x 128 dims] in the K' buffer; then
            // (f q).G^T on the tensor cores into S columns 0..63, scaled by c into the last 64 K columns of Q'
            const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
            const uint32_t* grow = a.g_rows + (size_t)seed_of(uid, hkv) * kQjlDim * 4;
            const int pi = tid >> 2, quarter = tid & 3;       // projection row, and which 32 of its 128 signs
            const uint32_t rowg = sK + (uint32_t)(pi >> 3) * kUSbo + (uint32_t)(pi & 7) * 16;
            {
                const uint32_t gw = __ldg(grow + pi * 4 + quarter);
#pragma unroll
                for (int by = 0; by < 4; ++by) {
                    const uint4 m = u_lds16(sSign + 16 * ((gw >> (8 * by)) & 0xFFu));
                    u_sts16(rowg + (uint32_t)(4 * quarter + by) * kULbo, 0x3C003C00u ^ m.x, 0x3C003C00u ^ m.y, 0x3C003C00u ^ m.z, 0x3C003C00u ^ m.w);
                }
            }
            u_fence_async_smem();
            __syncthreads();
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    tc_mma_ss(tmem + kUColS, u_desc(sQ + ks * 2 * kULbo, kULbo, kUSbo), u_desc(sK + ks * 2 * kULbo, kULbo, kUSbo),
                              u_idesc(128, 64, false), ks > 0);
                tc_commit(bar_s);
            }
            ok = __syncthreads_and(u_mbar_wait_bounded(bar_s, ph_s)) != 0;
            ph_s ^= 1u;
            if (!ok) break;
            tc_fence_after();
            const uint32_t rowq = sQ + (uint32_t)(x >> 3) * kUSbo + (uint32_t)(x & 7) * 16;
            const float qjl_mul = kQjlCoef * lut_scale;     // the sign term does not pass through the centroid table
            {
                const int j = half;                         // each thread of the column takes 32 of its 64 projections
                uint32_t v[32];
                tc_ld32(t_lane + kUColS + 32 * j, v);
                tc_wait_ld();
#pragma unroll
                for (int kc = 0; kc < 4; ++kc) {
                    uint32_t h[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        h[e] = u_half2(__uint_as_float(v[8 * kc + 2 * e]) * qjl_mul, __uint_as_float(v[8 * kc + 2 * e + 1]) * qjl_mul);
                    u_sts16(rowq + (uint32_t)(16 + 4 * j + kc) * kULbo, h[0], h[1], h[2], h[3]);
                }
            }
            tc_fence_before();
            __syncthreads();                         // the K' buffer (it held G) may now be overwritten by the first tile
        }

        // ---- key tiles ---------------------------------------------------------------------------------------------
        float m_run = -INFINITY, l_run = 0.f;
        bool o_valid = false;                        // O holds a product already (false: the next one overwrites it)
        // the packed bytes of key x of a tile, fetched one tile ahead (keys past the end repeat the last one): the K
        // nibbles, sign bytes and norm by the key's first thread, the V nibbles by its second
        uint4 nw[4];
        uint2 sb = make_uint2(0u, 0u);
        float nrm = 0.f;
        auto fetch_tile = [&](int k0) {
            const int nv = nkeys - k0 < kUTile ? nkeys - k0 : kUTile;
            const int64_t ridx = row0 + k0 + (x < nv ? x : nv - 1);
            const uint4* np = reinterpret_cast<const uint4*>((half == 0 ? a.k_nib : a.v_nib) + ridx * kNibBytes);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) nw[c4] = u_ldg16(np + c4);
            if (half == 0 && a.with_qjl) {
                sb = __ldg(reinterpret_cast<const uint2*>(a.k_qjl + ridx * kQjlBytes));
                nrm = fminf(__ldg(a.k_norms + ridx), 65504.f);
            }
        };
        if (nkeys > 0) fetch_tile(0);
        for (int k0 = 0; k0 < nkeys; k0 += kUTile) {
            const int nvalid = nkeys - k0 < kUTile ? nkeys - k0 : kUTile;
            bool mine_ok = true;                         // this thread's own bounded wait (made uniform at the next barrier)
            if (half == 0) {
                const uint32_t rowk = sK + (uint32_t)(x >> 3) * kUSbo + (uint32_t)(x & 7) * 16;
                u_dequant_row(rowk, kULbo, lut_lane, nw);
                if (a.with_qjl) {
                    const uint32_t n2 = u_half2(nrm, nrm);
                    const uint32_t sw[2] = {sb.x, sb.y};
                    uint4 m[8];                              // all eight mask lookups before the first store (see u_dequant_row)
#pragma unroll
                    for (int j = 0; j < 8; ++j) m[j] = u_lds16_const(sSign + 16 * ((sw[j >> 2] >> (8 * (j & 3))) & 0xFFu));
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        u_sts16(rowk + (uint32_t)(16 + j) * kULbo, n2 ^ m[j].x, n2 ^ m[j].y, n2 ^ m[j].z, n2 ^ m[j].w);
                }
            } else {
            // V^ may be overwritten once the previous tile's second product has read it: only the threads that write it
            // wait here (the K' rows are dequantised meanwhile); every thread tracks the parity
            if (o_valid) {
                mine_ok = u_mbar_wait_bounded(bar_o, ph_o);
                tc_fence_after();
            }
            const uint32_t rowv = sV + (uint32_t)(x & 7) * 16 + (uint32_t)(x >> 3) * kUVLbo;
            // Pair layout of V (groups of eight keys that lie completely below the user's length): the row of a pair's
            // first key holds the even-d nibbles of both keys, the row of the second key the odd-d ones, so a table
            // lookup yields (first key, second key) at one dim.  The two threads of a pair (lanes l and l ^ 3) exchange
            // their lookups and each keeps its own key's halves: (own low, other low) for the first key, (other high,
            // own high) for the second.  A group is paired as a whole, and groups coincide with runs of eight lanes.
            const bool v_pair = a.v_paired && (int64_t)(k0 + x) < paired_limit;
            if (__ballot_sync(0xffffffffu, v_pair) != 0u) {
                const uint32_t sel = v_pair ? ((x & 2) ? 0x3276u : 0x5410u) : 0x3210u;
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    const uint32_t ws[8] = {nw[2 * hb].x, nw[2 * hb].y, nw[2 * hb].z, nw[2 * hb].w,
                                            nw[2 * hb + 1].x, nw[2 * hb + 1].y, nw[2 * hb + 1].z, nw[2 * hb + 1].w};
                    uint32_t l[8][4];                        // 32 lookups, then their exchanges and eight stores
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        l[e][0] = u_lut<0>(lut_lane, ws[e]); l[e][1] = u_lut<1>(lut_lane, ws[e]);
                        l[e][2] = u_lut<2>(lut_lane, ws[e]); l[e][3] = u_lut<3>(lut_lane, ws[e]);
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) l[e][k] = __byte_perm(l[e][k], __shfl_xor_sync(0xffffffffu, l[e][k], 3), sel);
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) u_sts16(rowv + (uint32_t)(8 * hb + e) * kUVSbo, l[e][0], l[e][1], l[e][2], l[e][3]);
                }
            } else {
                u_dequant_row(rowv, kUVSbo, lut_lane, nw);
            }
            }
            if (o_valid) ph_o ^= 1u;
            if (k0 + kUTile < nkeys) fetch_tile(k0 + kUTile);            // in flight during the products and the softmax
            u_fence_async_smem();
            tc_fence_before();
            ok = __syncthreads_and(mine_ok) != 0;
            if (!ok) break;
            if (tid == 0) {
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks)
                    tc_mma_ss(tmem + kUColS, u_desc(sQ + ks * 2 * kULbo, kULbo, kUSbo), u_desc(sK + ks * 2 * kULbo, kULbo, kUSbo),
                              u_idesc(128, 128, false), ks > 0);
                tc_commit(bar_s);
            }
            ok = __syncthreads_and(u_mbar_wait_bounded(bar_s, ph_s)) != 0;
            ph_s ^= 1u;
            if (!ok) break;
            tc_fence_after();

            // ---- online softmax of column x over the tile's keys, 64 per thread: first the tile maximum (the two
            //      threads of a column hand each other theirs), then the weights ------------------------------------
            float tmax = -INFINITY;
            uint32_t sv[2][32];                                // this thread's 64 scores: both loads in flight, one wait
            tc_ld32(t_lane + kUColS + 64 * half, sv[0]);
            tc_ld32(t_lane + kUColS + 64 * half + 32, sv[1]);
            tc_wait_ld();
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int j = 2 * half + jj;
                uint32_t (&v)[32] = sv[jj];
                if (nvalid == kUTile) {                        // full tile: no per-key bound checks
                    float t0 = tmax, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        t0 = fmaxf(t0, __uint_as_float(v[i]));     t1 = fmaxf(t1, __uint_as_float(v[i + 1]));
                        t2 = fmaxf(t2, __uint_as_float(v[i + 2])); t3 = fmaxf(t3, __uint_as_float(v[i + 3]));
                    }
                    tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (32 * j + i < nvalid) tmax = fmaxf(tmax, __uint_as_float(v[i]));
                }
            }
            // The column's maximum over the tile is the larger of its two threads' maxima; it exceeds the threshold
            // exactly when one of them does, so the hand-over (and its barrier) is needed only when some thread's does.
            tmax *= post;
            if (__syncthreads_or(col_on && tmax > m_run + kUSlack)) {
                xch[tid] = tmax;
                __syncthreads();
                tmax = fmaxf(tmax, xch[tid ^ kUTile]);
                const bool raise = col_on && tmax > m_run + kUSlack;
                // lazy reference maximum: raised only when a score exceeds it by 2^kUSlack; the accumulated row of O
                // and the running sum are rescaled (lanes that keep their maximum multiply by one)
                const float m_new = raise ? fmaxf(m_run, tmax) : m_run;
                const float alpha = raise ? u_ex2(m_run - m_new) : 1.f;
                l_run *= alpha;
                m_run = m_new;
                if (o_valid) {
#pragma unroll 1
                    for (int jj = 0; jj < 2; ++jj) {
                        const int j = 2 * half + jj;           // this thread's 64 of the 128 output dims
                        uint32_t v[32];
                        tc_ld32(t_lane + kUColO + 32 * j, v);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tc_st32(t_lane + kUColO + 32 * j, v);
                    }
                    tc_wait_st();
                }
            }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int j = 2 * half + jj;
                uint32_t (&v)[32] = sv[jj];                    // the scores are still in registers from the first pass
                uint32_t pk[16];
                if (nvalid == kUTile) {                        // full tile; unused columns carry the maximum +inf: weights 0
                    const float mneg = col_on ? -m_run : -INFINITY;
                    float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const float p0 = u_ex2(fmaf(__uint_as_float(v[2 * i]), post, mneg));
                        const float p1 = u_ex2(fmaf(__uint_as_float(v[2 * i + 1]), post, mneg));
                        const float p2 = u_ex2(fmaf(__uint_as_float(v[2 * i + 2]), post, mneg));
                        const float p3 = u_ex2(fmaf(__uint_as_float(v[2 * i + 3]), post, mneg));
                        pk[i] = u_half2(p0, p1);
                        pk[i + 1] = u_half2(p2, p3);
                        // the normaliser sums the weights as the second product sees them (rounded to fp16)
                        const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&pk[i]));
                        const float2 r23 = __half22float2(*reinterpret_cast<const __half2*>(&pk[i + 1]));
                        l0 += r01.x; l1 += r01.y; l2 += r23.x; l3 += r23.y;
                    }
                    l_run += (l0 + l1) + (l2 + l3);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float p0 = 0.f, p1 = 0.f;
                        if (col_on) {
                            if (32 * j + 2 * i < nvalid) p0 = u_ex2(fmaf(__uint_as_float(v[2 * i]), post, -m_run));
                            if (32 * j + 2 * i + 1 < nvalid) p1 = u_ex2(fmaf(__uint_as_float(v[2 * i + 1]), post, -m_run));
                        }
                        pk[i] = u_half2(p0, p1);
                        const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&pk[i]));
                        l_run += r01.x + r01.y;
                    }
                }
                tc_st16(t_lane + kUColP + 16 * j, pk);
            }
            tc_wait_st();
            tc_fence_before();
            __syncthreads();
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    tc_mma_ts(tmem + kUColO, tmem + kUColP + 8 * ks, u_desc(sV + ks * 2 * kUVLbo, kUVLbo, kUVSbo),
                              u_idesc(128, 128, true), (o_valid || ks > 0) ? 1u : 0u);
                tc_commit(bar_o);
            }
            o_valid = true;
        }
        if (!ok) break;
        if (o_valid) {
            ok = __syncthreads_and(u_mbar_wait_bounded(bar_o, ph_o)) != 0;
            ph_o ^= 1u;
            if (!ok) break;
            tc_fence_after();
        }

        // ---- epilogue: row x of O -> the output row of column x (or its split-K partial state); the column's two
        //      threads add up their sums of weights and write 64 dims each -------------------------------------------
        xch[tid] = l_run;
        __syncthreads();
        const float l_tot = l_run + xch[tid ^ kUTile];
        float* dst = nullptr;
        float mul = 0.f;
        if (a.n_splits == 1) {
            dst = a.out + qrow * kHeadDim;
            mul = l_tot > 0.f ? 1.f / (l_tot * lut_scale) : 0.f;
        } else {
            float* w = a.ws + (qrow * a.n_splits + split) * kWsStride;
            dst = w;
            mul = 1.f / lut_scale;
            if (col_on && half == 0) { w[128] = m_run * 0.6931471805599453f; w[129] = l_tot; }
        }
        if (a.unrotate_out && a.n_splits == 1) {
          if (half == 0) {                              // the inverse rotation needs the whole row in one thread
            float o[128];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t v[32];
                if (o_valid) { tc_ld32(t_lane + kUColO + 32 * j, v); tc_wait_ld(); }
#pragma unroll
                for (int i = 0; i < 32; ++i) o[32 * j + i] = o_valid ? __uint_as_float(v[i]) * mul : 0.f;
            }
            u_wht128(o);
            if (col_on) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
          }
        } else {
#pragma unroll 1
            for (int jj = 0; jj < 2; ++jj) {
                const int j = 2 * half + jj;
                uint32_t v[32];
                if (o_valid) { tc_ld32(t_lane + kUColO + 32 * j, v); tc_wait_ld(); }
                if (col_on) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(dst + 32 * j + 4 * i) =
                            o_valid ? make_float4(__uint_as_float(v[4 * i]) * mul, __uint_as_float(v[4 * i + 1]) * mul,
                                                  __uint_as_float(v[4 * i + 2]) * mul, __uint_as_float(v[4 * i + 3]) * mul)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
        tc_fence_before();
        __syncthreads();                             // every lane has read O and S before the next item reuses them
    }

    if (!ok && tid == 0 && a.status) atomicExch(a.status, OMNI_ERR_DEVICE_WAIT);
    // hand the tensor memory back (the allocating warp), after every thread is done with it
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" :: "r"(tmem), "r"(kUTmemCols) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
bool umma_eligible(const AttnArgs& a) {
    const int64_t cols = (int64_t)(a.Hq / a.Hkv) * a.T;
    return cols >= 1 && cols <= 4096 && a.Hkv <= 65535;
}

template <int DT>
static int32_t launch_umma_t(const AttnArgs& a, cudaStream_t st) {
    int dev = 0, sms = 148;
    OMNI_CUDA(cudaGetDevice(&dev));
    OMNI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t n_ctiles = ((int64_t)(a.Hq / a.Hkv) * a.T + kUTile - 1) / kUTile;
    const int64_t items = a.B * a.n_splits * a.Hkv * n_ctiles;
    auto kern = qattn_umma_kernel<DT>;
    {
        static std::mutex mu;
        static std::vector<std::pair<const void*, int>> done;
        const void* key = reinterpret_cast<const void*>(kern);
        std::lock_guard<std::mutex> lk(mu);
        bool seen = false;
        for (const auto& p : done) seen = seen || (p.first == key && p.second == dev);
        if (!seen) {
            OMNI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kUSmemBytes));
            done.emplace_back(key, dev);
        }
    }
    const int64_t ctas = items < sms ? items : sms;
    kern<<<(unsigned)ctas, kUThreads, kUSmemBytes, st>>>(a, items);
    return check_cuda(cudaGetLastError(), "qattn_umma_kernel launch");
}

int32_t launch_umma(const AttnArgs& a, cudaStream_t st) {
    switch (a.q_dtype) {
        case OMNI_F32:  return launch_umma_t<OMNI_F32>(a, st);
        case OMNI_BF16: return launch_umma_t<OMNI_BF16>(a, st);
        case OMNI_F16:  return launch_umma_t<OMNI_F16>(a, st);
    }
    return set_error(OMNI_ERR_ARG, "qattn: unknown q dtype code %d", a.q_dtype);
}

}  // namespace omni
