// Tensor-core decode attention over the packed INT4 + QJL cache (sm_100a).
//
// One warp owns one (user, kv head, key split, tile of up to 8 query columns); a column is one (query head of
// the group, query token), and a kv head with more than 8 columns is served by several work items that read the
// same keys (the later ones from L2).  Keys are taken 16 at a time and everything is computed transposed so that
// the key axis is the MMA "M":
//     S^T[key, col]  = sum_d  K^[key, d] * q[col, d]                 (8 fp16 MMAs, A = dequantised K)
//                    + norm[key] * sum_i s_i[key] * (q.g_i)[col]      (2 int8 MMAs, A = -bit_i, B = q.g in int8)
//     O^T[d,  col]  += sum_key V^[key, d] * P[key, col]               (8 fp16 MMAs, A = dequantised V^T)
// (mma.sync m16n8k16 fp16 -> fp32 and m16n8k32 s8 -> s32).
//
// Data movement.  The 64-byte nibble rows of K and V are brought in by TMA (cp.async.bulk.tensor.2d, one
// 32-row box per array and stage = two 16-key blocks, 64-byte swizzle) into a private ring of stages per warp,
// completion tracked by one mbarrier per stage; the lane that issues a copy is lane 0 of the warp that consumes
// it, so no cross-warp handshake exists.  Sign bytes and norms (12 of the 140 bytes per key) are read with plain
// loads one stage ahead, behind one bulk L2 prefetch per work item.  Every wait on an mbarrier is bounded; when
// the bound is hit the warp records it in the status word, waits (bounded again) for its other copies and leaves.
//
// Dequantisation.  A fragments are built straight from the packed bytes with table lookups in shared memory: a
// 256-entry table maps a byte to half2(cb[low nibble], cb[high nibble]), replicated per lane so every lookup is
// bank-conflict free.  The table takes a 64 KiB region placed on a 64 KiB boundary of the shared window, so that
// a single PRMT (byte -> address bits 8..15) forms the complete address.  The contraction index of each MMA is a
// permutation of d chosen so that each thread reads 16 contiguous bytes of a key row; for V the two nibbles of a
// pair come from two different keys and the index byte is formed with one shift and one LOP3 per four lookups.
// The 64 sign bits of a key become int8 operands in registers (a multiply spreads 4 bits to the byte MSBs, PRMT
// replicates them).  The rows of the score tile are a permutation rho of the 16 keys chosen so that (a) the
// transposed softmax weights come out of MOVMATRIX in the order the V fragments need and (b) every shared-memory
// read of a stage is conflict free under the 64-byte swizzle.
//
// Work distribution.  Persistent grid, one CTA per SM.  Calls without key splits assign items statically (equal
// sizes); split-K calls draw tickets from a counter in the workspace so ragged cache lengths stay balanced.
#include "qattn.cuh"
#include <cuda.h>
#include <mutex>
#include <utility>
#include <vector>

// This file is compiled twice: as it stands, and (through qattn_mma_lora.cu, which defines OMNI_MMA_LORA as 1) with
// the per-user query update folded into the prologue.  The second set of kernels is kept apart so that the extra
// code cannot change the register allocation of the first, whose main loop sits at the register limit.
#ifndef OMNI_MMA_LORA
#define OMNI_MMA_LORA 0
#endif

namespace omni {

constexpr bool kLoraBuild = OMNI_MMA_LORA != 0;

#ifndef OMNI_MMA_WARPS
#define OMNI_MMA_WARPS 12
#endif
#ifndef OMNI_MMA_STAGES
#define OMNI_MMA_STAGES 2
#endif
constexpr int kMmaWarps = OMNI_MMA_WARPS;
constexpr int kStages = OMNI_MMA_STAGES;                 // per-warp ring of stages
constexpr int kStageKeys = 32;                           // keys per stage: two 16-key MMA blocks
constexpr int kLutSpan = 65536;                          // 256 entries x 256 B
constexpr int kStageBytes = 2 * kStageKeys * kNibBytes;  // K rows then V rows of one stage
constexpr int kWarpScratchBytes = 8 * 128 * 4 + 8 * 16;  // fp32 query rows of 8 columns (reused for q.g) + per-column scalars
// Per-warp private block, 512-byte aligned (the swizzle pattern of a stage repeats every 512 bytes):
// [kStages stages][scratch][kStages mbarriers][pad]
constexpr int kWarpBlockBytes = ((kStages * kStageBytes + kWarpScratchBytes + 8 * kStages + 511) / 512) * 512;
// Dynamic shared memory: the whole SM.  The tables take the 64 KiB that start at the first 64 KiB
// boundary of the shared window; the per-warp blocks fill the space in front of and behind them.
constexpr int kMmaSmemBytes = 227 * 1024;
static_assert(kMmaWarps * kWarpBlockBytes + kLutSpan + kWarpBlockBytes <= kMmaSmemBytes,
              "per-warp blocks do not fit beside the tables for every placement of the 64 KiB boundary");
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kWaitLimit = 1u << 20;                // try_wait attempts before a wait is declared expired

// ---- PTX wrappers ----------------------------------------------------------------------
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
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream2(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];\n" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldg_stream_f32(const void* p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds8(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
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
// Bulk L2 prefetch (issued by the TMA unit): `bytes` (multiple of 16) from a 16-byte aligned address.
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(p), "r"(bytes) : "memory");
}
// centroid-table lookup: byte WHICH of w selects the entry; lut_lane has zero bits 8..15
template <int WHICH>
__device__ __forceinline__ uint32_t lut_at(uint32_t lut_lane, uint32_t w) {
    const uint32_t addr = __byte_perm(w, lut_lane, 0x7604 | (WHICH << 4));
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));   // read-only table: free to be scheduled early
    return v;
}
// ---- QJL correction operands --------------------------------------------------------------
// The 64 sign bits of a key go to the int8 tensor cores: A = -bit built in registers (a multiply spreads
// 4 bits to the 4 byte MSBs, PRMT replicates them), B = q.g quantised to int8 per column.
struct SignB {
    uint32_t zh[4], zl[4];  // q.g of column g, projections 16t .. 16t+15, as 16-bit integers z = 256 * zh + zl
                            // (zh signed, zl unsigned; four per word).  One 8-bit limb is not enough: the quantisation
                            // noise of the 64-term sum is multiplied by the key's residual norm, and heavy-tailed
                            // data (outlier channels) has norms of 10 and more
    int zq[4];              // accumulator seed (sum of z)/2 for columns 2t, 2t+1, 2t, 2t+1
    float cs0, cs1;         // -2 * quantisation step of columns 2t, 2t+1
};
__device__ __forceinline__ void imma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1, const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// four int8 (0 or -1) from the 4 bits of `nib` that sit at bit positions LOW..LOW+3 (LOW = 0 or 4)
template <int LOW>
__device__ __forceinline__ uint32_t neg_bits_s8(uint32_t s) {
    const uint32_t spread = (s & (0xFu << LOW)) * (LOW == 0 ? 0x10204080u : 0x01020408u);   // bit j -> MSB of byte j
    uint32_t r;
    asm("prmt.b32 %0, %1, %1, 0xBA98;\n" : "=r"(r) : "r"(spread));   // selector MSBs: replicate the byte's sign bit
    return r;                                                  // replicate each MSB
}

// four int8 of +-1 from 4 bits of a Rademacher row: bit 1 -> +1, bit 0 -> -1 (bits at LOW..LOW+3 of w)
template <int LOW>
__device__ __forceinline__ uint32_t pm1_bytes(uint32_t w) {
    const uint32_t spread = (~w & (0xFu << LOW)) * (LOW == 0 ? 0x10204080u : 0x01020408u);
    uint32_t r;
    asm("prmt.b32 %0, %1, %1, 0xBA98;\n" : "=r"(r) : "r"(spread));
    return r | 0x01010101u;
}
__device__ __forceinline__ void imma_acc_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_acc_s8u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- mbarrier / TMA ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when `limit` attempts did not see the phase complete
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = kWaitLimit) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, int32_t row, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 :: "r"(dst), "l"(map), "r"(0), "r"(row), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

// ---- per-thread view of one 16-key block ---------------------------------------------------
// Score-tile row r of the MMA holds key rho(r) of the block: rho = {0,3,1,2,4,7,5,6} for r < 8 and
// rho(r) = rho(r-8) + 8 above.  Thread (g, t) (g = lane/4, t = lane%4) therefore reads the K rows
// rho(g), rho(g)+8 and, after the transposition of the weights, the V rows rho(2t), rho(2t+1) and
// those plus 8.
__device__ __forceinline__ int rho8(int r) { return (0x65742130 >> (4 * r)) & 7; }

struct KeyBlock {           // packed bytes of one 16-key block as this thread needs them
    uint4 ka, kb;           // K nibbles: keys rho(g) and rho(g)+8, bytes 16t..16t+15
    uint2 v0, v1, v2, v3;   // V nibbles, bytes 8g..8g+7.  Reference layout: rows of keys rho(2t), rho(2t+1), rho(2t)+8,
                            // rho(2t+1)+8.  Pair layout (VPAIR): v0 / v1 = even-d / odd-d nibbles of the key pair
                            // (rho(2t), rho(2t+1)), low nibble = first key; v2 / v3 the same eight keys further on
    uint32_t sa, sb;        // K sign bits: keys rho(g), rho(g)+8, bits 16t..16t+15
    float na, nb;           // K residual norms: keys rho(g), rho(g)+8
};

// Sign bytes and norms of one block (plain loads, kept one block ahead of their use).
struct AuxRegs { uint32_t sa, sb; float na, nb; };
__device__ __forceinline__ void load_aux(AuxRegs& x, const uint8_t* ps, const float* pn) {
    x.sa = ldg_stream2(ps);
    x.sb = ldg_stream2(ps + 8 * kQjlBytes);
    x.na = ldg_stream_f32(pn);
    x.nb = ldg_stream_f32(pn + 8);
}

// Partial last block, read with plain loads: rows past the end are clamped to the last valid key
// (their scores are masked).  row0 = first row of the block in the packed arrays.
// two rows of the reference layout -> the pair layout of the same 16 nibble columns
__device__ __forceinline__ void pair_rows(uint2& x, uint2& y) {
    const uint2 A = x, B = y;
    x.x = (A.x & 0x0F0F0F0Fu) | ((B.x << 4) & 0xF0F0F0F0u);  y.x = ((A.x >> 4) & 0x0F0F0F0Fu) | (B.x & 0xF0F0F0F0u);
    x.y = (A.y & 0x0F0F0F0Fu) | ((B.y << 4) & 0xF0F0F0F0u);  y.y = ((A.y >> 4) & 0x0F0F0F0Fu) | (B.y & 0xF0F0F0F0u);
}

// `paired_rows` (0, 8 or 16; VPAIR only): how many rows from row0 on are stored in the pair layout -- the groups of
// eight keys that lie completely below the user's length.  The block comes out in the layout the template says:
// with VPAIR the groups still in the reference layout (the user's last, incomplete group) are paired here.
template <bool QJL, bool VPAIR>
__device__ __forceinline__ void load_tail_block(KeyBlock& kb, const AttnArgs& a, int64_t row0, int nvalid, int paired_rows,
                                                int kr, int va, int vb, int g, int t) {
    const int last = nvalid - 1;
    const int64_t rk = row0 + min(kr, last), rk8 = row0 + min(kr + 8, last);
    kb.ka = ldg_stream16(a.k_nib + rk * kNibBytes + 16 * t);
    kb.kb = ldg_stream16(a.k_nib + rk8 * kNibBytes + 16 * t);
    const bool p0 = VPAIR && paired_rows >= 8, p1 = VPAIR && paired_rows >= 16;      // stored pair-wise: every row exists
    kb.v0 = ldg_stream8(a.v_nib + (row0 + (p0 ? va : min(va, last))) * kNibBytes + 8 * g);
    kb.v1 = ldg_stream8(a.v_nib + (row0 + (p0 ? vb : min(vb, last))) * kNibBytes + 8 * g);
    kb.v2 = ldg_stream8(a.v_nib + (row0 + (p1 ? va + 8 : min(va + 8, last))) * kNibBytes + 8 * g);
    kb.v3 = ldg_stream8(a.v_nib + (row0 + (p1 ? vb + 8 : min(vb + 8, last))) * kNibBytes + 8 * g);
    if (VPAIR && !p0) pair_rows(kb.v0, kb.v1);
    if (VPAIR && !p1) pair_rows(kb.v2, kb.v3);
    if (QJL) {
        kb.sa = ldg_stream2(a.k_qjl + rk * kQjlBytes + 2 * t);
        kb.sb = ldg_stream2(a.k_qjl + rk8 * kQjlBytes + 2 * t);
        kb.na = ldg_stream_f32(a.k_norms + rk);
        kb.nb = ldg_stream_f32(a.k_norms + rk8);
    }
}

struct WarpState {
    float O[8][4];          // O^T accumulators: [m-tile][c-fragment]
    float m0, m1, l0, l1;   // reference maximum (log2 units) and partial sums for columns 2t, 2t+1
};

constexpr float kLazyMaxSlack = 6.f;   // log2 units a score may exceed the reference maximum before it is raised


// ONECOL: the kv head has a single query column (plain decode without query grouping).  Only column 0 of the
// score tile is real then, so the scalar softmax work of the second column of every lane is left out.
template <bool QJL, bool TAIL, bool ONECOL, bool VPAIR>
__device__ __forceinline__ void process_key_block(const KeyBlock& kb, WarpState& st, const uint32_t (&qB)[8][2],
                                                  const SignB& sg, float post0, float post1,
                                                  uint32_t lut_lane, int nvalid, int kl) {
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
        // sum_i s_i z_i = -2 * (sum_i (-bit_i) z_i + Z/2): the seed Z/2 rides in as the MMA addend
        const uint32_t sa8 = kb.sa >> 8, sb8 = kb.sb >> 8;
        const uint32_t a0 = neg_bits_s8<0>(kb.sa), a1 = neg_bits_s8<0>(kb.sb), a2 = neg_bits_s8<4>(kb.sa), a3 = neg_bits_s8<4>(kb.sb);
        const uint32_t a4 = neg_bits_s8<0>(sa8), a5 = neg_bits_s8<0>(sb8), a6 = neg_bits_s8<4>(sa8), a7 = neg_bits_s8<4>(sb8);
        int dh[4] = {0, 0, 0, 0}, dl[4] = {sg.zq[0], sg.zq[1], sg.zq[2], sg.zq[3]};
        imma_acc_s8s8(dh, a0, a1, a2, a3, sg.zh[0], sg.zh[1]);
        imma_acc_s8u8(dl, a0, a1, a2, a3, sg.zl[0], sg.zl[1]);
        imma_acc_s8s8(dh, a4, a5, a6, a7, sg.zh[2], sg.zh[3]);
        imma_acc_s8u8(dl, a4, a5, a6, a7, sg.zl[2], sg.zl[3]);
        int d1[4];
        d1[0] = dh[0] * 256 + dl[0]; d1[2] = dh[2] * 256 + dl[2];
        if (!ONECOL) { d1[1] = dh[1] * 256 + dl[1]; d1[3] = dh[3] * 256 + dl[3]; }
        s00 = post0 * fmaf(kb.na * sg.cs0, (float)d1[0], cd[0] + ce[0]);
        s80 = post0 * fmaf(kb.nb * sg.cs0, (float)d1[2], cd[2] + ce[2]);
        if (!ONECOL) {
            s01 = post1 * fmaf(kb.na * sg.cs1, (float)d1[1], cd[1] + ce[1]);
            s81 = post1 * fmaf(kb.nb * sg.cs1, (float)d1[3], cd[3] + ce[3]);
        }
    } else {
        s00 = post0 * (cd[0] + ce[0]); s80 = post0 * (cd[2] + ce[2]);
        if (!ONECOL) { s01 = post1 * (cd[1] + ce[1]); s81 = post1 * (cd[3] + ce[3]); }
    }
    if (ONECOL) { s01 = -INFINITY; s81 = -INFINITY; }
    if (TAIL) {
        if (kl >= nvalid) { s00 = -INFINITY; s01 = -INFINITY; }
        if (kl + 8 >= nvalid) { s80 = -INFINITY; s81 = -INFINITY; }
    }
    // Lazy running maximum: the reference point m of a column is raised only when some score
    // exceeds it by more than kLazyMaxSlack, so the cross-lane reduction and the rescale of the
    // accumulators run on few blocks; in between, weights are at most 2^kLazyMaxSlack.
    const bool exceed = (fmaxf(s00, s80) > st.m0 + kLazyMaxSlack) ||
                        (!ONECOL && fmaxf(s01, s81) > st.m1 + kLazyMaxSlack);
    if (__any_sync(kFullMask, exceed)) {
        float mx0 = fmaxf(s00, s80), mx1 = fmaxf(s01, s81);
#pragma unroll
        for (int m = 4; m <= 16; m <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, m));
            if (!ONECOL) mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, m));
        }
        const float mn0 = fmaxf(st.m0, mx0);
        const float al0 = ex2_approx(st.m0 - mn0);
        st.l0 *= al0;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) { st.O[mt][0] *= al0; st.O[mt][2] *= al0; }
        st.m0 = mn0;
        if (!ONECOL) {
            const float mn1 = fmaxf(st.m1, mx1);
            const float al1 = ex2_approx(st.m1 - mn1);
            st.l1 *= al1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) { st.O[mt][1] *= al1; st.O[mt][3] *= al1; }
            st.m1 = mn1;
        }
    }
    const float p00 = ex2_approx(s00 - st.m0), p80 = ex2_approx(s80 - st.m0);
    const float p01 = ONECOL ? 0.f : ex2_approx(s01 - st.m1), p81 = ONECOL ? 0.f : ex2_approx(s81 - st.m1);
    // The weights enter the V product rounded to fp16; the normaliser sums the SAME rounded values, so a key that
    // carries the whole softmax returns its V row exactly instead of scaled by the rounding of its weight.
    const uint32_t ph0 = pack_half2(p00, p01), ph1 = pack_half2(p80, p81);
#ifndef OMNI_L_FROM_FP32
    {
        const __half2 h0 = *reinterpret_cast<const __half2*>(&ph0), h1 = *reinterpret_cast<const __half2*>(&ph1);
        st.l0 += __low2float(h0) + __low2float(h1);
        if (!ONECOL) st.l1 += __high2float(h0) + __high2float(h1);
    }
#else
    st.l0 += p00 + p80;
    if (!ONECOL) st.l1 += p01 + p81;
#endif
    // P^T as the B operand: transpose the two 8x8 (key x column) blocks across the warp
    const uint32_t pb0 = movmatrix_trans(ph0);
    const uint32_t pb1 = movmatrix_trans(ph1);
    // V: index byte = nibble of key A | nibble of key B << 4 (the pair layout stores exactly these bytes)
    {
        const uint32_t A[2] = {kb.v0.x, kb.v0.y}, B[2] = {kb.v1.x, kb.v1.y};
        const uint32_t C[2] = {kb.v2.x, kb.v2.y}, D[2] = {kb.v3.x, kb.v3.y};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t x01 = VPAIR ? A[h] : (A[h] & 0x0F0F0F0Fu) | ((B[h] << 4) & 0xF0F0F0F0u);
            const uint32_t y01 = VPAIR ? B[h] : ((A[h] >> 4) & 0x0F0F0F0Fu) | (B[h] & 0xF0F0F0F0u);
            const uint32_t x23 = VPAIR ? C[h] : (C[h] & 0x0F0F0F0Fu) | ((D[h] << 4) & 0xF0F0F0F0u);
            const uint32_t y23 = VPAIR ? D[h] : ((C[h] >> 4) & 0x0F0F0F0Fu) | (D[h] & 0xF0F0F0F0u);
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


// The B operands of one work item -- the scaled query columns as fp16 pairs, the q.g projections quantised to int8
// with their seeds and steps, the per-column power-of-two post-scales -- as the registers of the main loop.
struct QueryOperands {
    uint32_t qB[8][2];
    SignB sg;
    float post0, post1;
};
constexpr int kPrepWords = 32;              // 16 + 4 + 4 + 2 + 2 + 2 words per lane, padded to eight 16-byte vectors
static_assert(kPrepBytesPerUnit == kPrepWords * 4 * 32, "prepared operands: size used by the workspace layout");

// Builds them from the query rows of (user b, kv head hkv, columns col0 .. col0 + ncols).  `qrow` is this warp's
// shared scratch (8 x 128 fp32 query rows, reused for the q.g projections) and `colinfo` the per-column scalars
// behind it.  Every lane of the warp must call.
// `inv_lut` = 1 / lut_scale_of(the head's codebook): the score operands carry it, the sign correction does not.
template <int DT, bool QJL, bool LORA>
__device__ __forceinline__ void build_query_operands(const AttnArgs& a, int64_t b, int hkv, int col0, int ncols, int Gq, float qs,
                                                     float inv_lut, float* qrow, float4* colinfo, int lane, QueryOperands& qo) {
    const int g = lane >> 2, t = lane & 3;
    float* qg_s = qrow;
    uint32_t (&qB)[8][2] = qo.qB;
    SignB& sg = qo.sg;
    // ---- prologue: B operands (scaled queries, q.g projections) --------------------------------
    // 1. every column's query row goes to shared memory in fp32 together with its scalars
    // per-user low-rank update: the up projections of all columns first (left where the rows go next), added below
    const bool updated = LORA && lora_fold_tile(a.lora, b, a.T, a.Hq, hkv, Gq, col0, ncols, lane, a.status, qrow);
    for (int c = 0; c < ncols; ++c) {
        const int cg = col0 + c;
        const int64_t qrow_idx = (b * a.Hq + (int64_t)hkv * Gq + cg / a.T) * a.T + (cg % a.T);
        float qv[4];
        Elem<DT>::load4(a.q, qrow_idx * kHeadDim + 4 * lane, qv);
        if (LORA && updated) {
            const float4 up = *reinterpret_cast<const float4*>(qrow + c * 128 + 4 * lane);   // this lane's own store
            qv[0] = fmaf(up.x, a.lora.alpha, qv[0]); qv[1] = fmaf(up.y, a.lora.alpha, qv[1]);
            qv[2] = fmaf(up.z, a.lora.alpha, qv[2]); qv[3] = fmaf(up.w, a.lora.alpha, qv[3]);
        }
        if (a.rotate_q) wht128_warp(qv, lane);                  // the rotation folded into the query (fp32, not rounded)
        const float amax = warp_max(fmaxf(fmaxf(fabsf(qv[0]), fabsf(qv[1])), fmaxf(fabsf(qv[2]), fabsf(qv[3]))));
        // fp16 operands stay below 2^10 in magnitude; the power of two is re-applied to the scores
        const float mx = amax * fabsf(qs) * inv_lut;
        float post = 1.f;
        if (mx > 1024.f) post = exp2f(ceilf(log2f(mx * (1.f / 1024.f))));
        const float f = qs / post;
        // int16 fixed point for the q.g projections: amax * sq in [2^14 - 32, 2^15 - 64)
        const int E = (__float_as_uint(amax) >> 23) & 0xFF;
        const float sq = (E < 16 || E == 255) ? 0.f : __uint_as_float(((uint32_t)(267 - E) << 23) | 0x7F8000u);
        *reinterpret_cast<float4*>(qrow + c * 128 + 4 * lane) = make_float4(qv[0], qv[1], qv[2], qv[3]);
        if (lane == 0) colinfo[c] = make_float4(f * inv_lut, post, sq > 0.f ? kQjlCoef * f / sq : 0.f, sq);
    }
    __syncwarp();
    // 2. thread (g, t) owns column g: its 32 dims d = 32t .. 32t+31 as fp16 (scores) and as int8 limbs (q.g)
    uint32_t bh[4][2], bl[4][2];
    if (g < ncols) {
        const float4 ci = colinfo[g];
        float qd[32];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 v = *reinterpret_cast<const float4*>(qrow + g * 128 + 32 * t + 4 * k);
            qd[4 * k] = v.x; qd[4 * k + 1] = v.y; qd[4 * k + 2] = v.z; qd[4 * k + 3] = v.w;
            qB[k][0] = pack_half2(v.x * ci.x, v.y * ci.x);
            qB[k][1] = pack_half2(v.z * ci.x, v.w * ci.x);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __float_as_uint(fmaf(qd[8 * ks + k], ci.w, 12582912.f));   // low 16 bits = int16
            const uint32_t p01 = __byte_perm(v[0], v[1], 0x5140), p23 = __byte_perm(v[2], v[3], 0x5140);
            const uint32_t p45 = __byte_perm(v[4], v[5], 0x5140), p67 = __byte_perm(v[6], v[7], 0x5140);
            bl[ks][0] = __byte_perm(p01, p23, 0x5410); bh[ks][0] = __byte_perm(p01, p23, 0x7632);
            bl[ks][1] = __byte_perm(p45, p67, 0x5410); bh[ks][1] = __byte_perm(p45, p67, 0x7632);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) { qB[k][0] = 0u; qB[k][1] = 0u; }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) { bl[ks][0] = 0u; bl[ks][1] = 0u; bh[ks][0] = 0u; bh[ks][1] = 0u; }
    }
    float post0 = 1.f, post1 = 1.f;
    if (2 * t < ncols) post0 = colinfo[2 * t].y;
    if (2 * t + 1 < ncols) post1 = colinfo[2 * t + 1].y;
#pragma unroll
    for (int k = 0; k < 4; ++k) { sg.zh[k] = 0u; sg.zl[k] = 0u; sg.zq[k] = 0; }
    sg.cs0 = 0.f; sg.cs1 = 0.f;
    if (QJL) {
        // 3. q.g for all columns on the int8 tensor cores: A = G (+-1, built from the bit rows), B = the limbs;
        //    MMA k index 4t'+j / 16+4t'+j  <->  d = 32t' + 8ks + j / + 4 + j
        const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
        const uint32_t* grow = a.g_rows + (size_t)seed_of(uid, hkv) * kQjlDim * 4;
        const float inv0 = (2 * t < ncols) ? colinfo[2 * t].z : 0.f, inv1 = (2 * t + 1 < ncols) ? colinfo[2 * t + 1].z : 0.f;
        __syncwarp();                                            // all reads of the query rows are done
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            const uint32_t w0 = __ldg(grow + (16 * mt + g) * 4 + t), w1 = __ldg(grow + (16 * mt + g + 8) * 4 + t);
            int chi[4] = {0, 0, 0, 0}, clo[4] = {0, 0, 0, 0};
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t x0 = w0 >> (8 * ks), x1 = w1 >> (8 * ks);
                const uint32_t a0 = pm1_bytes<0>(x0), a1 = pm1_bytes<0>(x1), a2 = pm1_bytes<4>(x0), a3 = pm1_bytes<4>(x1);
                imma_acc_s8s8(chi, a0, a1, a2, a3, bh[ks][0], bh[ks][1]);
                imma_acc_s8u8(clo, a0, a1, a2, a3, bl[ks][0], bl[ks][1]);
            }
            // C element j: projection 16mt + g + 8(j>>1), column 2t + (j&1)
            if (2 * t < ncols) {
                qg_s[(2 * t) * 64 + 16 * mt + g] = (float)(chi[0] * 256 + clo[0]) * inv0;
                qg_s[(2 * t) * 64 + 16 * mt + g + 8] = (float)(chi[2] * 256 + clo[2]) * inv0;
            }
            if (2 * t + 1 < ncols) {
                qg_s[(2 * t + 1) * 64 + 16 * mt + g] = (float)(chi[1] * 256 + clo[1]) * inv1;
                qg_s[(2 * t + 1) * 64 + 16 * mt + g + 8] = (float)(chi[3] * 256 + clo[3]) * inv1;
            }
        }
        __syncwarp();
        // 4. quantise column g's 64 projections to 16-bit integers with one step; keep their sum even (it is halved)
        //    (every lane runs the shuffles; lanes of unused columns work on zeros)
        const bool mine = g < ncols;
        float v[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (mine) x = *reinterpret_cast<const float4*>(qg_s + g * 64 + 16 * t + 4 * k);
            v[4 * k] = x.x; v[4 * k + 1] = x.y; v[4 * k + 2] = x.z; v[4 * k + 3] = x.w;
        }
        float am = 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) am = fmaxf(am, fabsf(v[k]));
        am = fmaxf(am, __shfl_xor_sync(kFullMask, am, 1));
        am = fmaxf(am, __shfl_xor_sync(kFullMask, am, 2));
        const float step = am > 0.f ? am * (1.f / 32767.f) : 1.f, rstep = 1.f / step;
        int z[16], zsum = 0;
#pragma unroll
        for (int k = 0; k < 16; ++k) { z[k] = __float2int_rn(v[k] * rstep); zsum += z[k]; }
        zsum += __shfl_xor_sync(kFullMask, zsum, 1);
        zsum += __shfl_xor_sync(kFullMask, zsum, 2);
        const int z_first = __shfl_sync(kFullMask, z[0], lane & ~3);     // the column's first projection (lane t = 0)
        if (zsum & 1) {                                                  // uniform over the column's four lanes
            const int fix = z_first < 32767 ? 1 : -1;
            if (t == 0) z[0] += fix;
            zsum += fix;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // bytes 0 (low limb) and 1 (high limb, arithmetic: z = 256 * (z >> 8) + (z & 255)) of four integers
            const uint32_t p01 = __byte_perm(z[4 * k], z[4 * k + 1], 0x5140), p23 = __byte_perm(z[4 * k + 2], z[4 * k + 3], 0x5140);
            sg.zl[k] = __byte_perm(p01, p23, 0x5410);
            sg.zh[k] = __byte_perm(p01, p23, 0x7632);
        }
        const float mycs = mine ? -2.f * step : 0.f;
        const int myzh = zsum / 2;
        // the thread's score columns are 2t and 2t+1: fetch their seeds and steps from those columns' lanes
        sg.zq[0] = sg.zq[2] = __shfl_sync(kFullMask, myzh, 8 * t);
        sg.zq[1] = sg.zq[3] = __shfl_sync(kFullMask, myzh, 8 * t + 4);
        sg.cs0 = __shfl_sync(kFullMask, mycs, 8 * t);
        sg.cs1 = __shfl_sync(kFullMask, mycs, 8 * t + 4);
    }
    __syncwarp();

    qo.post0 = post0; qo.post1 = post1;
}

__device__ __forceinline__ void pack_query_operands(const QueryOperands& qo, uint4 (&v)[kPrepWords / 4]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = make_uint4(qo.qB[2 * k][0], qo.qB[2 * k][1], qo.qB[2 * k + 1][0], qo.qB[2 * k + 1][1]);
    v[4] = make_uint4(qo.sg.zh[0], qo.sg.zh[1], qo.sg.zh[2], qo.sg.zh[3]);
    v[5] = make_uint4(qo.sg.zl[0], qo.sg.zl[1], qo.sg.zl[2], qo.sg.zl[3]);
    v[6] = make_uint4((uint32_t)qo.sg.zq[0], (uint32_t)qo.sg.zq[1], __float_as_uint(qo.sg.cs0), __float_as_uint(qo.sg.cs1));
    v[7] = make_uint4(__float_as_uint(qo.post0), __float_as_uint(qo.post1), 0u, 0u);
}
__device__ __forceinline__ void unpack_query_operands(const uint4 (&v)[kPrepWords / 4], QueryOperands& qo) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        qo.qB[2 * k][0] = v[k].x; qo.qB[2 * k][1] = v[k].y; qo.qB[2 * k + 1][0] = v[k].z; qo.qB[2 * k + 1][1] = v[k].w;
    }
    qo.sg.zh[0] = v[4].x; qo.sg.zh[1] = v[4].y; qo.sg.zh[2] = v[4].z; qo.sg.zh[3] = v[4].w;
    qo.sg.zl[0] = v[5].x; qo.sg.zl[1] = v[5].y; qo.sg.zl[2] = v[5].z; qo.sg.zl[3] = v[5].w;
    qo.sg.zq[0] = qo.sg.zq[2] = (int)v[6].x; qo.sg.zq[1] = qo.sg.zq[3] = (int)v[6].y;
    qo.sg.cs0 = __uint_as_float(v[6].z); qo.sg.cs1 = __uint_as_float(v[6].w);
    qo.post0 = __uint_as_float(v[7].x); qo.post1 = __uint_as_float(v[7].y);
}

// Preparation launch of split-K calls: one warp per (user, kv head, tile of 8 query columns) builds the item's
// B operands once and stores them lane by lane; every split of the item then fetches seven 16-byte vectors per
// lane instead of repeating the projections.
// Users in order of decreasing cache length, as (user, clamped length) pairs: a counting sort over 1,024 length
// classes by one CTA of 128 threads (the order inside a class is whatever the atomics make it: it only decides
// which warp serves which work item, never a result).  The ticket scheduler hands items out in this order, so the
// long ones start first and the short ones even out the end of the launch.
static __device__ void sort_users_by_length(const AttnArgs& a) {
    __shared__ int hist[1024];
    __shared__ int warp_sum_s[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < 1024; i += 128) hist[i] = 0;
    __syncthreads();
    const int64_t S = a.S > 0 ? a.S : 1;
    for (int64_t b = tid; b < a.B; b += 128) {
        int64_t len = a.seq_lens[b];
        len = len < 0 ? 0 : (len > a.S ? a.S : len);
        atomicAdd(&hist[1023 - (int)(len * 1023 / S)], 1);
    }
    __syncthreads();
    int mine[8], sum = 0;                               // thread t owns classes 8t .. 8t+7
#pragma unroll
    for (int k = 0; k < 8; ++k) { mine[k] = hist[8 * tid + k]; sum += mine[k]; }
    int incl = sum;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const int o = __shfl_up_sync(kFullMask, incl, m);
        if (lane >= m) incl += o;
    }
    if (lane == 31) warp_sum_s[warp] = incl;
    __syncthreads();
    int start = incl - sum;
    for (int w = 0; w < warp; ++w) start += warp_sum_s[w];
#pragma unroll
    for (int k = 0; k < 8; ++k) { hist[8 * tid + k] = start; start += mine[k]; }
    __syncthreads();
    for (int64_t b = tid; b < a.B; b += 128) {
        int64_t len = a.seq_lens[b];
        len = len < 0 ? 0 : (len > a.S ? a.S : len);
        const int pos = atomicAdd(&hist[1023 - (int)(len * 1023 / S)], 1);
        a.user_order[pos] = make_int2((int)b, (int)len);
    }
}

template <int DT, bool QJL, bool LORA>
__global__ void __launch_bounds__(128) qattn_prep_kernel(AttnArgs a, int64_t n_units, unsigned n_unit_blocks) {
    __shared__ __align__(16) unsigned char scratch[4][kWarpScratchBytes];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x == n_unit_blocks) {                 // the extra CTA of a call with per-user lengths
        sort_users_by_length(a);
        return;
    }
    if (blockIdx.x == 0 && a.work_counter)             // the attention launch behind this one starts from zeroed tickets
        for (int i = threadIdx.x; i < (int)(kWorkCounterBytes / 4); i += blockDim.x) a.work_counter[i] = 0u;
    const int Gq = a.Hq / a.Hkv, ncols_all = Gq * a.T, n_ctiles = (ncols_all + 7) / 8;
    const float qs = a.scale * kLog2e;
    float* qrow = reinterpret_cast<float*>(scratch[warp]);
    float4* colinfo = reinterpret_cast<float4*>(qrow + 8 * 128);
    for (int64_t unit = (int64_t)blockIdx.x * 4 + warp; unit < n_units; unit += (int64_t)n_unit_blocks * 4) {
        const int col0 = 8 * (int)(unit % n_ctiles);
        const int hkv = (int)((unit / n_ctiles) % a.Hkv);
        const int64_t b = unit / n_ctiles / a.Hkv;
        const int ncols = ncols_all - col0 < 8 ? ncols_all - col0 : 8;
        QueryOperands qo;
        const float inv_lut = 1.f / lut_scale_of(a.codebooks + (a.cb_per_head ? hkv * 16 : 0));
        build_query_operands<DT, QJL, LORA>(a, b, hkv, col0, ncols, Gq, qs, inv_lut, qrow, colinfo, lane, qo);
        uint4 v[kPrepWords / 4];
        pack_query_operands(qo, v);
        uint4* dst = reinterpret_cast<uint4*>(a.qprep) + unit * (kPrepWords / 4) * 32 + lane;
#pragma unroll
        for (int k = 0; k < kPrepWords / 4; ++k) dst[32 * k] = v[k];
        __syncwarp();
    }
}

// Per-warp ring of TMA stages: each holds kStageKeys rows of K nibbles followed by as many of V.
// The stage filled next and the stage consumed next advance round-robin; `*_phase` is the parity of
// the mbarrier phase that the fill completes / the consumer waits for.
struct Ring {
    uint32_t stage0;        // shared address of stage 0 (stages are contiguous, kStageBytes apart)
    uint32_t bar0;          // shared address of mbarrier 0 (8 bytes apart)
    uint32_t fill, use;     // stage indices
    uint32_t use_phase;     // parity to wait for at `use`
    uint32_t in_flight;     // fills issued and not yet consumed
};

__device__ __forceinline__ void ring_issue(Ring& r, const CUtensorMap* mk, const CUtensorMap* mv, int32_t row, int lane) {
    if (lane == 0) {
        const uint32_t bar = r.bar0 + 8 * r.fill, dst = r.stage0 + r.fill * kStageBytes;
        // no proxy fence is needed before the refill: every lane has already consumed (not merely issued)
        // its reads of this stage, and the caller's __syncwarp() ordered that before this point
        mbar_expect_tx(bar, kStageBytes);
        tma_load_rows(dst, mk, row, bar);
        tma_load_rows(dst + kStageKeys * kNibBytes, mv, row, bar);
    }
    r.fill = (r.fill + 1 == kStages) ? 0u : r.fill + 1;
    ++r.in_flight;
}
__device__ __forceinline__ void ring_consumed(Ring& r) {
    if (r.use + 1 == kStages) { r.use = 0; r.use_phase ^= 1u; } else { ++r.use; }
    --r.in_flight;
}

template <int DT, bool QJL, bool ONECOL, bool VPAIR, bool LORA>
__global__ void __launch_bounds__(kMmaWarps * 32, 1)
qattn_mma_kernel(AttnArgs a, int64_t n_items, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kr = rho8(g);                                   // K / score row of this thread (and kr + 8)
    const int va = rho8(2 * t), vb = rho8(2 * t + 1);         // V rows of this thread (and those + 8)
    const bool head_in_item = (gridDim.y == 1 && a.Hkv > 1);  // shared codebook: a CTA serves all kv heads
    const int cb_head = blockIdx.y;

    // ---- shared memory carve-up -------------------------------------------------------------
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t lut_off = (kLutSpan - (smem_base & (kLutSpan - 1))) & (kLutSpan - 1);
    // warps [0, n_front) live in front of the tables, the others behind them
    const uint32_t n_front = lut_off / kWarpBlockBytes;
    const uint32_t my_off = (uint32_t)warp < n_front ? (uint32_t)warp * kWarpBlockBytes
                                                     : lut_off + kLutSpan + ((uint32_t)warp - n_front) * kWarpBlockBytes;
    {
        // a codebook the fp16 table cannot hold to the error budget: the whole grid stands down (the same test in
        // the lane-per-key kernel, launched behind this one, makes that kernel serve the call)
        const int n_cb = a.cb_per_head ? a.Hkv * 16 : 16;
        bool wide = false;
        for (int i = threadIdx.x; i < n_cb; i += blockDim.x) wide = wide || centroid_is_wide(__ldg(a.codebooks + i));
        if (__syncthreads_or(wide)) return;
    }
    const float lut_scale = lut_scale_of(a.codebooks + (a.cb_per_head ? cb_head * 16 : 0));
    const float inv_lut = 1.f / lut_scale;
    {
        const float* cb = a.codebooks + (a.cb_per_head ? cb_head * 16 : 0);
        uint32_t* lut = reinterpret_cast<uint32_t*>(smem + lut_off);
        for (int i = threadIdx.x; i < 256 * 8; i += blockDim.x) {       // four lanes' copies of an entry per store
            const int byte = i >> 3, quad = i & 7;
            const uint32_t v = pack_half2(__ldg(cb + (byte & 15)) * lut_scale, __ldg(cb + (byte >> 4)) * lut_scale);
            *reinterpret_cast<uint4*>(lut + byte * 64 + 4 * quad) = make_uint4(v, v, v, v);
        }
    }
    const uint32_t lut_lane = smem_base + lut_off + 4 * lane;                  // bits 8..15 are zero
    float* qrow = reinterpret_cast<float*>(smem + my_off + kStages * kStageBytes);   // [8][128] fp32 query rows, later [8][64] q.g projections
    float4* colinfo = reinterpret_cast<float4*>(qrow + 8 * 128);                      // per column: f, post, q.g scale, -
    Ring ring;
    ring.stage0 = smem_base + my_off;
    ring.bar0 = smem_base + my_off + kStages * kStageBytes + kWarpScratchBytes;
    ring.fill = 0; ring.use = 0; ring.use_phase = 0; ring.in_flight = 0;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(ring.bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        fence_proxy_async();
    }
    __syncthreads();

    // swizzled offsets inside a stage (64-byte swizzle: 16-byte chunk index ^= (row >> 1) & 3)
    const uint32_t off_k = kr * kNibBytes + ((t ^ ((kr >> 1) & 3)) << 4);               // row kr + 8: + 512
    const uint32_t off_va = kStageKeys * kNibBytes + va * kNibBytes + (((g >> 1) ^ ((va >> 1) & 3)) << 4) + 8 * (g & 1);
    const uint32_t off_vb = kStageKeys * kNibBytes + vb * kNibBytes + (((g >> 1) ^ ((vb >> 1) & 3)) << 4) + 8 * (g & 1);

    const int Gq = a.Hq / a.Hkv;
    const int ncols_all = Gq * a.T;                 // query columns of a kv head: (q head in group, token)
    const int n_ctiles = (ncols_all + 7) / 8;       // handled 8 at a time; each tile is a work item of its own
    const float qs = a.scale * kLog2e;
    bool alive = true;

    // Work distribution.  Every warp starts on item warp * gridDim.x + blockIdx.x (items go round the CTAs first, so
    // a call with few items uses one warp on each of many SMs rather than twelve warps on a few).  Without a counter the next
    // item lies one grid of warps further on (equal-sized items: nothing to balance).  With one (split-K calls,
    // whose items differ in length when the users' caches do) a warp takes a ticket for its next item when it
    // starts the current one, so the atomic's latency is covered by the item's own work.
    const int64_t item_stride = (int64_t)gridDim.x * kMmaWarps;
    uint32_t* const counter = a.work_counter ? a.work_counter + blockIdx.y : nullptr;
    for (int64_t item = (int64_t)warp * gridDim.x + blockIdx.x; item < n_items;) {
        uint32_t ticket = 0u;
        if (counter && lane == 0) ticket = atomicAdd(counter, 1u);
        int64_t rest = item;
        // the column tile varies fastest, so the tiles of one (user, kv head, split) run on neighbouring warps at
        // about the same time and all but the first find the keys in L2
        const int col0 = 8 * (int)(rest % n_ctiles);
        rest /= n_ctiles;
        const int ncols = ncols_all - col0 < 8 ? ncols_all - col0 : 8;
        int hkv = cb_head;
        if (head_in_item) { hkv = (int)(rest % a.Hkv); rest /= a.Hkv; }
        const int split = (int)(rest % a.n_splits);
        int64_t b = rest / a.n_splits;

        // ---- key range of this split; start the first copies before the prologue ------------------
        int64_t len;
        if (!ONECOL && a.user_order) {                  // items are numbered by decreasing cache length (not in the
                                                        // one-column variants, which have no register to spare)
            const int2 e = __ldg(a.user_order + b);
            b = e.x;
            len = e.y;
        } else {
            len = a.seq_lens ? (int64_t)a.seq_lens[b] : a.S;
            len = len < 0 ? 0 : (len > a.S ? a.S : len);
        }
        int64_t per = (len + a.n_splits - 1) / a.n_splits;
        per = (per + 31) / 32 * 32;
        const int64_t s0 = (int64_t)split * per;
        const int64_t s1 = (s0 + per < len) ? s0 + per : len;
        const int64_t slot = a.cache_slots ? (int64_t)a.cache_slots[b] : b;
        const int64_t row0 = slot * a.ks_b + (int64_t)hkv * a.ks_h + s0;
        // a warp whose wait expired earlier reads nothing more: its remaining items get neutral results below
        const int nkeys = (alive && s1 > s0) ? (int)(s1 - s0) : 0;
        // full stages come in by TMA, whose row coordinate is a signed 32-bit number; the rest (fewer than 32 keys,
        // or every key of a range that lies beyond that coordinate space) is read with plain loads
        const int nstage = (row0 + nkeys <= 0x7fffffffLL) ? nkeys / kStageKeys : 0;
        {
            const int prime = nstage < kStages ? nstage : kStages;
            for (int j = 0; j < prime; ++j) ring_issue(ring, &map_k, &map_v, (int32_t)(row0 + kStageKeys * j), lane);
        }
        const uint8_t* ps = a.k_qjl + (row0 + kr) * kQjlBytes + 2 * t;      // sign bytes / norm of row kr, block 0
        const float* pn = a.k_norms + row0 + kr;
        AuxRegs aux_a, aux_b;                                   // sign bytes / norms of the two blocks of the next stage
        if (QJL && nstage > 0) {
            if (lane == 2) prefetch_l2_bulk(reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(a.k_qjl + row0 * kQjlBytes) & ~(uintptr_t)15),
                                            (uint32_t)(nstage * kStageKeys * kQjlBytes) & ~15u);
            if (lane == 3) prefetch_l2_bulk(reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(a.k_norms + row0) & ~(uintptr_t)15),
                                            (uint32_t)(nstage * kStageKeys * 4) & ~15u);
            load_aux(aux_a, ps, pn);
            load_aux(aux_b, ps + 16 * kQjlBytes, pn + 16);
        }

        // ---- prologue: B operands (scaled queries, q.g projections) --------------------------------
        // computed here, or fetched when a preparation launch has stored them (split-K calls, whose items would
        // otherwise repeat this work once per split)
        QueryOperands qo;
        if (a.qprep) {
            const int64_t unit = (b * a.Hkv + hkv) * n_ctiles + col0 / 8;
            const uint4* src = reinterpret_cast<const uint4*>(a.qprep) + unit * (kPrepWords / 4) * 32 + lane;
            uint4 v[kPrepWords / 4];
#pragma unroll
            for (int k = 0; k < kPrepWords / 4; ++k) v[k] = __ldg(src + 32 * k);
            unpack_query_operands(v, qo);
        } else {
            build_query_operands<DT, QJL, LORA>(a, b, hkv, col0, ncols, Gq, qs, inv_lut, qrow, colinfo, lane, qo);
        }
        const uint32_t (&qB)[8][2] = qo.qB;
        const SignB& sg = qo.sg;
        const float post0 = qo.post0, post1 = qo.post1;

        WarpState st;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) { st.O[mt][0] = 0.f; st.O[mt][1] = 0.f; st.O[mt][2] = 0.f; st.O[mt][3] = 0.f; }
        st.m0 = -INFINITY; st.m1 = -INFINITY; st.l0 = 0.f; st.l1 = 0.f;

        // ---- full stages: wait, pull the bytes of a 16-key block into registers, process; refill -----
        KeyBlock kb;
        for (int j = 0; j < nstage; ++j) {
            // the outcome is made warp-uniform: the lanes poll on their own and could disagree at the limit
            if (!__all_sync(kFullMask, mbar_wait_bounded(ring.bar0 + 8 * ring.use, ring.use_phase))) { alive = false; break; }
            const uint32_t base = ring.stage0 + ring.use * kStageBytes;
            // both 16-key blocks of the stage are pulled into registers up front, so that the table lookups of the
            // second block can overlap the softmax of the first
            KeyBlock kc;
            kb.ka = lds16(base + off_k);
            kb.kb = lds16(base + off_k + 8 * kNibBytes);
            kb.v0 = lds8(base + off_va);
            kb.v1 = lds8(base + off_vb);
            kb.v2 = lds8(base + off_va + 8 * kNibBytes);
            kb.v3 = lds8(base + off_vb + 8 * kNibBytes);
            kc.ka = lds16(base + 16 * kNibBytes + off_k);
            kc.kb = lds16(base + 16 * kNibBytes + off_k + 8 * kNibBytes);
            kc.v0 = lds8(base + 16 * kNibBytes + off_va);
            kc.v1 = lds8(base + 16 * kNibBytes + off_vb);
            kc.v2 = lds8(base + 16 * kNibBytes + off_va + 8 * kNibBytes);
            kc.v3 = lds8(base + 16 * kNibBytes + off_vb + 8 * kNibBytes);
            if (QJL) {
                kb.sa = aux_a.sa; kb.sb = aux_a.sb; kb.na = aux_a.na; kb.nb = aux_a.nb;
                kc.sa = aux_b.sa; kc.sb = aux_b.sb; kc.na = aux_b.na; kc.nb = aux_b.nb;
                if (j + 1 < nstage) {                          // the next stage's sign bytes and norms
                    ps += kStageKeys * kQjlBytes; pn += kStageKeys;
                    load_aux(aux_a, ps, pn);
                    load_aux(aux_b, ps + 16 * kQjlBytes, pn + 16);
                }
            }
            process_key_block<QJL, false, ONECOL, VPAIR>(kb, st, qB, sg, post0, post1, lut_lane, 16, kr);
            process_key_block<QJL, false, ONECOL, VPAIR>(kc, st, qB, sg, post0, post1, lut_lane, 16, kr);
            // every lane has consumed its bytes of the stage: it can be refilled
            ring_consumed(ring);
            __syncwarp();
            if (j + kStages < nstage) ring_issue(ring, &map_k, &map_v, (int32_t)(row0 + kStageKeys * (j + kStages)), lane);
        }
        if (!alive && ring.in_flight) {
            // A wait expired.  Report it, give the copies still in flight a bounded chance to land before this
            // warp's shared memory is handed back, and turn the item's state into the neutral partial result
            // (maximum -inf, sum 0, zero accumulators) so that a merge never reads memory this launch left unwritten.
            if (lane == 0 && a.status) atomicExch(a.status, OMNI_ERR_DEVICE_WAIT);
            while (ring.in_flight) {
                mbar_wait_bounded(ring.bar0 + 8 * ring.use, ring.use_phase);
                ring_consumed(ring);
            }
            __syncwarp();
        }
        if (!alive) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) { st.O[mt][0] = 0.f; st.O[mt][1] = 0.f; st.O[mt][2] = 0.f; st.O[mt][3] = 0.f; }
            st.m0 = -INFINITY; st.m1 = -INFINITY; st.l0 = 0.f; st.l1 = 0.f;
        }
        for (int k0 = nstage * kStageKeys; alive && k0 < nkeys; k0 += 16) {     // blocks with plain clamped loads
            const int nvalid = nkeys - k0 < 16 ? nkeys - k0 : 16;
            // groups of eight keys that lie completely below the user's length are stored pair-wise
            const int64_t paired_left = (len & ~(int64_t)7) - (s0 + k0);
            load_tail_block<QJL, VPAIR>(kb, a, row0 + k0, nvalid, paired_left >= 16 ? 16 : (paired_left >= 8 ? 8 : 0), kr, va, vb, g, t);
            process_key_block<QJL, true, ONECOL, VPAIR>(kb, st, qB, sg, post0, post1, lut_lane, nvalid, kr);
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
            const bool real = c < ncols;                       // every lane runs the shuffles below; only real columns store
            const int cg = col0 + (real ? c : 0);
            const int64_t qrow = (b * a.Hq + (int64_t)hkv * Gq + cg / a.T) * a.T + (cg % a.T);
            const float l = j ? st.l1 : st.l0;
            const float m = j ? st.m1 : st.m0;
            float* dst;
            float mul;
            if (a.n_splits == 1) {
                dst = a.out + qrow * kHeadDim + 16 * g;
                mul = l > 0.f ? inv_lut / l : 0.f;
            } else {
                float* w = a.ws + (qrow * a.n_splits + split) * kWsStride;
                dst = w + 16 * g;
                mul = inv_lut;
                if (real && g == 0) { w[128] = m * 0.6931471805599453f; w[129] = l; }   // max back in natural-log units
            }
            float v[16];                          // d = 16g + i, i = 4mp + e  (m-tiles 2mp, 2mp+1)
#pragma unroll
            for (int mp = 0; mp < 4; ++mp) {
                v[4 * mp] = st.O[2 * mp][j] * mul;         v[4 * mp + 1] = st.O[2 * mp][2 + j] * mul;
                v[4 * mp + 2] = st.O[2 * mp + 1][j] * mul; v[4 * mp + 3] = st.O[2 * mp + 1][2 + j] * mul;
            }
            if (a.unrotate_out && a.n_splits == 1) {
                // inverse rotation of the finished row (the transform is its own inverse): four stages inside the
                // thread's 16 dims, three across the eight lanes that share this column (lane bits 2..4 = g)
#pragma unroll
                for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if ((i & h) == 0) {
                            const float u = v[i], w2 = v[i | h];
                            v[i] = u + w2; v[i | h] = u - w2;
                        }
                    }
                }
#pragma unroll
                for (int mk = 4; mk <= 16; mk <<= 1) {
                    const bool lower = (lane & mk) != 0;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float o = __shfl_xor_sync(kFullMask, v[i], mk);
                        v[i] = lower ? o - v[i] : v[i] + o;
                    }
                }
                const float sc = __uint_as_float(OMNI_WHT_SCALE_BITS);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] *= sc;
            }
            if (real) {
#pragma unroll
                for (int mp = 0; mp < 4; ++mp)
                    *reinterpret_cast<float4*>(dst + 4 * mp) = make_float4(v[4 * mp], v[4 * mp + 1], v[4 * mp + 2], v[4 * mp + 3]);
            }
        }
        item = counter ? item_stride + (int64_t)__shfl_sync(kFullMask, ticket, 0) : item + item_stride;
    }
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static std::mutex mu;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D view [rows][64 bytes] of a nibble array with a kStageKeys-row box and the 64-byte swizzle.  The row
// extent is the largest a 32-bit row coordinate can address: only full kStageKeys-row boxes that lie inside
// the caller's arrays are ever requested, so nothing depends on out-of-bounds clipping.
// The descriptor depends on the base address alone, so the last few are kept: a serving loop calls with the same
// cache arrays every step and skips the driver call.
struct MapCacheEntry { const uint8_t* base; CUtensorMap map; };
constexpr int kMapCacheSize = 8;
static MapCacheEntry g_map_cache[kMapCacheSize];
static int g_map_cache_next = 0;
static std::mutex g_map_cache_mutex;

static int32_t encode_nibble_map(CUtensorMap* map, const uint8_t* base);

static int32_t make_nibble_map(CUtensorMap* map, const uint8_t* base) {
    {
        std::lock_guard<std::mutex> lk(g_map_cache_mutex);
        for (int i = 0; i < kMapCacheSize; ++i)
            if (g_map_cache[i].base == base && base != nullptr) { *map = g_map_cache[i].map; return OMNI_OK; }
    }
    const int32_t rc = encode_nibble_map(map, base);
    if (rc != OMNI_OK) return rc;
    std::lock_guard<std::mutex> lk(g_map_cache_mutex);
    g_map_cache[g_map_cache_next] = MapCacheEntry{base, *map};
    g_map_cache_next = (g_map_cache_next + 1) % kMapCacheSize;
    return OMNI_OK;
}

static int32_t encode_nibble_map(CUtensorMap* map, const uint8_t* base) {
    EncodeTiledFn fn = encode_tiled_fn();
    OMNI_REQUIRE(fn != nullptr, OMNI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)kNibBytes, (cuuint64_t)0x7fffffffull};
    const cuuint64_t strides[1] = {(cuuint64_t)kNibBytes};
    const cuuint32_t box[2] = {(cuuint32_t)kNibBytes, (cuuint32_t)kStageKeys};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    OMNI_REQUIRE(r == CUDA_SUCCESS, OMNI_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return OMNI_OK;
}

#if !OMNI_MMA_LORA
// Self-test of the bounded wait: one warp waits, with the caller's poll limit, on an mbarrier that nothing ever
// arrives on.  The wait must run out, the warp must report OMNI_ERR_DEVICE_WAIT through the status word exactly
// like the decode kernel does, and the kernel must return normally (nothing spins unbounded, nothing traps).
__global__ void bounded_wait_probe_kernel(uint32_t limit, int32_t* status) {
    __shared__ __align__(8) unsigned long long bar_storage;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bar_storage);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    const bool ok = __all_sync(kFullMask, mbar_wait_bounded(bar, 0u, limit));
    if (!ok && threadIdx.x == 0 && status) atomicExch(status, OMNI_ERR_DEVICE_WAIT);
}

int32_t launch_wait_probe(uint32_t limit, int32_t* status, cudaStream_t st) {
    bounded_wait_probe_kernel<<<1, 32, 0, st>>>(limit, status);
    return check_cuda(cudaGetLastError(), "bounded_wait_probe_kernel launch");
}

bool mma_eligible(const AttnArgs& a) {
    // any number of query columns per kv head: they are processed in tiles of 8 (one MMA N extent)
    const int64_t cols = (int64_t)(a.Hq / a.Hkv) * a.T;
    return cols <= 4096 && a.Hkv <= 65535;
}

#endif  // !OMNI_MMA_LORA

// Per-device facts that never change while the process lives: looked up once, then read without a driver call.
static int g_sm_count[kMaxDevices];          // 0 = not yet queried
static std::mutex g_once_mutex;

static int32_t sm_count_of(int dev, int* sms) {
    if (dev < 0 || dev >= kMaxDevices) {
        OMNI_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
        return OMNI_OK;
    }
    std::lock_guard<std::mutex> lk(g_once_mutex);
    if (g_sm_count[dev] == 0) OMNI_CUDA(cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
    *sms = g_sm_count[dev];
    return OMNI_OK;
}

// The opt-in to the full shared-memory carve-out is per kernel and per device; it is made once for each pair.
// (All instantiations of the kernel share one function-pointer type, so the record is keyed by address.)
static int32_t allow_full_smem(const void* kern, int dev) {
    static std::vector<std::pair<const void*, int>> done;
    std::lock_guard<std::mutex> lk(g_once_mutex);
    for (const auto& p : done)
        if (p.first == kern && p.second == dev) return OMNI_OK;
    OMNI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmemBytes));
    done.emplace_back(kern, dev);
    return OMNI_OK;
}

template <int DT>
static int32_t launch_mma_t(const AttnArgs& a, cudaStream_t st) {
    int dev = 0, sms = 148;
    OMNI_CUDA(cudaGetDevice(&dev));
    int32_t rc = sm_count_of(dev, &sms);
    if (rc != OMNI_OK) return rc;
    // Persistent CTAs, one per SM.  With one shared codebook a CTA serves every kv head
    // (grid.y == 1, the head is part of the item index); with per-head codebooks a CTA is
    // bound to one head because its lookup table is built from that head's centroids.
    int64_t items, ctas;
    unsigned gy;
    const int64_t n_ctiles = ((int64_t)(a.Hq / a.Hkv) * a.T + 7) / 8;
    // ticket counters: cleared by the preparation launch when there is one, by a memset node otherwise
    if (a.work_counter && !a.qprep) OMNI_CUDA(cudaMemsetAsync(a.work_counter, 0, kWorkCounterBytes, st));
    if (a.cb_per_head) {
        items = a.B * a.n_splits * n_ctiles;
        ctas = sms / a.Hkv > 0 ? sms / a.Hkv : 1;
        gy = (unsigned)a.Hkv;
    } else {
        items = a.B * a.n_splits * a.Hkv * n_ctiles;
        ctas = sms;
        gy = 1;
    }
    if (ctas > items) ctas = items;                 // few items: one per CTA, spread over the SMs
    dim3 grid((unsigned)ctas, gy);
    CUtensorMap map_k, map_v;
    rc = make_nibble_map(&map_k, a.k_nib);
    if (rc != OMNI_OK) return rc;
    if (a.v_nib == a.k_nib) {
        map_v = map_k;
    } else {
        rc = make_nibble_map(&map_v, a.v_nib);
        if (rc != OMNI_OK) return rc;
    }
    if (a.qprep) {
        const int64_t units = a.B * a.Hkv * n_ctiles;
        int64_t blocks = (units + 3) / 4;
        if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
        const unsigned grid_prep = (unsigned)blocks + (a.user_order ? 1u : 0u);     // one more CTA sorts the users by length
        if (a.with_qjl) qattn_prep_kernel<DT, true, kLoraBuild><<<grid_prep, 128, 0, st>>>(a, units, (unsigned)blocks);
        else            qattn_prep_kernel<DT, false, kLoraBuild><<<grid_prep, 128, 0, st>>>(a, units, (unsigned)blocks);
        rc = check_cuda(cudaGetLastError(), "qattn_prep_kernel launch");
        if (rc != OMNI_OK) return rc;
    }
    const bool one_col = (a.Hq / a.Hkv) * a.T == 1;
    if (one_col && a.user_order) return set_error(OMNI_ERR_ARG, "qattn: the one-column kernels take the users in index order");
    auto kern = a.v_paired
        ? (a.with_qjl ? (one_col ? qattn_mma_kernel<DT, true, true, true, kLoraBuild> : qattn_mma_kernel<DT, true, false, true, kLoraBuild>)
                      : (one_col ? qattn_mma_kernel<DT, false, true, true, kLoraBuild> : qattn_mma_kernel<DT, false, false, true, kLoraBuild>))
        : (a.with_qjl ? (one_col ? qattn_mma_kernel<DT, true, true, false, kLoraBuild> : qattn_mma_kernel<DT, true, false, false, kLoraBuild>)
                      : (one_col ? qattn_mma_kernel<DT, false, true, false, kLoraBuild> : qattn_mma_kernel<DT, false, false, false, kLoraBuild>));
    rc = allow_full_smem(reinterpret_cast<const void*>(kern), dev);
    if (rc != OMNI_OK) return rc;
    kern<<<grid, kMmaWarps * 32, kMmaSmemBytes, st>>>(a, items, map_k, map_v);
    return check_cuda(cudaGetLastError(), "qattn_mma_kernel launch");
}

#if OMNI_MMA_LORA
int32_t launch_mma_lora(const AttnArgs& a, cudaStream_t st) {
#else
int32_t launch_mma(const AttnArgs& a, cudaStream_t st) {
    if (a.lora.x) return launch_mma_lora(a, st);
#endif
    switch (a.q_dtype) {
        case OMNI_F32:  return launch_mma_t<OMNI_F32>(a, st);
        case OMNI_BF16: return launch_mma_t<OMNI_BF16>(a, st);
        case OMNI_F16:  return launch_mma_t<OMNI_F16>(a, st);
    }
    return set_error(OMNI_ERR_ARG, "qattn: unknown q dtype code %d", a.q_dtype);
}

}  // namespace omni
