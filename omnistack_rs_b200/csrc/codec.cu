// KV-cache codec: rotation, INT4 Lloyd-Max codes, residual norm, QJL sign bits, and
// the inverse.  One warp owns one 128-element row; lane l holds elements 4l..4l+3.
//
// Bit-exactness notes (they mirror what the reference computes on the CPU):
//   * rotation: fp32 butterflies in stage order, separate roundings (no FMA), one
//     multiply by float32(1/sqrt(128)); 16-bit inputs are rounded back to their type;
//   * code = first index minimising |y - c| in fp32 (strict "<" scan from c = 0);
//   * the sign of each of the 64 projections is taken from an fp64 accumulation of the
//     fp32 residuals, i.e. the mathematically exact sign up to 2^-53 relative error --
//     the reference's sgemm agrees whenever its own fp32 rounding does not decide the bit.
#include "common.cuh"
#include "codec_fast.cuh"
#include <cstdlib>
#include <algorithm>
#include <vector>

namespace omni {

struct CodecArgs {
    const void* x;            // input rows (quantize) / unused (dequantize)
    int64_t xs_b, xs_h, xs_t; // element strides of x
    const float* codebooks;
    int cb_per_head;
    const int32_t* user_ids;
    int32_t user_id;
    int64_t B; int H; int64_t T;
    uint8_t* nib; uint8_t* qjl; float* norms;   // packed arrays (outputs of quantize, inputs of dequantize)
    int64_t os_b, os_h;       // row strides of the packed arrays
    const int64_t* out_offsets;
    int64_t out_offset;
    const uint32_t* g_rows;   // [1024][64][4]
    const uint64_t* g_cols;   // [1024][128]
    int row_seeded;           // 1: seed = (user_id & 1023) ^ (base + flat row index)
    int base_head_idx;
    int with_qjl;
    float* out;               // dequantize output, contiguous [rows][128]
};

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ void decode_row(const CodecArgs& a, int64_t r, int64_t& b, int& h, int64_t& t) {
    t = r % a.T;
    int64_t bh = r / a.T;
    h = (int)(bh % a.H);
    b = bh / a.H;
}

template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) rotate_kernel(const void* x, void* y, int64_t n_rows) {
    const int lane = threadIdx.x & 31;
    int64_t w = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nw = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t r = w; r < n_rows; r += nw) {
        float v[4];
        Elem<DT>::load4(x, r * kHeadDim + 4 * lane, v);
        wht128_warp(v, lane);
        Elem<DT>::store4(y, r * kHeadDim + 4 * lane, v);
    }
}

template <int DT, bool ROTATE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) quantize_kernel(CodecArgs a) {
    __shared__ double e_s[kWarpsPerBlock][kHeadDim];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int64_t n_rows = a.B * a.H * a.T;
    const int64_t nw = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t r = (int64_t)blockIdx.x * kWarpsPerBlock + wib; r < n_rows; r += nw) {
        int64_t b, t; int h;
        decode_row(a, r, b, h, t);
        float y[4];
        Elem<DT>::load4(a.x, b * a.xs_b + h * a.xs_h + t * a.xs_t + 4 * lane, y);
        if (ROTATE) {
            wht128_warp(y, lane);
#pragma unroll
            for (int k = 0; k < 4; ++k) y[k] = Elem<DT>::round(y[k]);
        }
        const float* cb = a.codebooks + (a.cb_per_head ? h * 16 : 0);
        float cbr[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) cbr[c] = __ldg(cb + c);

        uint32_t packed = 0;
        float e[4];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float best = fabsf(__fsub_rn(y[k], cbr[0]));
            float deq = cbr[0];
            uint32_t code = 0;
#pragma unroll
            for (int c = 1; c < 16; ++c) {
                float d = fabsf(__fsub_rn(y[k], cbr[c]));
                if (d < best) { best = d; deq = cbr[c]; code = c; }
            }
            packed |= code << (4 * k);
            e[k] = __fsub_rn(y[k], deq);
            ss = fmaf(e[k], e[k], ss);
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(kFullMask, ss, m);

        // residual to shared memory as fp64 for the projections
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 4; ++k) e_s[wib][4 * lane + k] = (double)e[k];
        __syncwarp();

        const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
        const int seed = a.row_seeded ? (((uid & 1023) ^ (a.base_head_idx + (int)r)) & 1023) : seed_of(uid, h);
        const uint4* grow = reinterpret_cast<const uint4*>(a.g_rows) + (size_t)seed * kQjlDim;
        const uint4 g0 = __ldg(grow + lane), g1 = __ldg(grow + lane + 32);
        const uint32_t w0[4] = {g0.x, g0.y, g0.z, g0.w};
        const uint32_t w1[4] = {g1.x, g1.y, g1.z, g1.w};
        double acc0 = 0.0, acc1 = 0.0;
        const double2* es2 = reinterpret_cast<const double2*>(e_s[wib]);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll 8
            for (int j = 0; j < 32; j += 2) {
                double2 ev = es2[(w * 32 + j) >> 1];
                acc0 += ((w0[w] >> j) & 1u) ? ev.x : -ev.x;
                acc0 += ((w0[w] >> (j + 1)) & 1u) ? ev.y : -ev.y;
                acc1 += ((w1[w] >> j) & 1u) ? ev.x : -ev.x;
                acc1 += ((w1[w] >> (j + 1)) & 1u) ? ev.y : -ev.y;
            }
        }
        const uint32_t lo = __ballot_sync(kFullMask, acc0 >= 0.0);
        const uint32_t hi = __ballot_sync(kFullMask, acc1 >= 0.0);

        const int64_t ro = b * a.os_b + h * a.os_h + t + (a.out_offsets ? a.out_offsets[b] : a.out_offset);
        reinterpret_cast<uint16_t*>(a.nib + ro * kNibBytes)[lane] = (uint16_t)packed;
        if (lane == 0 && a.qjl) {
            *reinterpret_cast<uint2*>(a.qjl + ro * kQjlBytes) = make_uint2(lo, hi);
            a.norms[ro] = sqrtf(ss);
        }
    }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) dequantize_kernel(CodecArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t n_rows = a.B * a.H * a.T;
    const int64_t nw = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t r = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < n_rows; r += nw) {
        int64_t b, t; int h;
        decode_row(a, r, b, h, t);
        const int64_t ri = b * a.os_b + h * a.os_h + t;
        const float* cb = a.codebooks + (a.cb_per_head ? h * 16 : 0);
        const uint32_t packed = reinterpret_cast<const uint16_t*>(a.nib + ri * kNibBytes)[lane];
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __ldg(cb + ((packed >> (4 * k)) & 0xF));
        if (a.with_qjl) {
            const uint2 sb = *reinterpret_cast<const uint2*>(a.qjl + ri * kQjlBytes);
            const uint64_t sig = ((uint64_t)sb.y << 32) | sb.x;
            const float coef = __fmul_rn(a.norms[ri], kQjlCoef);
            const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
            const int seed = a.row_seeded ? (((uid & 1023) ^ (a.base_head_idx + (int)r)) & 1023) : seed_of(uid, h);
            const uint64_t* gc = a.g_cols + (size_t)seed * kHeadDim + 4 * lane;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                // sum_i s_i * g_id with s, g in {-1,+1}: matches minus mismatches
                const int sum = kQjlDim - 2 * __popcll(sig ^ __ldg(gc + k));
                v[k] = __fadd_rn(v[k], __fmul_rn((float)sum, coef));
            }
        }
        *reinterpret_cast<float4*>(a.out + r * kHeadDim + 4 * lane) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// Head-seeded dequantisation, the streaming form: a warp takes a run of consecutive tokens of one (user, head), so
// the head's 16 centroids (one per lane, fetched by shuffle) and this lane's four columns of G stay in registers
// for the whole run; per token it reads 2 bytes of codes per lane plus the broadcast sign word and norm, and
// writes 16 bytes per lane.  kDeqFlight tokens are in flight per iteration.
constexpr int kDeqRun = 64;     // tokens per work unit
constexpr int kDeqFlight = 4;   // tokens whose loads are issued together

__global__ void __launch_bounds__(kWarpsPerBlock * 32) dequantize_heads_kernel(CodecArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t runs_per_head = (a.T + kDeqRun - 1) / kDeqRun;
    const int64_t n_units = a.B * a.H * runs_per_head;
    const int64_t nw = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t u = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); u < n_units; u += nw) {
        const int64_t run = u % runs_per_head, bh = u / runs_per_head;
        const int h = (int)(bh % a.H);
        const int64_t b = bh / a.H;
        const float cb_lane = __ldg(a.codebooks + (a.cb_per_head ? h * 16 : 0) + (lane & 15));
        uint64_t gc[4] = {0ull, 0ull, 0ull, 0ull};
        if (a.with_qjl) {
            const int32_t uid = a.user_ids ? a.user_ids[b] : a.user_id;
            const uint64_t* gp = a.g_cols + (size_t)seed_of(uid, h) * kHeadDim + 4 * lane;
#pragma unroll
            for (int k = 0; k < 4; ++k) gc[k] = __ldg(gp + k);
        }
        const int64_t t_begin = run * kDeqRun, t_end = (t_begin + kDeqRun < a.T) ? t_begin + kDeqRun : a.T;
        const int64_t in0 = b * a.os_b + h * a.os_h, out0 = (b * a.H + h) * a.T;
        for (int64_t t = t_begin; t < t_end; t += kDeqFlight) {
            uint32_t p[kDeqFlight];
            uint2 sg[kDeqFlight];
            float cf[kDeqFlight];
#pragma unroll
            for (int u = 0; u < kDeqFlight; ++u) {             // all loads of the batch first
                const int64_t r = in0 + (t + u < t_end ? t + u : t_end - 1);
                p[u] = reinterpret_cast<const uint16_t*>(a.nib + r * kNibBytes)[lane];
                sg[u] = make_uint2(0u, 0u);
                cf[u] = 0.f;
                if (a.with_qjl) {
                    sg[u] = *reinterpret_cast<const uint2*>(a.qjl + r * kQjlBytes);
                    cf[u] = __fmul_rn(a.norms[r], kQjlCoef);
                }
            }
#pragma unroll
            for (int u = 0; u < kDeqFlight; ++u) {
                float v[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] = __shfl_sync(kFullMask, cb_lane, (p[u] >> (4 * k)) & 0xF);
                if (a.with_qjl) {
                    const uint64_t sig = ((uint64_t)sg[u].y << 32) | sg[u].x;
#pragma unroll
                    for (int k = 0; k < 4; ++k)         // sum_i s_i * g_id with s, g in {-1,+1}: matches minus mismatches
                        v[k] = __fadd_rn(v[k], __fmul_rn((float)(kQjlDim - 2 * __popcll(sig ^ gc[k])), cf[u]));
                }
                if (t + u < t_end)
                    *reinterpret_cast<float4*>(a.out + (out0 + t + u) * kHeadDim + 4 * lane) = make_float4(v[0], v[1], v[2], v[3]);
            }
        }
    }
}

static int grid_for_rows(int64_t n_rows) {
    int64_t blocks = (n_rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t cap = 148 * 8 * 4;     // a few resident waves of 256-thread blocks per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <int DT>
static int32_t launch_quantize(const CodecArgs& a, int rotate, cudaStream_t st) {
    const int grid = grid_for_rows(a.B * a.H * a.T);
    if (rotate) quantize_kernel<DT, true><<<grid, kWarpsPerBlock * 32, 0, st>>>(a);
    else        quantize_kernel<DT, false><<<grid, kWarpsPerBlock * 32, 0, st>>>(a);
    return check_cuda(cudaGetLastError(), "quantize_kernel launch");
}

// OMNI_QUANT_KERNEL=scan forces the one-row-per-warp kernel (tests and profiling); default: the fast
// kernel whenever the call fits it.
static bool fast_kernel_allowed() {
    const char* e = getenv("OMNI_QUANT_KERNEL");
    return !(e && e[0] == 's');
}

// Row-seeded calls: row i uses seed (user_id mod 1024) xor (base + i).  The xor only touches the low ten bits, so
// the rows whose key base + i lies in one aligned block of 1,024 keys use exactly the seeds of that block, in a
// permuted order.  Block 0 is the resident table; later blocks come from extended_tables_for_block.  `fn` is
// called once per block with (first row, row count, key of the first row, tables).
template <class Fn>
static int32_t for_each_seed_block(int32_t base, int32_t user_id, int64_t n_rows, Fn&& fn) {
    const DeviceTables* tb = tables_for_current_device();
    if (!tb) return OMNI_ERR_NOT_INIT;
    for (int64_t r = 0; r < n_rows;) {
        const int64_t key = (int64_t)base + r, block = key >> 10;
        const int64_t end_key = std::min<int64_t>((block + 1) << 10, (int64_t)base + n_rows);
        DeviceTables t = *tb;
        if (block > 0) {
            std::vector<int> slots;
            slots.reserve((size_t)(end_key - key));
            for (int64_t k = key; k < end_key; ++k) slots.push_back((int)(((user_id & 1023) ^ k) & 1023));
            const int32_t rc = extended_tables_for_block(block, slots, &t);
            if (rc != OMNI_OK) return rc;
        }
        const int32_t rc = fn(r, end_key - key, (int32_t)key, t);
        if (rc != OMNI_OK) return rc;
        r += end_key - key;
    }
    return OMNI_OK;
}

static int32_t quantize_common(CodecArgs& a, int32_t dtype, int32_t rotate, void* stream) {
    if (!a.g_rows) {
        const DeviceTables* tb = tables_for_current_device();
        if (!tb) return OMNI_ERR_NOT_INIT;
        a.g_rows = tb->rows; a.g_cols = tb->cols;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (!a.row_seeded && fast_kernel_allowed()) {
        FastQuantArgs f{a.x, a.xs_b, a.xs_h, a.xs_t, a.codebooks, a.cb_per_head, a.user_ids, a.user_id, a.B, a.H, a.T,
                        a.nib, a.qjl, a.norms, a.os_b, a.os_h, a.out_offsets, a.out_offset, a.g_rows};
        if (fast_quantize_eligible(f, dtype)) return launch_fast_quantize(f, dtype, rotate, st);
    }
    switch (dtype) {
        case OMNI_F32:  return launch_quantize<OMNI_F32>(a, rotate, st);
        case OMNI_BF16: return launch_quantize<OMNI_BF16>(a, rotate, st);
        case OMNI_F16:  return launch_quantize<OMNI_F16>(a, rotate, st);
    }
    return set_error(OMNI_ERR_ARG, "unknown dtype code %d", dtype);
}

}  // namespace omni

using namespace omni;

extern "C" int32_t omni_rotate(const void* x, void* y, int64_t n_rows, int32_t dtype, void* stream) {
    OMNI_REQUIRE(n_rows >= 0, OMNI_ERR_ARG, "omni_rotate: n_rows < 0");
    if (n_rows == 0) return OMNI_OK;
    OMNI_REQUIRE(x && y, OMNI_ERR_ARG, "omni_rotate: NULL buffer");
    OMNI_REQUIRE(aligned(x, 16) && aligned(y, 16), OMNI_ERR_ARG, "omni_rotate: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    // 16-bit rows: 8 rows per warp (fewer cross-lane stages; the warp-per-row kernel is shuffle-bound there).
    // fp32 rows: warp per row, whose 16-byte accesses are fully coalesced (98 % of the copy peak).
    // OMNI_ROTATE_KERNEL=rows8|warp forces one of them (tests).
    const char* forced = getenv("OMNI_ROTATE_KERNEL");
    const bool rows8 = forced ? forced[0] == 'r' : dtype != OMNI_F32;
    if (rows8) return launch_fast_rotate(x, y, n_rows, dtype, st);
    const int grid = grid_for_rows(n_rows);
    switch (dtype) {
        case OMNI_F32:  rotate_kernel<OMNI_F32><<<grid, kWarpsPerBlock * 32, 0, st>>>(x, y, n_rows); break;
        case OMNI_BF16: rotate_kernel<OMNI_BF16><<<grid, kWarpsPerBlock * 32, 0, st>>>(x, y, n_rows); break;
        case OMNI_F16:  rotate_kernel<OMNI_F16><<<grid, kWarpsPerBlock * 32, 0, st>>>(x, y, n_rows); break;
        default: return set_error(OMNI_ERR_ARG, "omni_rotate: unknown dtype code %d", dtype);
    }
    return check_cuda(cudaGetLastError(), "rotate_kernel launch");
}

extern "C" int32_t omni_quantize_heads(const void* x, int32_t dtype, int32_t rotate,
                                       const float* codebooks, int32_t cb_per_head,
                                       const int32_t* user_ids, int32_t user_id,
                                       int64_t B, int32_t H, int64_t T,
                                       int64_t xs_b, int64_t xs_h, int64_t xs_t,
                                       uint8_t* nib, uint8_t* qjl, float* norms,
                                       int64_t os_b, int64_t os_h,
                                       const int64_t* out_offsets, int64_t out_offset, void* stream) {
    OMNI_REQUIRE(B >= 0 && H >= 0 && T >= 0, OMNI_ERR_ARG, "omni_quantize_heads: negative extent");
    if (B == 0 || H == 0 || T == 0) return OMNI_OK;
    OMNI_REQUIRE(H <= kSeeds, OMNI_ERR_UNSUPPORTED, "omni_quantize_heads: H=%d exceeds %d heads", H, kSeeds);
    OMNI_REQUIRE(x && codebooks && nib, OMNI_ERR_ARG, "omni_quantize_heads: NULL buffer");
    OMNI_REQUIRE((qjl == nullptr) == (norms == nullptr), OMNI_ERR_ARG,
                 "omni_quantize_heads: qjl and norms must both be given or both be NULL (nibble rows only)");
    const size_t in_align = dtype == OMNI_F32 ? 16 : 8;
    OMNI_REQUIRE(aligned(x, in_align) && xs_b % 4 == 0 && xs_h % 4 == 0 && xs_t % 4 == 0, OMNI_ERR_ARG,
                 "omni_quantize_heads: input rows must be %zu-byte aligned (strides multiples of 4 elements)", in_align);
    OMNI_REQUIRE(aligned(qjl, 8) && aligned(nib, 2) && aligned(norms, 4), OMNI_ERR_ARG,
                 "omni_quantize_heads: packed outputs misaligned");
    CodecArgs a{};
    a.x = x; a.xs_b = xs_b; a.xs_h = xs_h; a.xs_t = xs_t;
    a.codebooks = codebooks; a.cb_per_head = cb_per_head;
    a.user_ids = user_ids; a.user_id = user_id;
    a.B = B; a.H = H; a.T = T;
    a.nib = nib; a.qjl = qjl; a.norms = norms; a.os_b = os_b; a.os_h = os_h;
    a.out_offsets = out_offsets; a.out_offset = out_offset;
    return quantize_common(a, dtype, rotate, stream);
}

extern "C" int32_t omni_quantize_rows(const float* x, const float* codebook, int32_t base_head_idx, int32_t user_id,
                                      int64_t n_rows, uint8_t* nib, uint8_t* qjl, float* norms, void* stream) {
    OMNI_REQUIRE(n_rows >= 0, OMNI_ERR_ARG, "omni_quantize_rows: n_rows < 0");
    if (n_rows == 0) return OMNI_OK;
    OMNI_REQUIRE(base_head_idx >= 0 && (int64_t)base_head_idx + n_rows <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED,
                 "omni_quantize_rows: row keys [%d, %lld) leave the 31-bit key space", base_head_idx,
                 (long long)(base_head_idx + n_rows));
    OMNI_REQUIRE(x && codebook && nib && qjl && norms, OMNI_ERR_ARG, "omni_quantize_rows: NULL buffer");
    OMNI_REQUIRE(aligned(x, 16) && aligned(qjl, 8) && aligned(nib, 2), OMNI_ERR_ARG, "omni_quantize_rows: misaligned buffer");
    return for_each_seed_block(base_head_idx, user_id, n_rows, [&](int64_t r0, int64_t n, int32_t key0, const DeviceTables& t) {
        CodecArgs a{};
        a.x = x + r0 * kHeadDim; a.xs_b = kHeadDim; a.xs_h = 0; a.xs_t = 0;
        a.codebooks = codebook; a.cb_per_head = 0; a.user_id = user_id;
        a.B = n; a.H = 1; a.T = 1;
        a.nib = nib + r0 * kNibBytes; a.qjl = qjl + r0 * kQjlBytes; a.norms = norms + r0; a.os_b = 1; a.os_h = 0;
        a.row_seeded = 1; a.base_head_idx = key0;
        a.g_rows = t.rows; a.g_cols = t.cols;
        return quantize_common(a, OMNI_F32, 0, stream);
    });
}

static int32_t dequantize_common(CodecArgs& a, void* stream) {
    if (!a.g_rows) {
        const DeviceTables* tb = tables_for_current_device();
        if (!tb) return OMNI_ERR_NOT_INIT;
        a.g_rows = tb->rows; a.g_cols = tb->cols;
    }
    if (!a.row_seeded) {
        const int grid = grid_for_rows(a.B * a.H * ((a.T + kDeqRun - 1) / kDeqRun));
        dequantize_heads_kernel<<<grid, kWarpsPerBlock * 32, 0, (cudaStream_t)stream>>>(a);
        return check_cuda(cudaGetLastError(), "dequantize_heads_kernel launch");
    }
    const int grid = grid_for_rows(a.B * a.H * a.T);
    dequantize_kernel<<<grid, kWarpsPerBlock * 32, 0, (cudaStream_t)stream>>>(a);
    return check_cuda(cudaGetLastError(), "dequantize_kernel launch");
}

extern "C" int32_t omni_dequantize_heads(const uint8_t* nib, const uint8_t* qjl, const float* norms,
                                         const float* codebooks, int32_t cb_per_head,
                                         const int32_t* user_ids, int32_t user_id,
                                         int64_t B, int32_t H, int64_t T, int64_t is_b, int64_t is_h,
                                         int32_t with_qjl, float* out, void* stream) {
    OMNI_REQUIRE(B >= 0 && H >= 0 && T >= 0, OMNI_ERR_ARG, "omni_dequantize_heads: negative extent");
    if (B == 0 || H == 0 || T == 0) return OMNI_OK;
    OMNI_REQUIRE(H <= kSeeds, OMNI_ERR_UNSUPPORTED, "omni_dequantize_heads: H=%d exceeds %d heads", H, kSeeds);
    OMNI_REQUIRE(nib && codebooks && out && (!with_qjl || (qjl && norms)), OMNI_ERR_ARG, "omni_dequantize_heads: NULL buffer");
    OMNI_REQUIRE(aligned(out, 16) && aligned(nib, 2) && (!with_qjl || aligned(qjl, 8)), OMNI_ERR_ARG,
                 "omni_dequantize_heads: misaligned buffer");
    CodecArgs a{};
    a.codebooks = codebooks; a.cb_per_head = cb_per_head; a.user_ids = user_ids; a.user_id = user_id;
    a.B = B; a.H = H; a.T = T;
    a.nib = const_cast<uint8_t*>(nib); a.qjl = const_cast<uint8_t*>(qjl); a.norms = const_cast<float*>(norms);
    a.os_b = is_b; a.os_h = is_h; a.with_qjl = with_qjl; a.out = out;
    return dequantize_common(a, stream);
}

extern "C" int32_t omni_dequantize_rows(const uint8_t* nib, const uint8_t* qjl, const float* norms,
                                        const float* codebook, int32_t base_head_idx, int32_t user_id,
                                        int64_t n_rows, int32_t with_qjl, float* out, void* stream) {
    OMNI_REQUIRE(n_rows >= 0, OMNI_ERR_ARG, "omni_dequantize_rows: n_rows < 0");
    if (n_rows == 0) return OMNI_OK;
    OMNI_REQUIRE(base_head_idx >= 0 && (int64_t)base_head_idx + n_rows <= 0x7fffffffLL, OMNI_ERR_UNSUPPORTED,
                 "omni_dequantize_rows: row keys [%d, %lld) leave the 31-bit key space", base_head_idx,
                 (long long)(base_head_idx + n_rows));
    OMNI_REQUIRE(nib && codebook && out && (!with_qjl || (qjl && norms)), OMNI_ERR_ARG, "omni_dequantize_rows: NULL buffer");
    OMNI_REQUIRE(aligned(out, 16) && aligned(nib, 2) && (!with_qjl || aligned(qjl, 8)), OMNI_ERR_ARG,
                 "omni_dequantize_rows: misaligned buffer");
    return for_each_seed_block(base_head_idx, user_id, n_rows, [&](int64_t r0, int64_t n, int32_t key0, const DeviceTables& t) {
        CodecArgs a{};
        a.codebooks = codebook; a.cb_per_head = 0; a.user_id = user_id;
        a.B = n; a.H = 1; a.T = 1;
        a.nib = const_cast<uint8_t*>(nib) + r0 * kNibBytes;
        a.qjl = qjl ? const_cast<uint8_t*>(qjl) + r0 * kQjlBytes : nullptr;
        a.norms = norms ? const_cast<float*>(norms) + r0 : nullptr;
        a.os_b = 1; a.os_h = 0; a.with_qjl = with_qjl; a.out = out + r0 * kHeadDim;
        a.row_seeded = 1; a.base_head_idx = key0;
        a.g_rows = t.rows; a.g_cols = t.cols;
        return dequantize_common(a, stream);
    });
}
