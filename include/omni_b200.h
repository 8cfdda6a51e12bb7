/*
 * omni_b200 -- C ABI of the B200 (sm_100a) quantized-KV codec and fused decode attention.
 *
 * This is the boundary a host binding (ctypes, cffi, cgo ...) talks to.  Plain
 * pointers and sizes only: no torch, no C++ types.  Each entry point names the
 * routine of the OmniStack-RS reference (path inside that project : line) whose
 * GPU work it replaces.
 *
 * Conventions
 *   - every function returns an int32 status (OMNI_OK on success); a message for
 *     the last failure on the calling thread is available from omni_last_error();
 *   - pointers named *_dev / documented "device" are device addresses on the
 *     device that is current when the call is made; the library never allocates or
 *     frees caller-visible memory, it only owns the Rademacher tables that
 *     omni_init() uploads;
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous with
 *     respect to the host unless stated otherwise;
 *   - a "row" is one 128-element (user, head, token) vector.  A packed row is
 *     64 nibble bytes + 8 sign bytes + one fp32 norm, held in three arrays;
 *   - the seed of the +-1 projection matrix of (user, head h) is
 *     (user_id mod 1024) xor h, as in the reference (kernels/quantize.py:293-295,583).
 */
#ifndef OMNI_B200_H_
#define OMNI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMNI_HEAD_DIM   128
#define OMNI_QJL_DIM    64
#define OMNI_NIB_BYTES  64
#define OMNI_QJL_BYTES  8
#define OMNI_N_SEEDS    1024

/* status codes */
#define OMNI_OK               0
#define OMNI_ERR_ARG          1   /* null pointer, negative size, misaligned buffer            */
#define OMNI_ERR_UNSUPPORTED  2   /* shape outside what the kernels handle                      */
#define OMNI_ERR_CUDA         3   /* CUDA runtime / launch error, see omni_last_error()         */
#define OMNI_ERR_DEVICE_WAIT  4   /* a bounded device-side wait expired (status word non-zero)  */
#define OMNI_ERR_NOT_INIT     5   /* omni_init() has not been called for the current device     */

/* values a kernel may leave in a caller's device status word (0 = nothing to report) */
#define OMNI_STATUS_WAIT_EXPIRED  4   /* a bounded device-side wait ran out                      */
#define OMNI_STATUS_BAD_INDEX     7   /* an adapter index was at or past the adapter count       */
#define OMNI_STATUS_BAD_CODEBOOK  8   /* an attention call was given an infinite or NaN centroid */

/* element types of floating-point inputs */
#define OMNI_F32   0
#define OMNI_BF16  1
#define OMNI_F16   2

/* Library life cycle.  omni_init builds the 1024-seed Rademacher tables on the host
 * with MT19937 (the CPU generator behind torch.Generator, which the reference draws
 * G from: kernels/quantize.py:410-414) and uploads them to `device`.  Idempotent. */
int32_t omni_init(int32_t device);
int32_t omni_shutdown(void);
const char* omni_last_error(void);
int32_t omni_abi_version(void);

/* Host-only: copy the bit-packed G rows of seeds [seed_begin, seed_begin+seed_count)
 * to `out` (seed_count * 64 * 4 uint32; bit d of projection row i sits in word d/32,
 * position d%32).  Replaces the per-call torch.randint of kernels/quantize.py:410-414. */
int32_t omni_gtable_host(uint32_t* out, int32_t seed_begin, int32_t seed_count);

/* Normalised 128-point Walsh-Hadamard rotation of n_rows contiguous rows
 * (kernels/hadamard.py:51-85 `_wht_torch`, :155-191 `_wht_rotate`, :196 `rotate_queries`,
 * :214 `rotate_kv_cache`).  x and y are device arrays of `dtype`; y may equal x. */
int32_t omni_rotate(const void* x, void* y, int64_t n_rows, int32_t dtype, void* stream);

/* INT4 Lloyd-Max + QJL codec over x[B][H][T][128] (kernels/quantize.py:542-590
 * `quantize_heads`; with rotate != 0 it also applies the rotation first, i.e. the bake
 * step quantize_heads(_wht_torch(x)) of scripts/run_criteo_benchmark.py:355,367, and
 * with out_offsets / out_offset it appends into a preallocated cache).
 *   x            device, element strides xs_b, xs_h, xs_t (last axis contiguous)
 *   codebooks    device fp32, [H][16] when cb_per_head != 0, else [16]
 *   user_ids     device int32[B] or NULL (then `user_id` is used for every b)
 *   nib/qjl/norms device outputs; row index of (b,h,t) is
 *                b*os_b + h*os_h + t + (out_offsets ? out_offsets[b] : out_offset)
 *                and row r occupies nib[64 r .. ], qjl[8 r ..], norms[r]
 *   out_offsets  device int64[B] or NULL
 * qjl and norms may both be NULL: only the nibble rows are written then and the projections are
 * skipped (V rows, whose sign bits and norms attention never reads: kernels/fused_attention.py:455-464). */
int32_t omni_quantize_heads(const void* x, int32_t dtype, int32_t rotate,
                            const float* codebooks, int32_t cb_per_head,
                            const int32_t* user_ids, int32_t user_id,
                            int64_t B, int32_t H, int64_t T,
                            int64_t xs_b, int64_t xs_h, int64_t xs_t,
                            uint8_t* nib, uint8_t* qjl, float* norms,
                            int64_t os_b, int64_t os_h,
                            const int64_t* out_offsets, int64_t out_offset,
                            void* stream);

/* Inverse codec to fp32 out[B][H][T][128] (kernels/quantize.py:593-640 `dequantize_heads`).
 * Packed inputs use row strides is_b, is_h as above; with_qjl == 0 gives cb[code] only. */
int32_t omni_dequantize_heads(const uint8_t* nib, const uint8_t* qjl, const float* norms,
                              const float* codebooks, int32_t cb_per_head,
                              const int32_t* user_ids, int32_t user_id,
                              int64_t B, int32_t H, int64_t T,
                              int64_t is_b, int64_t is_h, int32_t with_qjl,
                              float* out, void* stream);

/* Unpacked QJL residual coding (quantization/qjl.py:78-104 `RademacherQJL.encode`, :106-135 `reconstruct`): one
 * byte (0/1) per projection, G selected by `seed` = (user_id mod 1024) xor head_idx in [0, 1024).
 * encode: err device fp32 [n_rows][128] -> signs device u8 [n_rows][64] (1 where the projection is >= 0,
 * decided in fp64) and norms device fp32 [n_rows].  reconstruct: signs, norms -> out device fp32 [n_rows][128]
 * = (sum_i (2 signs_i - 1) G[i][d]) * (norm * sqrt(2/pi) / 128).                                              */
int32_t omni_qjl_encode_bool(const float* err, int64_t n_rows, int32_t seed, uint8_t* signs, float* norms, void* stream);
int32_t omni_qjl_reconstruct_bool(const uint8_t* signs, const float* norms, int64_t n_rows, int32_t seed, float* out,
                                  void* stream);

/* Lloyd-Max fit of 16-level codebooks (quantization/codebook.py:64-108 `LloydMaxCalibrator.fit`, :148-172
 * `calibrate_per_group`): equal-mass initialisation, first-index nearest-centroid assignment in fp32, mean
 * update (an empty cell keeps its centroid), stop once the largest move is below `tol` or after `max_iters`
 * iterations, ascending output.  `sorted` holds the fp32 samples of all groups back to back on the device, each
 * group in ASCENDING order; group g is sorted[group_offsets[g] .. group_offsets[g+1]) (device int64
 * [n_groups+1], first entry 0, last n_total, at least 16 samples per group).  `workspace`: device scratch of
 * omni_lloyd_max_workspace_bytes(n_total) bytes (fp64 prefix sums).  codebooks: device fp32 [n_groups][16];
 * iters_out: device int32 [n_groups] (iterations run) or NULL.  Means are formed in fp64 and rounded once, so
 * the result equals the reference's to a few fp32 ulps rather than bit for bit.                                */
size_t  omni_lloyd_max_workspace_bytes(int64_t n_total);
int32_t omni_lloyd_max_fit(const float* sorted, int64_t n_total, const int64_t* group_offsets, int32_t n_groups,
                           int32_t max_iters, double tol, void* workspace, size_t workspace_bytes,
                           float* codebooks, int32_t* iters_out, void* stream);

/* Row-seeded codec (kernels/quantize.py:456-499 `quantize_rows`, :502-537
 * `dequantize_rows`): row i of n_rows contiguous fp32 rows uses seed
 * (user_id mod 1024) xor (base_head_idx + i), for any non-negative row key base_head_idx + i below 2^31 (the
 * reference seeds one MT19937 stream per row, kernels/quantize.py:486-492, :524-535).  Seeds below 1,024 come from
 * the resident tables; the G of larger seeds is generated on the host and uploaded one aligned block of 1,024
 * seeds at a time into a second, library-owned pair of tables, which makes such calls synchronise the device
 * (about 25 us of host time per new seed).  One shared [16] codebook. */
int32_t omni_quantize_rows(const float* x, const float* codebook, int32_t base_head_idx, int32_t user_id,
                           int64_t n_rows, uint8_t* nib, uint8_t* qjl, float* norms, void* stream);
int32_t omni_dequantize_rows(const uint8_t* nib, const uint8_t* qjl, const float* norms,
                             const float* codebook, int32_t base_head_idx, int32_t user_id,
                             int64_t n_rows, int32_t with_qjl, float* out, void* stream);

/* Fused attention over the packed cache (kernels/fused_attention.py:90-291
 * `_fused_attention_kernel`, :320 `_fused_attn_triton`, :471-565 `OmniAttention` /
 * `omni_attn`; numerics follow the CPU path :435-466 `_fused_attn_python`).
 *   q            device [B][Hq][T][128] of q_dtype, contiguous
 *   k_nib,k_qjl,k_norms,v_nib  packed cache; row of (slot, kv head h, key s) is
 *                slot*ks_b + h*ks_h + s, slot = cache_slots ? cache_slots[b] : b
 *   seq_lens     device int32[B] or NULL (then every user has S keys); values are
 *                clamped to [0, S]; a user with 0 keys gets a zero output row
 *   scale        softmax scale (the reference default is 1/sqrt(128))
 *   rotate_q / unrotate_out  fold the Walsh-Hadamard rotation into the query /
 *                out of the result (both 0 reproduces the reference, which expects a
 *                rotated q and returns the output in rotated space)
 *   v_paired     0: v_nib is in the reference layout.  1: it is in the pair layout that
 *                omni_v_pair_groups produces, for every group of eight keys that lies completely
 *                below the user's length (seq_lens[b], or S); the user's last, incomplete group
 *                is in the reference layout.  Same results, fewer instructions per key.
 *   n_splits     >= 1 partitions of the key axis; with n_splits > 1 `workspace` must
 *                hold omni_qattn_workspace_bytes(...) bytes of device scratch
 *   out          device fp32 [B][Hq][T][128]
 *   status_word  device int32 or NULL; set non-zero by the kernel if a bounded wait
 *                expires (OMNI_STATUS_WAIT_EXPIRED; the kernels never trap; the warp that
 *                gave up leaves neutral results -- zero rows, or partial states that a
 *                split-K merge ignores -- for the work it abandons) or if a centroid is
 *                infinite or NaN (OMNI_STATUS_BAD_CODEBOOK)
 * Codebooks may hold any finite fp32 centroids (kernels/quantize.py:620-636).  The tensor-core
 * kernel dequantises through fp16 tables, which meet the 3e-3 output budget only while every
 * |centroid| < 8; both kernels test that on the device, and a call with a wider codebook is
 * served by the fp32 CUDA-core kernel (slower, same results as the reference's fp32 path).  */
size_t  omni_qattn_workspace_bytes(int64_t B, int32_t Hq, int32_t T, int32_t n_splits);
int32_t omni_qattn_decode(const void* q, int32_t q_dtype,
                          const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                          const uint8_t* v_nib,
                          const float* codebooks, int32_t cb_per_head,
                          const int32_t* user_ids, int32_t user_id,
                          const int32_t* seq_lens, const int32_t* cache_slots,
                          int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                          int64_t ks_b, int64_t ks_h,
                          float scale, int32_t with_qjl, int32_t rotate_q, int32_t unrotate_out, int32_t v_paired,
                          int32_t n_splits, void* workspace, size_t workspace_bytes,
                          float* out, int32_t* status_word, void* stream);

/* Pair layout of the V nibble rows of a resident cache (no counterpart in the reference, whose tensors keep one
 * key per row; this is an internal format of a cache that this library appends to and reads).  The tensor-core
 * kernel's P.V product pairs two keys per operand register, so its table index is (nibble of key a) | (nibble of
 * key b) << 4.  Within each group of eight consecutive keys the pairs are (0,3), (1,2), (4,7), (5,6); the row of a
 * pair's first key receives byte j = code[a][2j] | code[b][2j] << 4 (even dims of both keys), the row of its
 * second key the odd dims.  The call converts, in place, the groups that became complete when a user's length
 * grew from lens_before[b] to lens_after[b] (device int64 [B]; or the scalars len_before / len_after when the
 * arrays are NULL): groups [before / 8, after / 8).  Applying it twice restores the reference layout.  Rows as in
 * omni_qattn_decode: (b, h, s) at b*ks_b + h*ks_h + s, S keys of capacity per (b, h). */
int32_t omni_v_pair_groups(uint8_t* v_nib, int64_t B, int32_t H, int64_t S, int64_t ks_b, int64_t ks_h,
                           const int64_t* lens_before, int64_t len_before,
                           const int64_t* lens_after, int64_t len_after, void* stream);

/* Per-user low-rank query update ahead of attention (kernels/fused_attention.py:166-191 fused prologue,
 * :401-430 `_apply_lora_to_q`): out[b,h,t,:] = q[b,h,t,:] + alpha * ((x[b,t,:] A[i]^T) B[i]^T)[h,:] with
 * i = lora_indices[b]; i < 0 copies q unchanged.  x [B][T][hidden], lora_a [n][rank][hidden],
 * lora_b [n][Hq*128][rank], all fp32 device arrays; q of q_dtype; out fp32 [B][Hq][T][128]; rank <= 128.
 * n_adapters = n: a row whose index is >= n is copied unchanged and `status_word` (device int32 or NULL) is
 * raised to OMNI_STATUS_BAD_INDEX (the reference's gather would fail there); no host-side check, no sync. */
int32_t omni_lora_q(const void* q, int32_t q_dtype, const float* x, const float* lora_a, const float* lora_b,
                    const int32_t* lora_indices, int32_t n_adapters, float lora_alpha, int64_t B, int32_t Hq,
                    int32_t T, int32_t hidden, int32_t rank, float* out, int32_t* status_word, void* stream);

/* Attention with the per-user low-rank query update in the same call (the reference passes x, lora_a, lora_b,
 * lora_indices and lora_alpha to `omni_attn`, kernels/fused_attention.py:537-560, and applies them in the
 * kernel prologue :166-191).  `lora` == NULL makes this omni_qattn_decode.  Otherwise the update is applied in the
 * prologue of the attention kernel that serves the call (the warp that owns a tile of query columns computes the
 * down projection and its columns' part of the up projection) when that is the warp-level tensor-core kernel and
 * the adapter is small (rank <= 32, rank * hidden <= 8192); for other calls it runs first on the same stream as a
 * launch of its own, into the front of `workspace`.  Both forms give the same bits.  The environment variable
 * OMNI_LORA_FOLD=0 / 1 forces the separate launch / the fold.  `workspace` must hold
 * omni_qattn_lora_workspace_bytes(...) bytes either way (room for the updated fp32 queries, then the split-K
 * partial states); q may be of any q_dtype.                                                                  */
typedef struct omni_lora {
    const float*   x;             /* device fp32 [B][T][hidden]                 */
    const float*   lora_a;        /* device fp32 [n_adapters][rank][hidden]     */
    const float*   lora_b;        /* device fp32 [n_adapters][Hq*128][rank]     */
    const int32_t* lora_indices;  /* device int32 [B]; < 0 = no adapter         */
    int32_t        n_adapters;
    int32_t        hidden;
    int32_t        rank;          /* <= 128                                     */
    float          alpha;
} omni_lora_t;
size_t  omni_qattn_lora_workspace_bytes(int64_t B, int32_t Hq, int32_t T, int32_t n_splits);
int32_t omni_qattn_decode_lora(const void* q, int32_t q_dtype,
                               const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                               const uint8_t* v_nib,
                               const float* codebooks, int32_t cb_per_head,
                               const int32_t* user_ids, int32_t user_id,
                               const int32_t* seq_lens, const int32_t* cache_slots,
                               int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                               int64_t ks_b, int64_t ks_h,
                               float scale, int32_t with_qjl, int32_t rotate_q, int32_t unrotate_out, int32_t v_paired,
                               int32_t n_splits, void* workspace, size_t workspace_bytes,
                               float* out, int32_t* status_word, void* stream, const omni_lora_t* lora);

/* Allocation-free decode attention.  No counterpart in the reference: it exists for hosts
 * that must not allocate device memory when they call into this library -- an inference
 * server or plugin host that owns the whole device heap and hands its plugins fixed
 * buffers, or a latency-critical serving loop that cannot afford the device-wide
 * synchronisation an allocation implies.  It is omni_qattn_decode with the split-K
 * workspace (and a private copy of the Rademacher rows) held in arrays that are part of
 * the library image, so neither this call nor any set-up it needs (omni_init included --
 * it is not required here) calls cudaMalloc/cudaFree or an allocating library routine.
 *   - the caller still passes every input and the output buffer;
 *   - the scratch array is omni_qattn_noalloc_scratch_bytes() = 32 MiB, enough for
 *     B*Hq*T*n_splits <= 63,542 partial states; larger requests return
 *     OMNI_ERR_UNSUPPORTED with a message (n_splits == 1 needs no scratch and is never
 *     rejected for size); every device that loads the library carries the 33 MiB until exit;
 *   - the FIRST call on each device resolves the arrays' device addresses, uploads the
 *     1 MiB row table with a blocking copy and then waits for the whole device
 *     (cudaDeviceSynchronize), so that a kernel on any stream, non-blocking ones included,
 *     finds the table complete: make that call once, with the device current, before any
 *     stream capture begins;
 *   - there is no status_word argument: the kernels report an expired bounded wait (and a
 *     non-finite centroid) in a status word that is also part of the library image;
 *     omni_qattn_noalloc_status() reads it;
 *   - all calls on a device share the one scratch array.  Every partial state a launch reads
 *     is written by that same launch first, so stale contents of earlier calls are harmless,
 *     but two calls whose kernels overlap on the GPU (different streams) race on it: keep
 *     calls with n_splits > 1 on one stream or order them with events.                    */
size_t  omni_qattn_noalloc_scratch_bytes(void);
int32_t omni_qattn_decode_noalloc(const void* q, int32_t q_dtype,
                                  const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                                  const uint8_t* v_nib,
                                  const float* codebooks, int32_t cb_per_head,
                                  const int32_t* user_ids, int32_t user_id,
                                  const int32_t* seq_lens, const int32_t* cache_slots,
                                  int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                                  int64_t ks_b, int64_t ks_h,
                                  float scale, int32_t with_qjl, int32_t rotate_q, int32_t unrotate_out, int32_t v_paired,
                                  int32_t n_splits, float* out, void* stream);
/* Reads the status word of the allocation-free entry point on the current device into *value_out (0 = nothing
 * to report, else an OMNI_STATUS_* value) and, with clear != 0, resets it.  Waits for the device first. */
int32_t omni_qattn_noalloc_status(int32_t* value_out, int32_t clear);

/* Self-test of the device-side bounded waits (no counterpart in the reference).  Launches one warp that waits,
 * for at most `poll_limit` polls (1 .. 2^20), on an mbarrier nothing ever arrives on -- the same wait routine the
 * decode kernel uses on its TMA ring.  The wait runs out, the warp writes OMNI_STATUS_WAIT_EXPIRED to
 * `status_word` (device int32, required) and the kernel returns normally; nothing hangs, faults or traps. */
int32_t omni_diag_bounded_wait(int32_t poll_limit, int32_t* status_word, void* stream);

/* One decode step with HOST query / result buffers (the serving loop of
 * scripts/run_criteo_benchmark.py:481-560, where q arrives per step and the cache is
 * resident); returns after everything has completed.
 *   - q_host and out_host page-locked (cudaHostAlloc / cudaHostRegister, e.g. a pinned torch tensor): the attention
 *     kernels read the queries and write the result rows in host memory themselves, so the transfer overlaps the
 *     attention work completely; q_stage / out_stage may be NULL, and a call without split-K (or whose workspace
 *     holds the partial states of all B users) is one launch whatever n_chunks says;
 *   - otherwise: q_host -> q_stage (device), omni_qattn_decode, out_stage (device) -> out_host, in `n_chunks` user
 *     chunks pipelined over two internal streams (the environment variable OMNI_HOST_STEP=staged selects this form
 *     for page-locked buffers as well).
 * Remaining arguments as in omni_qattn_decode; with n_splits > 1 the workspace must hold two slices of
 * omni_qattn_workspace_bytes(ceil(B / n_chunks), Hq, T, n_splits) bytes (one per internal stream).
 * status_word: device int32 or NULL, as in omni_qattn_decode. */
int32_t omni_qattn_decode_host(const void* q_host, int32_t q_dtype, void* q_stage,
                               const uint8_t* k_nib, const uint8_t* k_qjl, const float* k_norms,
                               const uint8_t* v_nib,
                               const float* codebooks, int32_t cb_per_head,
                               const int32_t* user_ids, int32_t user_id,
                               const int32_t* seq_lens, const int32_t* cache_slots,
                               int64_t B, int32_t Hq, int32_t Hkv, int32_t T, int64_t S,
                               int64_t ks_b, int64_t ks_h,
                               float scale, int32_t with_qjl, int32_t v_paired,
                               float* out_stage, float* out_host, int32_t n_chunks,
                               int32_t n_splits, void* workspace, size_t workspace_bytes,
                               int32_t* status_word);

#ifdef __cplusplus
}
#endif
#endif /* OMNI_B200_H_ */
