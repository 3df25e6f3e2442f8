/* wave_b200 — C ABI of the B200 (sm_100a) MXFP4 scaled-GEMM library.
 *
 * This is the boundary a binding of the reference would call instead of its own launch shim.
 * In the reference, a compiled kernel is launched by the C++ extension `wave_runtime`
 * (wave_lang/kernel/wave/runtime/runtime.cpp:123-203 `launch`, :231-240 `load_binary`), driven
 * from Python by `invoke_with_wave_runtime` (wave_lang/kernel/wave/utils/run_utils.py:62-134):
 * raw device pointers, problem sizes and the caller's stream go in, the launch is asynchronous
 * and nothing is returned but an error. The entry points below keep that contract: plain
 * pointers and sizes, an explicit stream, no allocation of caller-visible memory, no implicit
 * synchronisation, an int status with a thread-local message.
 *
 * Tensor contract (wave_lang/kernel/wave/templates/gemm.py:171-175):
 *   a        uint8 [M, K/2]   packed E2M1, two codes per byte, even k in the low nibble
 *   a_scale  uint8 [M, K/32]  E8M0, one per 32 K elements
 *   b        uint8 [N, K/2]   (N-major: the kernel computes a * b^T)
 *   b_scale  uint8 [N, K/32]
 *   c        f32 or bf16 [M, N], row pitch ldc elements, fully overwritten
 * K must be a multiple of 32. a, b must be 16-byte aligned and contiguous.
 *
 * The GEMM entry points read scales in the tcgen05 scale-factor layout ("packed scales");
 * wb200_repack_scales converts the row-major arrays above.
 */
#ifndef WAVE_B200_H_
#define WAVE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------- */
#define WB200_OK 0
#define WB200_ERR_INVALID_ARG (-1)   /* bad size, null pointer, unknown dtype or flag */
#define WB200_ERR_ALIGNMENT (-2)     /* pointer or pitch not aligned as required */
#define WB200_ERR_WORKSPACE (-3)     /* workspace missing or too small */
#define WB200_ERR_UNSUPPORTED (-4)   /* device is not sm_100, or shape outside the kernel's range */
#define WB200_ERR_DEVICE_TIMEOUT (-5) /* a bounded device-side wait gave up; results are invalid */
#define WB200_ERR_CUDA (-6)          /* a CUDA runtime/driver call failed; see wb200_last_error */

/* ---- output element types ------------------------------------------------------------------ */
#define WB200_F32 0
#define WB200_BF16 1

/* ---- flags of wb200_mxfp4_gemm ------------------------------------------------------------- */
#define WB200_PATH_AUTO 0u        /* pick by shape */
#define WB200_PATH_TILE_1CTA 1u   /* 128 x BN tiles, one CTA each */
#define WB200_PATH_TILE_2CTA 2u   /* 256 x BN tiles on CTA pairs (cta_group::2) */
#define WB200_PATH_SKINNY 3u      /* M <= 128: swapped operands, stream-K, needs a workspace */
#define WB200_PATH_TILE_SPLITK 4u /* M > 128 with few output tiles and a long K: K slices x tiles in one launch, f32
                                     partial products in the workspace, added in slice order; needs a workspace */
#define WB200_PATH_MASK 0xFu
#define WB200_TILE_N128 0x10u     /* force BN = 128 (default 256 for the tile paths) */
#define WB200_TILE_N192 0x40u     /* force BN = 192: both accumulators fit tensor memory without sharing columns */
#define WB200_ACCUMULATE 0x20u    /* c += a * b^T: the split-K templates' contract, which adds into a
                                     caller-initialised c (tagged_mxfp4_gemm.py:780-781, 830-831) */

#define WB200_OVERLAP_PREVIOUS 0x80u /* the caller asserts that b and b_scale_packed are NOT written by the kernel that
                                     precedes this call in the stream: the GEMM is then launched as a programmatic
                                     dependent of that kernel. On the skinny path (M <= 128) its set-up AND the first
                                     ring of weight loads overlap that kernel's tail; on the tile paths only the set-up
                                     (barriers, tensor-memory allocation, descriptor prefetch) does, and every load
                                     waits for the preceding kernel. Everything else (a, scales of a, c, workspace) is
                                     touched only after the preceding kernel has completed. Back-to-back GEMMs of a
                                     decode loop overlap their tails and heads this way. */
/* Tile order of the tile paths: output tiles are visited in groups of g N tiles (256 columns each, 128 / 192 with the
 * narrower tiles), each group swept down M with N fastest, so that the CTAs running at one time share few b tiles
 * and all of a group's a tiles in L2. This is the templates' `reorder_workgroups` / `group_size_n` pair
 * (tagged_mxfp4_gemm.py:38-60 and its _reorder_mxfp4_workgroups). g = 1..254 in bits 8..15; 0 keeps the default
 * (16); WB200_GROUP_N_ALL puts every N tile in one group, which is the plain row-major order the templates use
 * with reorder_workgroups = False. The result does not depend on the order. */
#define WB200_GROUP_N_SHIFT 8
#define WB200_GROUP_N_MASK 0xFF00u
#define WB200_GROUP_N(g) (((unsigned)(g) << WB200_GROUP_N_SHIFT) & WB200_GROUP_N_MASK)
#define WB200_GROUP_N_ALL WB200_GROUP_N(255)
/* The weight scales (b_scale_packed) were packed per tile of h weight rows by wb200_repack_scales_tiled instead of per
 * 128-row block: h / 8 in bits 16..20 (h = 8 .. 128 in steps of 8; 0 or 128 = the usual packing). Heights up to 128 are read by
 * the M <= 128 kernel only (WB200_PATH_AUTO with a workspace, or WB200_PATH_SKINNY); h is wb200_decode_tile_rows(N). */
/* h = 224 is the one height above 128: it selects the CTA-pair tile kernel with 224-column tiles (M > 128, WB200_PATH_AUTO
 * or WB200_PATH_TILE_2CTA), whose two accumulators sit side by side in tensor memory; its scales are packed two atom rows
 * per 224-row tile. Same results as the 256-wide tiles; measured no faster, kept as an option. */
#define WB200_B_TILE_ROWS_SHIFT 16
#define WB200_B_TILE_ROWS_MASK 0x1F0000u
#define WB200_B_TILE_ROWS(h) ((((unsigned)(h) / 8u) << WB200_B_TILE_ROWS_SHIFT) & WB200_B_TILE_ROWS_MASK)

/* Library version (major * 1000 + minor). */
int wb200_version(void);

/* Message of the last failure on this thread ("" when none). Replaces the std::runtime_error
 * text of HIP_CHECK_EXC in wave_lang/kernel/wave/runtime/runtime.cpp:96-109. */
const char* wb200_last_error(void);

/* Reads and clears the device status word of the current device after synchronising `stream`.
 * Returns WB200_OK or WB200_ERR_DEVICE_TIMEOUT; *detail (may be NULL) receives the raw word
 * (low byte: which wait gave up; upper bits: block index). */
int wb200_check_device_status(void* stream, int* detail);

/* Self-test of the bounded device-side waits: launches one tiny kernel that waits, for at most
 * limit_cycles SM cycles (<= 2e8, about 0.1 s), on a barrier nothing signals. The wait gives up, the kernel
 * ends normally, and the next wb200_check_device_status reports WB200_ERR_DEVICE_TIMEOUT with detail code 7.
 * The reference has no device-side waits to bound (its errors are host exceptions, runtime.cpp:96-109). */
int wb200_selftest_wait_timeout(long long limit_cycles, void* stream);

/* Debug-checked build. The reference's `use_bound_check` compile option guards memory accesses with bounds checks that
 * print and halt (wave_lang/kernel/wave/analysis/generate_bound_checks.py:17-63). Here a second build of this library
 * (compiled with -DWB200_CHECKS) tests an index predicate in front of every copy-engine issue and every global store of
 * the GEMM kernels: innermost TMA coordinate and shared-memory alignment, output row / column inside c, workspace
 * counter index. A failed predicate skips the access and is recorded; nothing traps. wb200_debug_checks synchronises
 * the current device and returns record[0] = code | CTA << 32 of the first failure (0: none), record[1] = its detail
 * word (the offending index), record[2] = number of failures since the last reset; reset != 0 clears the record.
 * wb200_debug_checks_selftest launches one thread that fails a predicate by construction (code 99, detail 1) and skips
 * the store behind it. Both return WB200_ERR_UNSUPPORTED from a library built without the flag. */
int wb200_debug_checks(unsigned long long* record, int reset);
int wb200_debug_checks_selftest(void* stream);

/* Bytes of the packed scale array for a [rows, K/32] scale matrix. */
size_t wb200_packed_scale_bytes(int rows, int K);

/* Weight-scale packing for the decode (M <= 128) kernel. That kernel deals whole tiles of weight rows to one CTA per
 * SM; with the usual 128-row tiles the last round is partly empty whenever ceil(N / 128) is not a multiple of the SM
 * count (N = 28672 on 148 SMs: 224 tiles, the second round runs on 76 SMs, each bounded by what one SM's ring can
 * stream). wb200_decode_tile_rows(N) returns the tile height h <= 128 (a multiple of 8) for which every SM of the
 * current device gets the same number of tiles, 128 when the usual packing is as good. A weight whose scales are
 * packed with wb200_repack_scales_tiled(.., h, ..) (one 512-byte atom row per tile: rows [t h, t h + h) of the
 * weight in atom rows 0 .. h - 1, padding byte above; wb200_packed_scale_bytes_tiled bytes) is then passed with
 * WB200_B_TILE_ROWS(h) in flags. Weights are packed once, so this costs nothing per call; the packing depends on N
 * and on the device's SM count, and the tile paths (M > 128) do not read it: a weight used at both ends of the M
 * range keeps both packings. The reference prepares its weight scales per kernel variant in the same way
 * (e8m0_shuffle for the preshuffle templates, wave_lang/kernel/wave/utils/mxfp_utils.py:113-128). */
int wb200_decode_tile_rows(int N);
size_t wb200_packed_scale_bytes_tiled(int rows, int K, int tile_rows);
int wb200_repack_scales_tiled(const void* scales, long long row_stride, int rows, int K, int tile_rows, void* packed,
                              void* stream);

/* Row-major E8M0 scales -> packed layout. Replaces the host-side scale preshuffle
 * e8m0_shuffle (wave_lang/kernel/wave/utils/mxfp_utils.py:113-128) of the reference's
 * preshuffled templates. src_row_stride in bytes (K/32 when contiguous). */
int wb200_repack_scales(const void* src, long long src_row_stride, int rows, int K, void* dst,
                        void* stream);

/* One scale per ROW (src [rows], element pitch src_row_stride bytes, 1 when contiguous), used for every K
 * block of that row: the a_scale [M] argument of the reference's broadcast-scale kernel
 * get_broadcasted_scale_gemm_mxfp4 (wave_lang/kernel/wave/templates/test_kernels.py:75-140), which
 * broadcasts it to [M, K/32] before the scaled MMA (:112-113). Output as wb200_repack_scales. */
int wb200_repack_scales_broadcast(const void* src, long long src_row_stride, int rows, int K, void* dst,
                                  void* stream);

/* Grouped form for the per-expert GEMM: rows [row_offsets[g], row_offsets[g+1]) of src are group g;
 * its packed scales start at 128-row block row_block_offsets[g] of dst (each group on a block boundary,
 * row_block_offsets[g+1] - row_block_offsets[g] >= ceil(rows of g / 128)); one launch for up to 32
 * groups. Offsets are HOST arrays. dst must hold row_block_offsets[num_groups] * wb200_packed_scale_bytes(128, K). */
int wb200_repack_scales_grouped(const void* src, long long src_row_stride, int num_groups, const int* row_offsets,
                                const int* row_block_offsets, int K, void* dst, void* stream);

/* Activation quantiser: x [rows, K] (f32 when x_dtype == WB200_F32, bf16 when WB200_BF16, row pitch ldx
 * elements, 16-byte aligned rows) -> packed E2M1 codes q [rows, K/2] and E8M0 scales, written row-major
 * (scale_rowmajor [rows, K/32], may be NULL) and/or in the packed layout the GEMM reads (scale_packed,
 * wb200_packed_scale_bytes(rows, K) bytes, may be NULL; padding bytes are filled too). Per 32-element
 * block: scale exponent floor(log2(amax)) - 2, values rounded to the nearest E2M1 value, ties to the even
 * code. The reference names this step as its direction ("fused dynamic quantization",
 * wave_lang/kernel/wave/templates/test_kernels.py:74) but ships no quantiser; its tests feed random
 * codes (wave_lang/kernel/wave/utils/mxfp_utils.py:20-57). */
int wb200_quantize_mxfp4(const void* x, int x_dtype, long long ldx, int rows, int K, void* q, void* scale_rowmajor,
                         void* scale_packed, void* stream);

/* Grouped GEMM driven by DEVICE routing arrays, for rows laid out by wb200_moe_align_block_size with
 * block_size = 256: a [max_rows, K/2] holds the routed rows of all experts, every expert padded to whole
 * 256-row blocks; expert_ids[i] (device) is the expert of block i; *num_rows (device) the padded total, row
 * blocks at or past it are skipped. a_scale_packed: the scales of all max_rows rows packed by wb200_repack_scales
 * (every expert starts on a block boundary, so one packing serves). c [max_rows, N]. Nothing about the routing
 * is read on the host: no synchronisation, and the call can be captured in a CUDA graph. max_rows: a multiple of
 * 256 (the buffers' capacity). Up to 32 experts. */
int wb200_mxfp4_moe_gemm(int num_experts, int max_rows, const int* expert_ids, const int* num_rows, int N, int K, const void* a,
                         const void* a_scale_packed, const void* const* b_ptrs, const void* const* b_scale_ptrs, void* c,
                         int c_dtype, long long ldc, void* stream);

/* ---- mixture-of-experts steps either side of wb200_mxfp4_grouped_gemm ------------------------- */

/* Sort routed (token, slot) pairs by expert and pad every expert to whole blocks: the outputs of the
 * reference's moe_align_block_size_pytorch (tests/kernel/moe/torch_kernels.py:10-97). topk_ids: DEVICE
 * array [num_ids] of expert ids in flat (token-major) order, int32 or int64. sorted_ids [sorted_capacity]:
 * flat indices grouped by expert, ascending inside an expert, each expert's run padded with the value
 * num_ids to a multiple of block_size, the unused rest filled with num_ids too. expert_ids: expert of every
 * block_size-row block. num_tokens_post_pad [1]: padded total. inverse [num_ids] (may be NULL, not in the
 * reference): position of flat index i in sorted_ids. Capacities must cover the worst case
 * num_ids + num_experts * (block_size - 1) entries (:116-119 of the reference's test). At most 256 experts. */
int wb200_moe_align_block_size(const void* topk_ids, int ids_are_int64, int num_ids, int num_experts, int block_size,
                               int* sorted_ids, int sorted_capacity, int* expert_ids, int expert_ids_capacity,
                               int* num_tokens_post_pad, int* inverse, void* stream);

/* dst[p, :] = src[sorted_ids[p] / top_k, :] when sorted_ids[p] < num_ids, else zeros: brings the packed
 * codes (or scales) of each routed token to its sorted row. Byte rows of row_bytes; 16-byte accesses when
 * bases, pitches and row_bytes are multiples of 16. */
int wb200_moe_gather_rows(const void* src, long long src_pitch, int row_bytes, const int* sorted_ids, int num_rows,
                          int num_ids, int top_k, void* dst, long long dst_pitch, void* stream);

/* out = x1 / (1 + exp(-x1)) * x2 elementwise on [rows, n] matrices of f32 or bf16 (pitches in elements):
 * get_silu_and_mul_kernel (wave_lang/kernel/wave/templates/moe.py:89-145). out may be NULL when q is
 * given: q [rows, n/2] and the scale outputs (as wb200_quantize_mxfp4) receive the f32 result quantised
 * to MXFP4 in the same pass, ready for the down-projection GEMM. num_rows (may be NULL): DEVICE value, rows at or
 * past it are skipped (the padded row count of a routed batch whose buffers have the worst-case size). */
int wb200_silu_and_mul(const void* x1, const void* x2, long long ld1, long long ld2, int dtype, int rows, int n, void* out,
                       long long ldo, void* q, void* scale_rowmajor, void* scale_packed, const int* num_rows, void* stream);

/* Quantise routed tokens straight to their expert-sorted rows: row t of x [tokens, K] (f32 or bf16) is quantised
 * once (as wb200_quantize_mxfp4) and its codes and row-major scales are written to the rows dst_rows[t * top_k + j]
 * of q / scale_rowmajor for j < top_k (DEVICE array, the `inverse` output of wb200_moe_align_block_size; negative
 * entries are skipped). Rows of q that no token maps to are not written. Replaces quantise + wb200_moe_gather_rows. */
int wb200_moe_quantize_scatter(const void* x, int x_dtype, long long ldx, int tokens, int K, int top_k, const int* dst_rows,
                               void* q, void* scale_rowmajor, void* stream);

/* out[t, :] = sum over j < top_k of weight[t * top_k + j] * y[row_of[t * top_k + j], :], f32 accumulation in
 * slot order, pairs with row_of < 0 skipped: the weighted sum that ends the reference's MoE
 * (tests/kernel/moe_test.py:123-127). y, out: f32 or bf16. */
int wb200_moe_combine(const void* y, long long ldy, int dtype, const int* row_of, const float* weight, int tokens, int top_k,
                      int cols, void* out, long long ldo, void* stream);

/* Test aid: out[r, k] = E2M1(q) * 2^(scale - 127) as f32, the dequantised operand of
 * mxfp4_to_f32 / e8m0_to_f32 (wave_lang/kernel/wave/utils/mxfp_utils.py:60-95). */
int wb200_mxfp4_dequant(const void* q, const void* scale, int rows, int K, float* out, void* stream);

/* Workspace the GEMM may use for this shape (0 when none). The skinny path (M <= 128) needs one:
 * f32 partial tiles plus per-tile counters. The split-K tile path (M > 128, so few 256 x 256 output
 * tiles that they fill less than half of the CTA pairs, K >= 2048) is taken by WB200_PATH_AUTO only
 * when a workspace of this size is passed: one f32 [M, N] slot per K slice. The first
 * wb200_workspace_init'ed bytes hold the counters; a workspace must be initialised once before its
 * first use and is left clean by every successful call. */
size_t wb200_mxfp4_gemm_workspace_bytes(int M, int N, int K);
int wb200_workspace_init(void* workspace, size_t bytes, void* stream);

/* c = dequant(a, a_scale) * dequant(b, b_scale)^T, scales in packed layout.
 * Replaces the launch of the kernel built from get_scaled_gemm_kernel / get_tagged_mxfp4_gemm
 * (wave_lang/kernel/wave/templates/gemm.py:134-205, tagged_mxfp4_gemm.py:38-145) through
 * wave_runtime.launch (runtime.cpp:123-203). Asynchronous on `stream`. */
int wb200_mxfp4_gemm(int M, int N, int K, const void* a, const void* a_scale_packed, const void* b,
                     const void* b_scale_packed, void* c, int c_dtype, long long ldc, void* workspace,
                     size_t workspace_bytes, unsigned flags, void* stream);

/* The per-call sequence of the reference-facing launch in one call: repack the ROW-MAJOR activation
 * scales a_scale [M, K/32] (row pitch a_scale_stride bytes) into a_scale_scratch (at least
 * wb200_packed_scale_bytes(M, K) bytes, caller-owned), then run wb200_mxfp4_gemm with it. Weight
 * scales arrive packed, because a weight's scales are packed once and reused. Saves one trip
 * through the caller's binding per GEMM; same kernels, same results. */
int wb200_mxfp4_gemm_repack_a(int M, int N, int K, const void* a, const void* a_scale, long long a_scale_stride,
                              void* a_scale_scratch, const void* b, const void* b_scale_packed, void* c, int c_dtype,
                              long long ldc, void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/* MXFP8: the same block-scaled GEMM with 8-bit operands, a [M, K] and b [N, K] bytes of E5M2
 * (elem_format WB200_E5M2, what the reference's testScaledGemmMXFP8 feeds,
 * tests/kernel/wave_gemm_mxfp_test.py:64-77, 416-501) or E4M3 (WB200_E4M3), one E8M0 scale per 32
 * elements, scales packed by wb200_repack_scales exactly as for MXFP4. flags may hold WB200_PATH_AUTO /
 * TILE_1CTA / TILE_2CTA / SKINNY, WB200_TILE_N128, WB200_ACCUMULATE and WB200_OVERLAP_PREVIOUS; the skinny path (M <= 128, chosen by
 * AUTO when a workspace is passed) takes the workspace of wb200_mxfp4_gemm_workspace_bytes(M, N, K). */
#define WB200_E4M3 0
#define WB200_E5M2 1
/* Mixed operand pair: or WB200_B_FP4 into elem_format and pass b as packed E2M1, [N, K/2] bytes (the MXFP4 weight
 * layout), with its E8M0 block scales as usual: a stays 8-bit (E4M3 or E5M2). The MMA is kind::mxf8f6f4 with the two
 * operand formats set independently; the copy engine expands the 4-bit values into the instruction's 8-bit container
 * layout on their way into shared memory, so the weights cross HBM at 4 bits each. K must be a multiple of 128 and b
 * 32-byte aligned. The reference reaches this pair through the same scaled MMA with different bitcasts of its i8
 * operands (F32_16x16x128_F8F6F4, wave_lang/kernel/wave/constraints.py:79-86); it has no test of it. */
#define WB200_B_FP4 0x10
int wb200_mxfp8_gemm(int M, int N, int K, const void* a, const void* a_scale_packed, const void* b,
                     const void* b_scale_packed, void* c, int c_dtype, long long ldc, int elem_format, void* workspace,
                     size_t workspace_bytes, unsigned flags, void* stream);

/* MXFP8 activation quantiser: as wb200_quantize_mxfp4 with one byte per element (q [rows, K]) of elem_format;
 * block scale exponent floor(log2(amax)) - 8 (E4M3, largest value 448) or - 15 (E5M2, 57344); values rounded to
 * nearest even and saturated by the conversion. Not in the reference (its MXFP8 test feeds random values). */
int wb200_quantize_mxfp8(const void* x, int x_dtype, long long ldx, int rows, int K, int elem_format, void* q,
                         void* scale_rowmajor, void* scale_packed, void* stream);

/* Allocation-free variant of the skinny (M <= 16) GEMM. No counterpart in the reference.
 *
 * For callers that may not allocate device memory at the point of the call and have no spare buffer
 * to lend as a workspace: a host that gave all device memory to its own arena at start-up and
 * forbids later cudaMalloc calls (an inference server with a fixed memory plan), a latency-critical
 * decode loop where the implicit synchronisation of cudaMalloc / cudaFree is not acceptable, or a
 * plug-in boundary that hands over tensors only. The stream-K partial tiles and tile counters that
 * wb200_mxfp4_gemm takes from the caller's workspace live here in a fixed array inside the library
 * image (about 2.5 MiB per GPU that loads the library, held until the process exits).
 *
 * Limits: M <= 16, N <= 65536, at most 160 SMs; larger problems are rejected with
 * WB200_ERR_UNSUPPORTED and a message. flags: 0 or WB200_ACCUMULATE. a, b, packed scales and c are
 * passed exactly as to wb200_mxfp4_gemm; results are bit-identical to its WB200_PATH_SKINNY path.
 *
 * The first call on each device looks up the array's device address (and does the library's
 * one-time device set-up); make that call before starting any stream capture. The call itself
 * calls no cudaMalloc, cudaFree or other allocating routine. All calls on a device share the one
 * array (the tile counters are cleared on the stream at the start of every call): two calls
 * whose kernels can overlap on the GPU - different streams without an ordering between them -
 * race on it and produce wrong results; serialise them. */
int wb200_mxfp4_gemm_skinny_noalloc(int M, int N, int K, const void* a, const void* a_scale_packed, const void* b,
                                    const void* b_scale_packed, void* c, int c_dtype, long long ldc, unsigned flags,
                                    void* stream);

/* Grouped (per-expert) GEMM: group g computes c[row_offsets[g] : row_offsets[g+1], :] =
 * a[rows of g] * b_g^T with its own weight matrix b_ptrs[g] ([N, K/2]) and packed scales
 * b_scale_ptrs[g]. a is the gathered activation matrix [total_rows, K/2]; a_scale_packed is
 * packed per group: group g's scales start at 128-row block row_block_offsets[g]. The pointer
 * and offset arrays live in HOST memory. The reference has no grouped MXFP4 kernel; its MoE
 * path loops a GEMM per expert from Python (tests/kernel/moe_test.py:183-240). */
int wb200_mxfp4_grouped_gemm(int num_groups, const int* row_offsets, const int* row_block_offsets,
                             int N, int K, const void* a, const void* a_scale_packed,
                             const void* const* b_ptrs, const void* const* b_scale_ptrs, void* c,
                             int c_dtype, long long ldc, void* stream);

/* ---- K-sharded multi-GPU GEMM: compute step with its output scattered by rows ------------------- */

/* c_p = a[row_offsets[p] : row_offsets[p+1], :] * b^T for every part p, part p written to the matrix at
 * c_ptrs[p] ([rows of p, N], pitch ldc, 16-byte aligned), in ONE persistent launch whose tiles are stored
 * as they finish. The output matrices may be another GPU's memory mapped into this process (CUDA IPC /
 * peer access): a rank of a K-sharded GEMM deposits its partial products for rows owned by rank p directly
 * in p's receive buffer over NVLink while the remaining tiles are still being computed. Parts start at
 * multiples of 128 rows (HOST arrays; up to 32 parts). The reference distributes GEMMs by M / N tiles only
 * (wave_lang/kernel/wave/templates/dist_gemm.py:49-50); it has no K-sharded form. */
#define WB200_SCATTER_TMA_STORE 1u /* write the outputs with TMA stores instead of ordinary 16-byte stores */
int wb200_mxfp4_gemm_scatter_rows(int num_parts, const int* row_offsets, int N, int K, const void* a,
                                  const void* a_scale_packed, const void* b, const void* b_scale_packed, void* const* c_ptrs,
                                  int c_dtype, long long ldc, unsigned flags, void* stream);

/* Receive buffers of the K-sharded GEMM, shared between the processes of one node with CUDA IPC.
 * create: cudaMalloc + zero fill on the current device, returns the pointer and a 64-byte handle to send to
 * the other processes; open: maps another process's buffer for the CURRENT device (the device whose kernels
 * will write to it; peer access to the owner is enabled as needed); close / destroy undo open / create. */
int wb200_peer_buffer_create(size_t bytes, void** ptr, void* handle64);
int wb200_peer_buffer_open(const void* handle64, void** ptr);
int wb200_peer_buffer_close(void* ptr);
int wb200_peer_buffer_destroy(void* ptr);

/* rows x width_bytes from src (row pitch src_pitch bytes) to dst (row pitch dst_pitch), asynchronous on `stream`, by the
 * copy engines. Either side may be another GPU's memory (a wb200_peer_buffer_open mapping, or peer access): this is how
 * a rank of the N-sharded GEMM deposits its column block of C in every other rank's [M, N] matrix, in place, with no
 * collective library and no interleaving pass afterwards. The reference merges per-device output slices into the
 * result on the host side of its wrapper (wave_lang/kernel/compiler/host_utils.py:330-376). */
int wb200_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows, void* stream);

/* out[i] = slots[0][i] + slots[1][i] + ... (f32, slot order, i < count; slot s starts at slots + s * slot_stride),
 * rounded once to out_dtype: the reduction over the ranks' partial products. */
int wb200_sum_slots(const float* slots, int num_slots, long long slot_stride, long long count, void* out, int out_dtype,
                    void* stream);

/* ---- N-sharded GEMM over the GPUs of one node, driven by ONE process --------------------------------
 *
 * Replaces the reference's multi-device launch: `DeviceConstraint` tiles M / N over devices
 * (wave_lang/kernel/wave/constraints.py:1105-1180), the host wrapper slices the inputs per device,
 * dispatches one kernel per device and merges the output slices (wave_lang/kernel/compiler/host_utils.py:158-376),
 * and `MultiDeviceLaunchable` owns one device object per GPU and invokes once
 * (wave_lang/runtime/multi_device_launch.py:38-273). Here device g owns the rows [n_bounds[g], n_bounds[g+1]) of b
 * (a column block of C) and keeps them resident; a is copied to every device; every device runs one GEMM on its
 * own stream; the column blocks are laid side by side wherever the whole C is wanted. No collective library is
 * involved and no kernel reads another GPU's memory: the GPUs exchange data through copy-engine copies only.
 * All memory is the caller's: the handle owns streams and events, nothing else. */
typedef struct wb200_multi_gpu wb200_multi_gpu_t;

typedef struct {
  void* a;                    /* [M, K/2] on this device: filled by wb200_multi_gpu_broadcast_a */
  void* a_scale;              /* [M, K/32] row-major on this device: filled by wb200_multi_gpu_broadcast_a */
  void* a_scale_packed;       /* wb200_packed_scale_bytes(M, K) on this device: written by wb200_multi_gpu_gemm */
  const void* b;              /* this device's rows of b, [n_g, K/2] */
  const void* b_scale_packed; /* their scales, packed once by the caller (wb200_repack_scales on this device) */
  void* c;                    /* [M, n_g] on this device, row pitch ldc elements */
  long long ldc;
  void* workspace;            /* wb200_mxfp4_gemm_workspace_bytes(M, n_g, K) on this device, initialised; may be null when 0 */
  size_t workspace_bytes;
} wb200_device_operands;

/* One stream per listed device; peer access is enabled between every pair that supports it. */
int wb200_multi_gpu_create(int num_devices, const int* device_ids, wb200_multi_gpu_t** out);
int wb200_multi_gpu_destroy(wb200_multi_gpu_t* h);
int wb200_multi_gpu_num_devices(const wb200_multi_gpu_t* h);
/* Rows of b owned by device `index` of `num_devices` (multiples of `granule`, 128 = the scale-factor atom height). Host only. */
int wb200_multi_gpu_shard_bounds(int N, int num_devices, int index, int granule, int* n0, int* n1);
/* Every device stream waits for the work queued so far on `stream` of device `device` (the producer of a): the
 * reference's launch is ordered after the caller's stream in the same way (run_utils.py:87). */
int wb200_multi_gpu_wait_for(wb200_multi_gpu_t* h, int device, void* stream);
/* Copy a [M, K/2] and a_scale [M, K/32] (contiguous; on device src_device, or in pinned host memory when
 * src_device < 0) into ops[g].a / ops[g].a_scale of every device, on the devices' streams. */
int wb200_multi_gpu_broadcast_a(wb200_multi_gpu_t* h, int M, int K, const void* a, const void* a_scale, int src_device,
                                const wb200_device_operands* ops);
/* On every device g: pack ops[g].a_scale, then c_g = a * b_g^T (wb200_mxfp4_gemm_repack_a), on the device's stream.
 * n_bounds: num_devices + 1 row offsets of the shards; a device with an empty shard is skipped. */
int wb200_multi_gpu_gemm(wb200_multi_gpu_t* h, int M, int K, const int* n_bounds, const wb200_device_operands* ops,
                         int c_dtype, unsigned flags);
/* Lay the column blocks side by side: for every destination j (a matrix [M, N] with row pitch dst_ld elements on
 * device dst_devices[j], or in pinned host memory when dst_devices[j] < 0), device g copies its block into columns
 * [n_bounds[g], n_bounds[g+1]) on its own stream, after its GEMM (2-D copy-engine copies; one per device and destination). */
int wb200_multi_gpu_gather_c(wb200_multi_gpu_t* h, int M, const int* n_bounds, const wb200_device_operands* ops, int c_dtype,
                             int num_dst, void* const* dst_ptrs, const int* dst_devices, long long dst_ld);
/* `stream` of device `device` waits for everything queued on the devices' streams; the host does not block. */
int wb200_multi_gpu_join(wb200_multi_gpu_t* h, int device, void* stream);
/* Host waits for every device stream; returns the first device-side status that is not clean. */
int wb200_multi_gpu_synchronize(wb200_multi_gpu_t* h);
/* Timing brackets on every device stream: end() synchronises and returns the largest elapsed time over the devices. */
int wb200_multi_gpu_time_begin(wb200_multi_gpu_t* h);
int wb200_multi_gpu_time_end(wb200_multi_gpu_t* h, float* max_ms);

#ifdef __cplusplus
}
#endif
#endif /* WAVE_B200_H_ */
