/*
 * lct_b200.h - C ABI of the B200 (sm_100a) BF16 lossless codec library.
 *
 * One entry point per kernel launch wrapper of the reference's
 * LCT/kernels/dispatch.py (the layer its host pipelines call), plus the
 * allocator launches of LCT/tensor_buffer.py.  Each declaration cites the
 * reference interface it replaces.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless said otherwise; sizes are in
 *     elements of the pointed-to type unless the name says bytes;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream).  All work is enqueued on it; no entry point synchronises,
 *     allocates or frees device memory;
 *   - return value: 0 on success, a positive cudaError_t if a launch failed,
 *     or one of the negative LCT_E_* codes for a rejected argument.  Device
 *     side conditions (arena exhausted, stale descriptor, ...) are reported
 *     through the status words documented below, never by trapping;
 *   - payload, side-byte, output and dense-operand buffers handed to the
 *     vectorised kernels must be 16-byte aligned except where noted.
 *
 * Format recap (identical to the reference's):
 *   BF16 bits v: exponent byte (v >> 7) & 0xFF, side byte (v & 0x7F) | ((v >> 8) & 0x80).
 *   A tensor is cut into blocks of `block_symbols` elements = `steps` rows of
 *   256 lanes.  Lane l at row n = block*steps + step holds logical element
 *   n*256 + (l ^ (n & 254)).  Stream s = block*256 + l owns `fixed_words`
 *   32-bit words, word w at encoded[w*streams + s], filled LSB first.
 */
#ifndef LCT_B200_H
#define LCT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LCT_E_BAD_GEOMETRY (-1)  /* steps/block_symbols/fixed_words not a supported layout */
#define LCT_E_NULL_POINTER (-2)
#define LCT_E_ALIGNMENT (-3)     /* a buffer that must be 16-byte aligned is not */
#define LCT_E_BAD_ARGUMENT (-4)
#define LCT_E_TOO_LARGE (-5)
#define LCT_E_SCRATCH_LIMIT (-6) /* tensor too large for the built-in scratch of lct_encode_noalloc */

/* Overflow ("fallback") storage of one compressed tensor, as the decoders see
 * it.  mode 0: the tensor has no overflow streams, the other fields are
 * ignored.  mode 1: private tensors lanes/starts/tail (tail bytes start at
 * tail + base).  mode 2: shared arena; lanes == starts == tail == arena
 * payload, and the region [descriptor[0], +descriptor[1]) holds
 * lanes[count] | starts[count] | tails.  Reference: FallbackStorage,
 * LCT/kernels/backends.py:36-50, and fallback_tail_args, dispatch.py:133-144. */
typedef struct lct_overflow {
  const uint8_t *lanes;
  const uint8_t *starts;
  const uint8_t *tail;
  const int32_t *descriptor; /* int32[4] = offset|-1, aligned size|0, status, generation */
  const int32_t *count;      /* int32[1]: number of overflow streams */
  const int32_t *blocks;     /* int32[3*blocks]: count | first entry | first tail byte */
  int64_t base;
  int32_t mode;
  int32_t reserved;
} lct_overflow;

/* One compressed operand for the decoders and fused operations. */
typedef struct lct_operand {
  const int32_t *encoded;        /* int32[streams*fixed_words + 4] */
  const uint8_t *side;           /* uint8[size] sign+mantissa bytes, storage order */
  const int32_t *shifted_decode; /* int32[1024], built at encode time */
  const int32_t *center;         /* int32[1] */
  const uint32_t *pair_table;    /* uint32[LCT_PAIR_TABLE_WORDS] from lct_build_pair_table for this codebook */
  lct_overflow overflow;
} lct_operand;

/* Library identity: "lct-b200 <version> sm_100a". Host pointer, static storage. */
const char *lct_version(void);
/* Text for a return code of this library (host pointer, static storage). */
const char *lct_error_string(int code);

/* Lane mapping of every later launch of this library in this process: 0 = the
 * default "swizzle" (lane l of global row n holds element n*256 + (l ^ (n & 254))),
 * 1 = "linear" (lane l holds element n*256 + l).  The reference fixes it at
 * import time (LCT/config.py:16-18, LCT/kernels/generic/layout.py:12-42) and asks
 * to keep it fixed while compressed tensors are in use; the same holds here.
 * Not stream-ordered: it is read on the host when a launch is enqueued. */
int lct_set_lane_mapping(int linear);
int lct_get_lane_mapping(void);

/* ---- codebook preparation ------------------------------------------------ */

/* Two-symbol lookup tables over 12 stream bits, derived from a codebook's
 * first-level decode table (int32[1024]): LCT_PAIR_TABLE_WORDS words, one
 * 4096-entry table per possible center (-128..127) with the symbols already
 * stored as exponent bytes, so a decoder CTA copies the 16 KB of its tensor's
 * center and needs no per-tensor table of its own.  Depends only on the
 * Distribution: callers build it once per codebook and device (4 MiB).  No
 * counterpart in the reference (its decoders look up one symbol at a time
 * in the per-tensor shifted table, LCT/kernels/primitives.py:17-36). */
#define LCT_PAIR_TABLE_WORDS (256 * 4096)
int lct_build_pair_table(const int32_t *decode_table, int rare_length, uint32_t *pair_table,
                         void *stream);

/* Sample the exponent center of `src` (int16 BF16 bits, or uint8 exponent
 * bytes when precomputed) and write center[1], shifted_encode[256] and
 * shifted_decode[1024].  Replaces dispatch.estimate_and_shift_encoding_table,
 * LCT/kernels/dispatch.py:33-48 (kernel: common/tables.py:86-99).  src needs
 * only its natural alignment. */
int lct_center_and_tables(const void *src, int64_t logical_numel, int precomputed,
                          const int32_t *encode_table, const int32_t *decode_table,
                          int32_t *center, int32_t *shifted_encode, int32_t *shifted_decode,
                          void *stream);

/* Same tables for a given center.  Either output may be NULL.  Replaces
 * dispatch.shift_encoding_table / shift_decoding_table, dispatch.py:16-30, 51-62. */
int lct_shift_tables(const int32_t *encode_table, const int32_t *decode_table,
                     const int32_t *center, int32_t *shifted_encode, int32_t *shifted_decode,
                     void *stream);

/* ---- encode --------------------------------------------------------------- */

/* Field split + fixed-budget Huffman encode of every block.  Writes
 * side[size] (skipped when precomputed), encoded[streams*fixed_words + 4]
 * (every word, unused ones zero), extra_starts[streams] (first overflow step,
 * 255 = none) and summaries[0 .. 2*blocks) = per-block overflow count and tail
 * bytes.  Replaces dispatch.encode_kernel, dispatch.py:294-316 (kernel:
 * generic/encode.py:10-169).  src may have any alignment. */
int lct_encode(const void *src, uint8_t *side, int32_t *encoded, const int32_t *shifted_encode,
               uint8_t *extra_starts, int32_t *summaries, int64_t size, int64_t logical_numel,
               int block_symbols, int steps, int fixed_words, int precomputed, void *stream);

/* Exclusive scan of the block summaries into summaries[2*blocks .. 4*blocks),
 * totals into counts[0..1] (counts[2..3] = 0) and, when arena_storage is not
 * NULL, a first-fit reservation of tail bytes + 2*count (rounded up to 16) in
 * that arena, reported in descriptor[4].  Replaces dispatch.prefix_allocate,
 * dispatch.py:70-85 (kernel: generic/metadata.py:13-38). */
int lct_scan_allocate(int32_t *summaries, int32_t *counts, int32_t *descriptor,
                      void *arena_storage, int64_t blocks, int max_free_regions, void *stream);

/* Write the compact overflow list (lanes, starts), the raw exponent tails and
 * blocks_out[3*blocks].  descriptor == NULL: private storage (lanes, starts,
 * tail are exact-size tensors).  Otherwise the three pointers are the arena
 * payload and nothing is written unless descriptor[2] == 0.  Replaces
 * dispatch.compact_extra with build_meta=True, dispatch.py:113-130 (kernel:
 * generic/compaction.py:135-190). */
int lct_compact_tails(const void *src, uint8_t *lanes, uint8_t *starts, uint8_t *tail,
                      const int32_t *descriptor, const int32_t *counts, int32_t *blocks_out,
                      const uint8_t *extra_starts, const int32_t *summaries, int64_t size,
                      int64_t logical_numel, int block_symbols, int steps, int precomputed,
                      void *stream);

/* lct_encode followed by the summary scan of lct_scan_allocate (no arena), for
 * callers that cannot allocate device memory: a serving loop that forbids
 * allocation once it has started, a host whose device memory all belongs to
 * another pool, a plain C program with no allocator.  The two work buffers lct_encode takes from its caller
 * (extra_starts, summaries) are replaced by a 272 KiB array inside the library
 * image, one per GPU that loads the library, held until the process exits.
 * The caller passes only the source, the outputs side[size] and
 * encoded[streams*fixed_words + 4], and counts[4], which receives the number of
 * overflow streams and their tail bytes (counts[2..3] = 0).  The result is
 * complete only when counts[0] == 0: then side + encoded are the whole
 * compressed form.  With overflow streams this entry point yields the totals
 * only (the per-lane overflow starts stay in the built-in array, which the ABI
 * does not expose), and the tensor must be encoded again through lct_encode +
 * lct_scan_allocate + lct_compact_tails with caller-provided scratch.
 *   - Limit: at most 1024 codec blocks (64 Mi elements in the 65536-element
 *     layouts, 32 Mi in the 32768-element ones); a larger tensor is rejected
 *     with LCT_E_SCRATCH_LIMIT before anything is launched.
 *   - Calls no cudaMalloc/cudaFree nor any allocating routine.  The first
 *     call on each GPU looks up the array's device address
 *     (cudaGetSymbolAddress, with that GPU current); make that first call
 *     outside any stream capture.
 *   - Every call on a GPU uses the same array.  Nothing in it needs clearing
 *     between calls (each call rewrites all it reads), but two calls that
 *     overlap on the GPU, e.g. on different streams, race on it.
 * Has no counterpart in the reference, whose host code allocates these
 * buffers with torch.empty on every encode. */
int lct_encode_noalloc(const void *src, uint8_t *side, int32_t *encoded,
                       const int32_t *shifted_encode, int32_t *counts, int64_t size,
                       int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                       int precomputed, void *stream);

/* The whole compression of one tensor into a shared arena as ONE call: the
 * launches of lct_center_and_tables, lct_encode, lct_scan_allocate and
 * lct_compact_tails, same arguments, same bytes everywhere.  Replaces the host
 * sequence of LCT/codec/encode.py:62-186 (encode_components, buffered branch)
 * with one crossing of the language boundary, and lets each kernel be
 * scheduled while its predecessor is still running (programmatic stream
 * serialisation): the encoder requests its first source rows while the center
 * is being sampled and waits on the device only before it reads the shifted
 * table.  `arena_storage` is the whole TensorBuffer storage (allocator words
 * first); tails go to its payload region as with lct_compact_tails + a
 * descriptor.  `side` may be NULL when `precomputed`. */
int lct_compress(const void *src, int precomputed, uint8_t *side, int32_t *encoded,
                 const int32_t *encode_table, const int32_t *decode_table, int32_t *center,
                 int32_t *shifted_encode, int32_t *shifted_decode, uint8_t *extra_starts,
                 int32_t *summaries, int32_t *counts, int32_t *descriptor, int32_t *blocks_out,
                 void *arena_storage, int max_free_regions, int64_t size, int64_t logical_numel,
                 int block_symbols, int steps, int fixed_words, void *stream);

/* Many tensors of ONE codebook and geometry compressed by four launches in
 * total (centers, encode, scan + arena reservations in job order, tails),
 * overflow tails in a shared arena.  Equivalent to calling
 * lct_center_and_tables, lct_encode, lct_scan_allocate and lct_compact_tails
 * once per job, in job order, and leaves the same bytes everywhere.  `jobs` is
 * a DEVICE array sorted by first_block.  Work buffers: extra_starts
 * uint8[256 * total_blocks], summaries int32[4 * total_blocks] (job j uses
 * the 4 * blocks_j ints from 4 * first_block), shifted_encode int32[256 * n_jobs].
 * No counterpart in the reference, which encodes one tensor per call. */
typedef struct lct_encode_job {
  const void *src;          /* int16 BF16 bits, any alignment */
  uint8_t *side;            /* uint8[size] */
  int32_t *encoded;         /* int32[streams*fixed_words + 4] */
  int32_t *center;          /* int32[1] */
  int32_t *shifted_decode;  /* int32[1024] */
  int32_t *counts;          /* int32[4] */
  int32_t *descriptor;      /* int32[4] */
  int32_t *blocks_out;      /* int32[3*blocks] */
  int64_t size;
  int64_t logical_numel;
  int64_t first_block;
} lct_encode_job;

int lct_compress_batch(const lct_encode_job *jobs /* device */, int n_jobs, int64_t total_blocks,
                       const int32_t *encode_table, const int32_t *decode_table,
                       void *arena_storage, int max_free_regions, uint8_t *extra_starts,
                       int32_t *summaries, int32_t *shifted_encode, int block_symbols, int steps,
                       int fixed_words, void *stream);

/* ---- decode and fused operations ------------------------------------------ */

/* Decode to int16 BF16 bits out[logical_numel], overflow tails substituted in
 * place.  Replaces dispatch.decode_kernel, dispatch.py:319-361 (kernels:
 * generic/decode.py:259-308). */
int lct_decode(const lct_operand *a /* host pointer */, int16_t *out, int64_t size,
               int64_t logical_numel, int block_symbols, int steps, int fixed_words,
               int rare_length, void *stream);

/* Many compressed tensors of ONE geometry decoded by one launch (weight sets
 * with many small tensors are launch-bound otherwise).  `jobs` is a DEVICE
 * array sorted by first_block; job j owns CTAs [first_block, first_block +
 * size/block_symbols).  Each job's `out` must be 16-byte aligned.  No
 * counterpart in the reference, which decodes one tensor per launch. */
typedef struct lct_decode_job {
  lct_operand operand;
  int16_t *out;          /* int16[logical_numel] */
  int64_t size;          /* padded element count */
  int64_t logical_numel;
  int64_t first_block;   /* sum of the earlier jobs' block counts */
  uint8_t *side_stage;   /* NULL, or uint8[size] scratch in THIS GPU's memory (16-byte aligned):
                            every CTA first copies its block's side bytes there with 16-byte
                            accesses and decodes from the copy.  For operands that live in a
                            peer GPU's memory: the decoder's own side-byte loads are 32 bytes
                            per warp and row, which uses NVLink at half the rate of full lines. */
} lct_decode_job;

int lct_decode_batch(const lct_decode_job *jobs /* device */, int n_jobs, int64_t total_blocks,
                     int block_symbols, int steps, int fixed_words, int rare_length,
                     void *stream);

#define LCT_OP_ADD 0            /* bf16(a + b)            generic/pointwise.py:340-343 */
#define LCT_OP_MULTIPLY 1       /* bf16(a * b)            generic/pointwise.py:346-349 */
#define LCT_OP_SCALAR_MUL_ADD 2 /* bf16(fma-ordered alpha*a + beta*b), pointwise.py:352-363 */
/* Two operations of the reference's optimizers on their BF16 state, with the
 * float32 arithmetic of the PyTorch CUDA kernels the reference calls there
 * (LCT/components/sparse_utils.py:88,193 momentum.lerp_(grad, w) and :194
 * square_avg.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)):
 *   LERP        w = *alpha; d = b - a;
 *               |w| < 0.5 ? bf16(fma(w, d, a)) : bf16(fma(-d, 1 - w, b))
 *   EMA_SQUARE  t = bf16(a * *alpha); bf16(fma(*beta, b * b, t))
 * alpha (and, for EMA_SQUARE, beta) must not be NULL; the *_is_one flags are
 * ignored. */
#define LCT_OP_LERP 3
#define LCT_OP_EMA_SQUARE 4

/* compA (op) B with B dense BF16 in logical order.  compressed_output == 0:
 * output = BF16[logical_numel].  Otherwise output = side bytes uint8[size]
 * (storage order) and auxiliary = exponent bytes uint8[size] (logical order,
 * padding untouched), ready for lct_encode(precomputed=1).  alpha/beta are
 * device float32 scalars, read only when the matching *_is_one flag is 0.
 * Overflow rows are computed in the same launch.  Replaces
 * dispatch.pointwise_dense + dispatch.pointwise_fallback, dispatch.py:168-212
 * (kernels: generic/pointwise.py:84-337).  `other` may have any alignment. */
int lct_pointwise(const lct_operand *a /* host pointer */, const void *other, void *output,
                  uint8_t *auxiliary, const float *alpha, const float *beta, int op,
                  int alpha_is_one, int beta_is_one, int compressed_output, int64_t size,
                  int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                  int rare_length, void *stream);

/* alpha * compA + compB, both compressed with the same geometry.  Outputs as
 * lct_pointwise.  Replaces dispatch.dual_maps_init, dual_tables_and_maps and
 * dual_mapped, dispatch.py:215-286 (kernels: generic/pointwise_scalar_dual.py). */
int lct_dual_scale_add(const lct_operand *a, const lct_operand *b /* host pointers */,
                       void *output, uint8_t *auxiliary, const float *alpha,
                       int compressed_output, int64_t size, int64_t logical_numel,
                       int block_symbols, int steps, int fixed_words, int rare_length,
                       void *stream);

/* Fused update of compressed state, compA <- compA (op) B, without the split
 * intermediate the reference writes between its pointwise kernel and its
 * encoder (LCT/codec/pointwise.py:263-278).  Two launches plus the usual
 * center / scan / tail launches:
 *   lct_update_sample   result exponent bytes at the (up to) 4096 positions the
 *                       center estimate samples (common/tables.py:24-28) into
 *                       samples[min(logical_numel, 4096)]; feed them to
 *                       lct_center_and_tables(samples, count, precomputed=1, ...)
 *                       to get the new center and shifted tables;
 *   lct_update_fused    decode A, apply op against dense B, re-encode with
 *                       shifted_encode: writes side_out[size], encoded_out,
 *                       extra_starts and summaries exactly as lct_encode does,
 *                       and for lanes that overflow their budget the raw result
 *                       exponents (from the overflow step on) into
 *                       spill[logical offset], uint8[size], which is then the
 *                       `src` of lct_compact_tails(precomputed=1).
 * Results are bit-identical to lct_pointwise(compressed_output=1) followed by
 * lct_center_and_tables / lct_encode(precomputed=1).
 * Optional sample-value cache: result_values (uint16[min(logical_numel, 4096)],
 * may be NULL) receives the BF16 bits of the RESULT at the sample positions;
 * handed back as known_values (may be NULL) when that result is the A of the
 * next update, they replace the walk over A's bit streams. */
int lct_update_sample(const lct_operand *a /* host pointer */, const void *other,
                      const float *alpha, const float *beta, int op, int alpha_is_one,
                      int beta_is_one, uint8_t *samples, const uint16_t *known_values,
                      uint16_t *result_values, int64_t size, int64_t logical_numel,
                      int block_symbols, int steps, int fixed_words, int rare_length,
                      void *stream);
int lct_update_fused(const lct_operand *a /* host pointer */, const void *other,
                     const float *alpha, const float *beta, int op, int alpha_is_one,
                     int beta_is_one, const int32_t *shifted_encode, uint8_t *side_out,
                     int32_t *encoded_out, uint8_t *extra_starts, int32_t *summaries,
                     uint8_t *spill, int64_t size, int64_t logical_numel, int block_symbols,
                     int steps, int fixed_words, int rare_length, void *stream);

/* The whole update into a shared arena as ONE call: lct_update_sample,
 * lct_center_and_tables(samples, precomputed=1), lct_update_fused,
 * lct_scan_allocate and lct_compact_tails(src=spill, precomputed=1), same
 * arguments, same bytes; the later kernels are scheduled while their
 * predecessors run (the fused kernel stages its input and builds its decode
 * tables while the new center is computed).  `encode_table`/`decode_table` are
 * the base tables of the RESULT's codebook, whose geometry must equal A's.
 * Work buffers: samples uint8[min(logical_numel, 4096)], shifted_encode
 * int32[256], extra_starts uint8[streams], summaries int32[4*blocks], spill
 * uint8[size]. */
int lct_update(const lct_operand *a /* host pointer */, const void *other, const float *alpha,
               const float *beta, int op, int alpha_is_one, int beta_is_one,
               const int32_t *encode_table, const int32_t *decode_table, uint8_t *samples,
               const uint16_t *known_values, uint16_t *result_values,
               int32_t *center, int32_t *shifted_encode, int32_t *shifted_decode,
               uint8_t *side_out, int32_t *encoded_out, uint8_t *extra_starts,
               int32_t *summaries, uint8_t *spill, int32_t *counts, int32_t *descriptor,
               int32_t *blocks_out, void *arena_storage, int max_free_regions, int64_t size,
               int64_t logical_numel, int block_symbols, int steps, int fixed_words,
               int rare_length, void *stream);

/* lct_update that also writes a dense BF16 tensor from the values it has in
 * registers anyway, so that an optimizer never materialises its decoded state:
 *   emit == LCT_EMIT_RESULT     dense_out = the new value of A (what AdamW's
 *                               weight update reads, sparse_utils.py:195-198);
 *   emit == LCT_EMIT_NESTEROV   dense_out = lerp(B, new A, *beta) with the LERP
 *                               arithmetic above: Muon's update direction
 *                               grad.lerp_(momentum, mu), sparse_utils.py:89-90.
 * dense_out is BF16[logical_numel], 16-byte aligned, and may be `other` itself
 * (every element of B is read by the thread that overwrites it, before it does).
 * emit == LCT_EMIT_NONE is lct_update.  Replaces the reference's sequence
 * decompress_free -> lerp_ -> lerp_ -> LCTTensor(...) of SparseMuon.step,
 * sparse_utils.py:133-146.
 * release_descriptor (may be NULL): descriptor of a region of the same arena -
 * the one A's overflow tails live in, for an in-place update - which is
 * returned to the arena right after the result's region has been reserved, by
 * the same kernel; release_status (int32[1]) receives what lct_buffer_free
 * would report.  The arena ends up as after lct_update + lct_buffer_free
 * (LCTensor.py:74-77: new value first, then old.free()).
 * When known_values is given, the sample pre-pass and the center are one
 * kernel and `samples` is not touched. */
#define LCT_EMIT_NONE 0
#define LCT_EMIT_RESULT 1
#define LCT_EMIT_NESTEROV 2
int lct_update_emit(const lct_operand *a /* host pointer */, const void *other, const float *alpha,
                    const float *beta, int op, int alpha_is_one, int beta_is_one,
                    const int32_t *encode_table, const int32_t *decode_table, uint8_t *samples,
                    const uint16_t *known_values, uint16_t *result_values,
                    int32_t *center, int32_t *shifted_encode, int32_t *shifted_decode,
                    uint8_t *side_out, int32_t *encoded_out, uint8_t *extra_starts,
                    int32_t *summaries, uint8_t *spill, int32_t *counts, int32_t *descriptor,
                    int32_t *blocks_out, void *arena_storage, int max_free_regions, int64_t size,
                    int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                    int rare_length, void *dense_out, int emit, int32_t *release_descriptor,
                    int32_t *release_status, void *stream);

/* Many compressed tensors of ONE geometry updated by one call (an optimizer
 * step over all its parameters): the five kernels of lct_update, each launched
 * once over all jobs - samples (16 CTAs per job), centers (one CTA per job),
 * the fused decode -> op -> re-encode (one CTA per block of every job), the
 * scans and arena reservations (in job order, so the arena ends up exactly as
 * after one lct_update per job), the tail compaction.  Same bytes in the same
 * output tensors as n_jobs calls of lct_update.  `jobs` is a DEVICE array
 * sorted by first_block; alpha, beta, op and the codebook are common to all
 * jobs.  Work buffers: samples uint8[4096 * n_jobs], shifted_encode
 * int32[256 * n_jobs], extra_starts uint8[256 * total_blocks], summaries
 * int32[4 * total_blocks] (job j uses the 4 * blocks_j ints from
 * 4 * first_block).  No counterpart in the reference, whose optimizers update
 * one tensor per call (LCT/components/sparse_utils.py:30-61). */
typedef struct lct_update_job {
  lct_operand a;                 /* the state to update */
  const void *other;             /* dense BF16 operand, int16[logical_numel] */
  const uint16_t *known_values;  /* NULL, or A's BF16 bits at the sample positions */
  uint16_t *result_values;       /* NULL, or uint16[min(logical_numel, 4096)] */
  uint8_t *side_out;             /* uint8[size] */
  int32_t *encoded_out;          /* int32[streams*fixed_words + 4] */
  uint8_t *spill;                /* uint8[size] work buffer */
  int32_t *center;               /* int32[1] */
  int32_t *shifted_decode;       /* int32[1024] */
  int32_t *counts;               /* int32[4] */
  int32_t *descriptor;           /* int32[4] */
  int32_t *blocks_out;           /* int32[3*blocks] */
  int64_t size;
  int64_t logical_numel;
  int64_t first_block;
  void *dense_out;               /* lct_update_batch_emit only: BF16[logical_numel], 16-byte aligned,
                                    may be `other`; ignored (may be NULL) otherwise */
} lct_update_job;

int lct_update_batch(const lct_update_job *jobs /* device */, int n_jobs, int64_t total_blocks,
                     const float *alpha, const float *beta, int op, int alpha_is_one,
                     int beta_is_one, const int32_t *encode_table, const int32_t *decode_table,
                     void *arena_storage, int max_free_regions, uint8_t *samples,
                     int32_t *shifted_encode, uint8_t *extra_starts, int32_t *summaries,
                     int block_symbols, int steps, int fixed_words, int rare_length,
                     void *stream);

/* lct_update_batch with the dense by-product of lct_update_emit for every job
 * (emit = LCT_EMIT_RESULT or LCT_EMIT_NESTEROV, written to jobs[j].dense_out):
 * the momentum step of all of Muon's parameters as one call, the Nesterov
 * directions overwriting the gradients (LCT/components/sparse_utils.py:88-90
 * for every parameter of :124-146 at once; the updates of different
 * parameters are independent, so doing them before the per-parameter
 * Newton-Schulz iterations changes no value). */
int lct_update_batch_emit(const lct_update_job *jobs /* device */, int n_jobs,
                          int64_t total_blocks, const float *alpha, const float *beta, int op,
                          int alpha_is_one, int beta_is_one, const int32_t *encode_table,
                          const int32_t *decode_table, void *arena_storage, int max_free_regions,
                          uint8_t *samples, int32_t *shifted_encode, uint8_t *extra_starts,
                          int32_t *summaries, int block_symbols, int steps, int fixed_words,
                          int rare_length, int emit, void *stream);

/* ---- shared overflow arena (TensorBuffer) ---------------------------------- */
/* storage layout: int32 free_starts[R] | free_sizes[R] | free_count | lock |
 * generation | pad to 16 bytes | payload[capacity]  (LCT/tensor_buffer.py:58-82).
 * Descriptor status: 0 ok, 1 no fit, 2 empty request, 5 freed, 7 lock wait
 * gave up.  Free status: 0 ok, 3 free list full, 4 invalid or stale, 7 lock
 * wait gave up.  (LCT/kernels/tensor_buffer.py:84-90, 171-178; 7 is new: the
 * reference spins without bound.) */

/* Replaces TensorBuffer.reset, tensor_buffer.py:130-136 (kernel :18-34). */
int lct_buffer_reset(void *storage, int max_free_regions, int32_t capacity_bytes, void *stream);
/* request = *requested_bytes + *item_count * item_bytes, rounded up to 16.
 * Replaces TensorBuffer.allocate / allocate_with_items, tensor_buffer.py:93-120. */
int lct_buffer_allocate(void *storage, const int32_t *requested_bytes,
                        const int32_t *item_count, int item_bytes, int32_t *descriptor,
                        int max_free_regions, void *stream);
/* Replaces the lct::tensor_buffer_free op, LCT/kernels/tensor_buffer_ops.py:5-15. */
int lct_buffer_free(void *storage, int32_t *descriptor, int32_t *status, int max_free_regions,
                    void *stream);
/* n regions returned under one lock, in list order: `descriptors` is a DEVICE
 * array of n descriptor pointers, status int32[n].  Same free list as n calls of
 * lct_buffer_free.  No counterpart in the reference. */
int lct_buffer_free_many(void *storage, int32_t *const *descriptors /* device */, int n,
                         int32_t *status, int max_free_regions, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LCT_B200_H */
