/*
 * void_b200 — C ABI of the B200 (sm_100a) block-sparse SpMM path: the quantized (INT8 / FP8) product and, on
 * the same kernels, the floating-point product, its gradients and the on-device format build.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, returns 0
 * (VOID_OK) or a negative status, never throws, never synchronises the stream and never
 * allocates device memory: workspaces are passed in by the caller.  The functions are what
 * a foreign-function binding of the reference's Python operators would bind; each comment
 * names the reference code (path inside the Khushiyant/void project) that the entry point
 * replaces.
 *
 * Vocabulary: a *tile* is one stored 32x32 block of A; a *tile row* is one row of the
 * block grid (32 matrix rows); a *panel* is a 32(k) x 128(n) slab of B; the *packed* form
 * of A is its tiles in tile-row-major order, 1024 bytes each, in the core-matrix order the
 * tensor cores read from shared memory (1024 * element bytes for the floating-point kinds).
 */
#ifndef VOID_B200_H_
#define VOID_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VOID_B200_ABI_VERSION 5

#if defined(__GNUC__)
#define VOID_API __attribute__((visibility("default")))
#else
#define VOID_API
#endif

/* status codes */
enum {
  VOID_OK = 0,
  VOID_ERR_BAD_ARG = -1,        /* null pointer, negative size, unknown enum value      */
  VOID_ERR_ALIGN = -2,          /* pointer or leading dimension breaks an alignment rule */
  VOID_ERR_SHAPE = -3,          /* sizes that the kernels do not support                 */
  VOID_ERR_ARCH = -4,           /* current device is not sm_100                          */
  VOID_ERR_CUDA = -5,           /* a CUDA runtime / driver call failed                   */
  VOID_ERR_WORKSPACE = -6,      /* caller workspace too small                            */
  VOID_ERR_DEVICE_TIMEOUT = -7, /* a bounded device-side wait gave up (see status word)  */
  VOID_ERR_TOO_LARGE = -8,      /* size beyond a documented maximum                      */
  VOID_ERR_TENSOR_MAP = -9      /* the driver refused the copy-engine descriptor of B    */
};

/* element kinds of the operands: 8-bit quantised (void_spmm_i8 / void_spmm_f8) and floating
 * point (void_spmm_fp; fp32 operands are multiplied as TF32, the precision tl.dot uses for
 * the reference's fp32 kernel on a GPU) */
enum { VOID_KIND_I8 = 0, VOID_KIND_F8E4M3 = 1, VOID_KIND_F16 = 2, VOID_KIND_BF16 = 3, VOID_KIND_TF32 = 4 };
/* output element types */
enum { VOID_OUT_F32 = 0, VOID_OUT_F16 = 1, VOID_OUT_BF16 = 2 };
/* epilogue activation codes; same numbering as get_activation_code, void/fusion.py:77-91 */
enum { VOID_ACT_NONE = 0, VOID_ACT_RELU = 1, VOID_ACT_GELU = 2, VOID_ACT_SILU = 3 };
/* how tile scales enter the result */
enum {
  VOID_SCALE_ROW_MEAN = 0, /* whole tile row in one accumulator, times the MEAN of the row's
                              tile scales: void/int_quant.py:479-481, :516-526            */
  VOID_SCALE_PER_TILE = 1  /* every tile's product is scaled by its own scale before it is
                              added: void/fp8.py:638-646, :657-659                        */
};

typedef void* void_stream_t; /* a cudaStream_t */

VOID_API const char* void_strerror(int status);
VOID_API int void_b200_abi_version(void);

/* ---------------------------------------------------------------------------------------
 * Tile index.  Replaces VOIDTensor.get_row_block_info, void/format.py:201-237 (same code in
 * void/int_quant.py:158-175 and void/fp8.py:712-720): row_ptr[nbr+1] = exclusive prefix sum
 * of tiles per tile row, block_indices[nnz] = argsort of (block_row * nbc + block_col).
 * Keys are unique, so the result is bit-exact with the reference's torch.argsort.
 * The tile list is not trusted: coordinates outside [0, nbr) x [0, nbc) are skipped and a coordinate
 * pair that occurs twice is counted once, so a bad list shows as row_ptr[nbr] < nnz (block_indices
 * then still holds valid positions only, but not a permutation) - check it before using the index.
 * ws: caller workspace of void_tile_index_ws_bytes(nbr, nbc) bytes (a bitmap of the block
 * grid plus per-row counters).
 * ------------------------------------------------------------------------------------- */
VOID_API size_t void_tile_index_ws_bytes(int32_t nbr, int32_t nbc);
VOID_API int void_build_tile_index(const int32_t* block_rows, const int32_t* block_cols, int64_t nnz,
                          int32_t nbr, int32_t nbc, int32_t* row_ptr, int32_t* block_indices,
                          void* ws, size_t ws_bytes, void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Format construction on the device.  Replaces the host-side work of dense_to_void,
 * void/format.py:352-446 (tile norms with torch ops, Morton codes and their sort in numpy
 * :413-424) and of csr_to_void, :248-349 (numpy throughout, one Python iteration per nonzero
 * :321-327).  Tiles are 32x32.  The kept tiles are ranked by a bitmap over Morton-code space
 * (morton(r, c) = bits of r on even positions, bits of c on odd ones, :41-51): rank order is
 * ascending Morton order, so nothing is sorted.
 *
 *   ws = caller workspace of void_format_ws_bytes(nbr, nbc) bytes (0: grid too large, more than
 *        16384 tiles along a side), shared by the calls of one conversion.
 *   1. void_dense_mark: a tile is kept when the sum of |x| over it exceeds threshold (:391-394);
 *      elem = VOID_ELEM_*; or void_csr_mark: a tile is kept when the CSR matrix stores an entry
 *      in it, zero or not (:287-296).  counts[2] (device, int64) receives the number of kept
 *      tiles and, for the dense form, the number of nonzero elements (nnz_original, :429).
 *   2. the caller reads counts[0], allocates, and calls void_morton_emit: block_rows,
 *      block_cols, morton_codes [n_blocks] in ascending Morton order.
 *   3. void_dense_gather copies the kept tiles (zero padding outside the matrix, :374-378);
 *      void_csr_scatter zero-fills values [n_blocks, 32, 32] and places every stored entry
 *      (entries with equal coordinates race; the reference keeps the later one).
 * ------------------------------------------------------------------------------------- */
enum { VOID_ELEM_F32 = 0, VOID_ELEM_F16 = 1, VOID_ELEM_BF16 = 2 };
VOID_API size_t void_format_ws_bytes(int32_t nbr, int32_t nbc);
VOID_API int void_dense_mark(const void* matrix, int32_t elem, int64_t ld, int32_t M, int32_t N,
                             float threshold, void* ws, size_t ws_bytes, int64_t* counts,
                             void_stream_t stream);
VOID_API int void_csr_mark(const int32_t* crow, const int32_t* col, int32_t M, int32_t N, void* ws,
                           size_t ws_bytes, int64_t* counts, void_stream_t stream);
VOID_API int void_morton_emit(const void* ws, int32_t nbr, int32_t nbc, int64_t n_blocks,
                              int32_t* block_rows, int32_t* block_cols, int64_t* morton_codes,
                              void_stream_t stream);
VOID_API int void_dense_gather(const void* matrix, int32_t elem, int64_t ld, int32_t M, int32_t N,
                               const int32_t* block_rows, const int32_t* block_cols,
                               int64_t n_blocks, void* values, void_stream_t stream);
VOID_API int void_csr_scatter(const int32_t* crow, const int32_t* col, const float* data, int32_t M,
                              int32_t N, const void* ws, int64_t n_blocks, float* values,
                              void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Pack.  Gathers the Morton-ordered 8-bit tiles (Int8VOIDTensor.values,
 * void/int_quant.py:116, or FP8VOIDTensor.values_fp8, void/fp8.py:445) into tile-row-major
 * order through block_indices and rewrites each 32x32 tile into 8x16-byte core matrices.
 * Also gathers tile_cols = block_cols[block_indices], tile_scales = scales[block_indices]
 * and row_scale[r] = (sum of the row's tile scales, added in row order) / count — the
 * reference's avg_scale for b_scale = 1, void/int_quant.py:516-526.  scales may hold one
 * value for all tiles (n_scales == 1, per-tensor mode).
 * packed must be 1024-byte aligned and hold nnz*1024 bytes.
 * ------------------------------------------------------------------------------------- */
VOID_API int void_pack_tiles(const void* values, const float* scales, int64_t n_scales,
                    const int32_t* block_cols, const int32_t* block_indices,
                    const int32_t* row_ptr, int64_t nnz, int32_t nbr, void* packed,
                    int32_t* tile_cols, float* tile_scales, float* row_scale,
                    void_stream_t stream);

/* FP8 tiles with their scales folded in (void_spmm_f8 with VOID_SCALE_ROW_MEAN and args->tile_terms = terms).
 * The reference multiplies every tile by its own scale before it is added to the row's sum
 * (void/fp8.py:638-659); the tensor cores cannot scale per tile, and reading every tile's product back to do
 * it in registers is what made the FP8 product slower than the INT8 one.  Here each element
 * a * scale_tile / R_row, R_row = the largest tile scale of the tile row, is stored as a sum of `terms`
 * (2 or 3) E4M3 numbers (nearest value, then the nearest value of the remainder): 8 significant bits with two
 * terms, 12 with three - the reference's own tl.dot rounds this operand to TF32's 11.  Packed tile j holds
 * its terms one after the other, (j * terms + k) * 1024; row_scale[r] receives R_row, which the epilogue
 * applies; tile_cols / tile_scales as in void_pack_tiles.  packed: nnz * terms * 1024 bytes, 1024-byte aligned. */
VOID_API int void_pack_tiles_f8_split(const void* values, const float* scales, int64_t n_scales,
                                      const int32_t* block_rows, const int32_t* block_cols,
                                      const int32_t* block_indices, const int32_t* row_ptr, int64_t nnz,
                                      int32_t nbr, int32_t terms, void* packed, int32_t* tile_cols,
                                      float* tile_scales, float* row_scale, void_stream_t stream);

/* Same gather for floating-point tiles (VOIDTensor.values, void/format.py:66): elem_bytes = 2
 * (fp16 / bf16) or 4 (fp32).  A packed tile takes 1024 * elem_bytes bytes and is stored as
 * [row / 8][k-chunk][row % 8][16 bytes] with 2 * elem_bytes 16-byte k-chunks per row, the order
 * the tensor cores read a K-major operand in.  fp32 tiles are rounded to the nearest TF32 value
 * on the way (the tensor cores would otherwise truncate them).  packed must be 1024-byte aligned. */
VOID_API int void_pack_tiles_fp(const void* values, int32_t elem_bytes, const int32_t* block_cols,
                                const int32_t* block_indices, int64_t nnz, void* packed,
                                int32_t* tile_cols, void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Quantisers.
 * void_quant_i8_tiles: per-tile symmetric INT8, scale = max(absmax/128, 1e-8),
 *   q = clamp(rint(x / scale), -128, 127): quantize_void_tensor / quantize_tensor /
 *   compute_scale_minmax, void/int_quant.py:328-388, :254-305, :178-214.
 * void_quant_fp8_tiles: per-tile E4M3, scale = max(amax/448, 1e-12), scale_inv = 1/scale,
 *   q = e4m3_rn(clamp(x * scale_inv, -448, 448)): quantize_to_fp8 with a fresh amax
 *   history, void/fp8.py:185-229, :91-105.
 * void_quant_cols: the same two formulas along the columns of a row-major [K,N] fp32
 *   matrix (per-column scales of B); the reference reaches this through
 *   quantize_tensor(B.T, PER_CHANNEL), void/int_quant.py:273-274, and
 *   quantize_to_fp8(B.T, per_row), void/fp8.py:177-180.  q is [K, ldq] bytes.
 * ------------------------------------------------------------------------------------- */
VOID_API int void_quant_i8_tiles(const float* values, int64_t nnz, int8_t* q, float* scales,
                        void_stream_t stream);
VOID_API int void_quant_fp8_tiles(const float* values, int64_t nnz, uint8_t* q, float* scale,
                         float* scale_inv, float* amax, void_stream_t stream);
VOID_API int void_quant_cols(const float* b, int64_t ldb, int32_t K, int32_t N, int32_t kind, void* q,
                    int64_t ldq, float* col_scale, float* col_scale_inv,
                    void_stream_t stream);
/* One symmetric INT8 scale for the whole [K, N] matrix (scale[0] = max(absmax/128, 1e-8)): the
 * PER_TENSOR quantisation void_spmm_int8 applies to a floating-point B, void/int_quant.py:565-573. */
VOID_API int void_quant_i8_tensor(const float* b, int64_t ldb, int32_t K, int32_t N, void* q, int64_t ldq,
                                  float* scale, void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Work plan.  A *segment* is a run of consecutive tiles of one tile row that one CTA
 * accumulates in tensor memory; a row cut into several segments is finished by the CTA
 * that arrives last (integer partial sums, so the result does not depend on arrival order).
 *
 * void_streamk_table reproduces compute_stream_k_workload, void/stream_k.py:36-110, on the
 * device: rows in order, each non-empty row cut into chunks of
 * target = min(ceil(nnz / n_workers), max_work) tiles; needs_atomic = chunk is not the
 * whole row.  n_workers_req <= 0 selects the reference default min(nnz, 1024).  The four
 * output arrays need capacity void_streamk_table_capacity(nnz, nbr) entries; the realised
 * count is written to *n_workers_out (device int32).
 *
 * void_plan_segments cuts the tile stream into n_cta contiguous shares of (nearly) equal
 * weight.  With split_rows = 0 share boundaries fall on tile-row boundaries; with
 * split_rows = 1 a boundary may fall on a chunk boundary of the worker table inside a heavy
 * row; with split_rows = 2 every worker of the table becomes a segment of its own.
 * Output: segs (8 int32 each: row, n_chunk, t0, t1, nseg, slot0, my_idx, counter),
 * cta_seg_ptr[n_cta+1], counts[4] = {n_segs, n_slots, n_counters, overflow flag}; segs needs
 * void_plan_capacity(...) entries.  n_counters is the number of split rows: each needs one
 * counter and one int32 accumulator of panels_per_item * 128 * 32 entries (void_spmm_args).
 * ------------------------------------------------------------------------------------- */
VOID_API int64_t void_streamk_table_capacity(int64_t nnz, int32_t nbr);
/* chunk length ("target_work") of the table: void/stream_k.py:61-67; 0 when nnz == 0 */
VOID_API int32_t void_streamk_target(int64_t nnz, int32_t n_workers_req, int32_t max_work);
/* ws: caller scratch of (nbr + 1) int32 */
VOID_API int void_streamk_table(const int32_t* row_ptr, int32_t nbr, int64_t nnz, int32_t n_workers_req,
                       int32_t max_work, int32_t* worker_rows, int32_t* worker_block_start,
                       int32_t* worker_block_end, uint8_t* worker_needs_atomic,
                       int32_t* n_workers_out, int32_t* ws, void_stream_t stream);
VOID_API int64_t void_plan_capacity(int64_t nnz, int32_t nbr, int32_t n_chunks, int32_t n_cta,
                                    int32_t split_rows, int32_t chunk_tiles);
VOID_API size_t void_plan_ws_bytes(int32_t nbr, int32_t n_cta);
/* row_cost (>= 1): what finishing one (tile row, column chunk) costs relative to one tile of work; it
 * weights the shares so that a CTA handed many short rows is not handed many tiles as well.
 * chunk_tiles: chunk length of the worker table (void_streamk_target), used when split_rows > 0.
 * woff: (nbr + 1) workers-before-row prefix left in the ws of void_streamk_table, needed for
 * split_rows = 2 only.  ws: device scratch of void_plan_ws_bytes(nbr, n_cta) bytes.          */
VOID_API int void_plan_segments(const int32_t* row_ptr, int32_t nbr, int32_t n_chunks, int32_t n_cta,
                                int32_t split_rows, int32_t chunk_tiles, int32_t row_cost,
                                const int32_t* woff, int32_t* segs, int64_t segs_capacity,
                                int32_t* cta_seg_ptr, int32_t* counts, void* ws, size_t ws_bytes,
                                void_stream_t stream);
/* The same splitting arithmetic over HOST arrays, run as plain loops on the CPU.  It exists so
 * that the splitter can be tested on machines without a GPU; the SpMM path never calls it.   */
VOID_API int void_plan_segments_host(const int32_t* row_ptr, int32_t nbr, int32_t n_chunks,
                                     int32_t n_cta, int32_t split_rows, int32_t chunk_tiles,
                                     int32_t row_cost, const int32_t* woff, int32_t* segs,
                                     int64_t segs_capacity, int32_t* cta_seg_ptr, int32_t* counts);

/* ---------------------------------------------------------------------------------------
 * SpMM  C = act(dequant(A_q . B_q) + bias).
 * void_spmm_i8 replaces void_spmm_int8_kernel / void_spmm_int8, void/int_quant.py:435-612;
 * void_spmm_f8 replaces void_spmm_fp8_kernel / void_spmm_fp8, void/fp8.py:577-742 (with B
 * also E4M3 and a per-column scale of B in the epilogue); act/bias give the fused epilogue
 * of void_spmm_activation_kernel, void/fusion.py:98-198, :38-43; a plan with split rows
 * gives the load-balanced form of stream_k_spmm_kernel, void/stream_k.py:113-230, without
 * its spin lock.
 * ------------------------------------------------------------------------------------- */
typedef struct void_spmm_args {
  /* A, packed (see void_pack_tiles) */
  const void* tiles;        /* nnz * 1024 * element bytes, 1024-byte aligned             */
  const int32_t* tile_cols; /* [nnz] block column of each packed tile                    */
  const float* tile_scales; /* [nnz] tile scales in packed order (VOID_SCALE_PER_TILE)   */
  const int32_t* row_ptr;   /* [nbr+1]                                                   */
  const float* row_scale;   /* [nbr] mean tile scale per row (VOID_SCALE_ROW_MEAN)       */
  int32_t nbr, nbc;
  int64_t nnz;
  /* B, row-major [K, N], ldb BYTES between k rows (multiple of 16)                       */
  const void* b;
  int64_t ldb;
  int32_t K, N;
  const float* col_scale; /* [N] per-column scale of B, or NULL                          */
  float b_scale;          /* scalar scale of B (1.0 when col_scale carries it)           */
  const float* bias;      /* [N] column bias added before the activation, or NULL        */
  /* C, row-major [M, N], ldc elements between rows                                      */
  void* out;
  int64_t ldc;
  int32_t M;
  int32_t out_dtype; /* VOID_OUT_*  */
  int32_t act;       /* VOID_ACT_*  */
  int32_t scale_mode; /* VOID_SCALE_* */
  /* optional raw accumulators, [nbr*32, N] int32 (INT8) or fp32 (FP8), ROW_MEAN mode    */
  void* acc_out;
  /* plan (see void_plan_segments); segs == NULL: one segment per (tile row, column chunk) */
  const int32_t* segs;
  const int32_t* cta_seg_ptr;
  int32_t n_cta;             /* CTAs the plan was made for; 0 without a plan             */
  void* partials;            /* n_counters * panels_per_item * 16 KiB of int32 row
                                accumulators, ZERO before the first use; left zero again */
  int64_t partials_bytes;    /* size of partials; a segment whose counter index does not fit
                                (index >= partials_bytes / (panels_per_item * 16 KiB)) is
                                skipped and the status word reads 2                       */
  int32_t* counters;         /* one per accumulator row of partials, zero before the first
                                use; left zero again                                      */
  void* worker_partials;     /* optional [n_segs, 32, N] int32: every segment's own sum  */
  /* device status word: 0; 1 = a bounded wait gave up; 2 = a split row of the plan does not fit
   * the scratch the caller provided                                                      */
  int32_t* status;
  /* launch shape; 0 = library default                                                   */
  int32_t panels_per_item; /* 128-column panels of B per work item: 1, 2 or 4            */
  int32_t stages;          /* shared-memory ring depth; 0: what fits beside the other CTAs of the SM, plus a
                            * shorter last stage from the bytes left over where that adds a fifth to the ring */
  int32_t grid;            /* CTAs to launch without a plan                              */
  int32_t tiles_per_stage; /* consecutive tiles of a row moved per ring stage: 1 ... 8         */
  /* diagnostics: NULL for every ordinary launch.  Not NULL selects a separately compiled diagnostic kernel
   * (slim INT8 row-accumulate or one-panel FP8 per-tile only, else VOID_ERR_BAD_ARG) that writes 64
   * uint64 nanosecond timestamps per launched CTA; the ordinary kernels contain none of that code.   */
  void* trace;
  int32_t cta_shape;       /* 0 default; 1 wide CTAs (13 warps, 2 per SM); 2 slim (7 warps, 4 per SM);
                              per-tile kernel with one panel only: 3 = 7 warps, 3 per SM; 4 = 10 warps, 3 per SM;
                              5 = 6 warps, 4 per SM */
  int32_t flags;           /* bit 1: no staged TMA store of 16-bit outputs (direct stores); bit 4: staged 16-bit
                              outputs leave in one store per result tile instead of one per epilogue warp;
                              bit 2: the caller vouches that the packed A (tiles, tile_cols, tile_scales,
                              row_ptr, row_scale) and the plan were completely written before any kernel
                              still in flight on the stream started - they are then read BEFORE the wait on
                              the previous kernel (programmatic dependent launch), which takes their
                              latency off the launch.  B, the scales of B, the biases and C are never
                              touched before that wait.                                               */
  /* [M] bias added per OUTPUT ROW before the activation, or NULL: the linear-layer form
   * act(W x + b[:, None]) of void_spmm_activation_row_bias_kernel, void/fusion.py:201-304 */
  const float* row_bias;
  /* 1: B and C are stored TRANSPOSED - b is [N, K] row-major (k contiguous, ldb bytes between its
   * rows n) and out is [N, M] row-major (ldc elements between its rows n).  This is the linear-layer
   * form y = x W^T with activations x [batch, in] and results y [batch, out] used as they lie in
   * memory, no transposed copies (the reference transposes both, void/fusion.py:586-598,
   * void/autograd.py:336).  Index meanings are unchanged: col_scale / bias are per n, row_bias per m.
   * Row-accumulate kernel only: not with VOID_SCALE_PER_TILE, FP8, a plan, acc_out or
   * worker_partials; at most two panels per work item.  0: as described above.               */
  int32_t transposed;
  /* 0 for every ordinary launch.  Test hooks: bits 0..15 = limit of every device-side wait in
   * milliseconds (0: the default of 2000); bit 16 = the first group of tiles of each CTA is never
   * delivered to the consumer, so that its wait runs out, the launch gives up in an orderly way and the
   * status word reads 1 - used to test that path without any faulting or unbounded wait.            */
  int32_t test_hooks;
  /* 0 or 1: one packed tile per stored tile.  2 or 3 (void_spmm_f8, VOID_SCALE_ROW_MEAN only): tiles packed by
   * void_pack_tiles_f8_split - every stored tile is a sum of that many E4M3 terms, 1024 bytes each, stored
   * one after the other; the kernel multiplies all terms by the same panel of B.                        */
  int32_t tile_terms;
  int32_t reserved;
  /* Reduction across GPUs inside the kernel (0: off).  Replaces the all_reduce of the full [M, N] result that
   * the reference runs after the local products of COLUMN_WISE / BLOCK_WISE shards, void/distributed.py:252-267.
   * With n_peers = world size, every segment of the plan is one rank's part of a tile row (nseg = number of ranks
   * that contribute, slot0 = the rank that OWNS the row, counter = the row's index in the owner's scratch).  The
   * kernel adds its int32 partial tile into peer_partials[owner] with system-scope atomic adds (NVLink when the
   * owner is another GPU), bumps peer_counters[owner][counter], and whichever rank arrives last reads the sums
   * back, dequantises and writes the owner's rows of C through peer_out[owner] - a pointer to the owner's C
   * shard moved back by the owner's first row, so that the GLOBAL tile row indexes it.  All three arrays hold
   * one pointer per rank, valid on this GPU (the rank's own buffers for its own index); partials_bytes is the
   * size of each rank's accumulator array.  No kernel waits for another GPU; the caller orders consecutive
   * launches (every rank's launch i must have finished before any rank's launch i+1 adds into the same
   * scratch, e.g. by a small collective on the stream).  Row-accumulate kernel only, not with transposed,
   * acc_out or worker_partials.                                                                        */
  int32_t n_peers;
  /* 1: instead of adding into one shared accumulator per row, every contributing rank STORES its int32 partial tile
   * into its own slot of the owner's scratch - peer_partials[owner] + ((counter * n_peers + this rank) * panels_per_item
   * + panel) * 16 KiB - with plain stores and nothing else (no counters, no last arriver; peer_counters / peer_out are
   * not used; a rank without tiles in a row stores nothing).  The owner adds the slots and dequantises with
   * void_reduce_slots once every rank's launch has finished.  partials_bytes = size of one rank's slot array.  */
  int32_t peer_slots;
  void* peer_partials[8];
  int32_t* peer_counters[8];
  void* peer_out[8];
  /* Launches without a plan: the order in which the persistent CTAs take the tile rows, int32 [nbr], a permutation of
   * 0 .. nbr - 1 (work item i is tile row row_order[i / chunks], column chunk i % chunks), or NULL for 0, 1, 2, ...
   * The CTAs that start first take the first items, so tile rows sorted by falling tile count give the longest rows
   * the earliest start and leave the shortest for the CTAs that share an SM with the most others.  The result does not
   * depend on the order.  Entries are clamped to 0 .. nbr - 1; a list that is not a permutation leaves tile rows of C
   * unwritten (and writes others twice) but reads and writes nothing outside the tensors. */
  const int32_t* row_order;
} void_spmm_args;

VOID_API int void_spmm_i8(const void_spmm_args* args, void_stream_t stream);
VOID_API int void_spmm_f8(const void_spmm_args* args, void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Floating-point product.  Replaces void_spmm_kernel / void_spmm, void/ops.py:43-217; with
 * act / bias also void_spmm_activation_kernel / void_spmm_gelu on a floating VOIDTensor,
 * void/fusion.py:98-198, :381-399; with a plan also stream_k_spmm_kernel / void_spmm_stream_k,
 * void/stream_k.py:113-301.
 * kind = VOID_KIND_TF32 (A tiles and B are fp32; products in TF32, fp32 accumulation),
 * VOID_KIND_F16 or VOID_KIND_BF16 (A tiles and B in that type; exact products, fp32
 * accumulation).  args->tiles comes from void_pack_tiles_fp; args->ldb is in BYTES and a
 * multiple of 16; scale_mode must be VOID_SCALE_ROW_MEAN with row_scale == NULL (no scales);
 * col_scale / b_scale / bias / act / out_dtype work as in void_spmm_i8.  With a plan, the
 * pieces of a split row are added with fp32 atomic adds, so the last bits of such rows can
 * differ from run to run (the reference's spin-lock version has the same property).
 * ------------------------------------------------------------------------------------- */
VOID_API int void_spmm_fp(const void_spmm_args* args, int32_t kind, void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Gradient of the floating-point product with respect to the stored tiles of A.  Replaces
 * void_spmm_backward_a_kernel and its launch in VOIDSpMMFunction.backward,
 * void/autograd.py:14-96, :196-219:
 *     grad_tiles[i] = grad_out[32*br_i : 32*br_i+32, :] . b[32*bc_i : 32*bc_i+32, :]^T
 * for the stored tiles only, fp32 accumulation, result in out_dtype.  (The other gradient,
 * dB = A^T . dC, is void_spmm_fp on the transposed tensor, void/autograd.py:178-191.)
 * grad_out [M, N] and b [K, N] are row-major of the element type of kind (VOID_KIND_TF32: fp32
 * multiplied as TF32; VOID_KIND_F16 / VOID_KIND_BF16), 16-byte aligned, ldg / ldb in BYTES and
 * multiples of 16.  items [n_items][4] int32 = (tile row, first packed tile, tile count <= 4, 0):
 * groups of consecutive packed tiles of one tile row; tile_cols / block_indices as produced by
 * void_pack_tiles_fp / void_build_tile_index; grad_tiles [nnz][32][32] is written at
 * block_indices[packed position], i.e. in the order of the caller's tile list.
 * ------------------------------------------------------------------------------------- */
VOID_API int void_spmm_tile_grad(const void* grad_out, int64_t ldg, const void* b, int64_t ldb,
                                 int32_t M, int32_t K, int32_t N, int32_t kind,
                                 const int32_t* items, int32_t n_items, const int32_t* tile_cols,
                                 const int32_t* block_indices, void* grad_tiles,
                                 int32_t out_dtype, int32_t* status, void_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * void_spmm_i8 for callers that have no way to hand over scratch memory.  (This entry point has
 * no counterpart in the reference; it exists for embedders of this library.)
 *
 * A planned launch with split tile rows needs device scratch: one int32 accumulator and one
 * arrival counter per split row.  void_spmm_i8 takes them from the caller (args->partials,
 * args->counters).  Some callers cannot provide them: a serving process whose own allocator
 * claimed the whole GPU at start-up, so that cudaMalloc would fail; code running under a "no
 * allocation after warm-up" rule (hard real-time loops, sandboxed plug-ins); a host language
 * binding that can pass pointers it was given but owns no device allocator.  For them this variant
 * uses an array that is part of the library's device image instead and allocates nothing: it
 * calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * Same arguments as void_spmm_i8 with a plan (args->segs, args->cta_seg_ptr, args->n_cta,
 * args->panels_per_item are required); args->partials and args->counters are ignored.
 * n_split_rows is the plan's counts[2] (void_plan_segments).
 *
 * Limits: n_split_rows * panels_per_item * 16 KiB <= 8 MiB and n_split_rows <= 4096; anything
 * larger returns VOID_ERR_TOO_LARGE.  The array costs 8 MiB + 16 KiB on every GPU that loads the
 * library, until the process exits.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call outside any stream capture.
 * "Allocates nothing" is about the calls: the array is part of the library's device image, and the CUDA
 * runtime reserves device memory for that image (these 8 MiB + 16 KiB included) when the library is first
 * used on a device (with lazy module loading: at the first call that launches a kernel or asks for the
 * array's address).  An embedder whose own allocator is going to claim the rest of the GPU should make its
 * first call of this entry point on each device - any small product - before it does so.
 * All calls on a device share the one array, and it keeps the previous call's contents: the part
 * a call uses (accumulators and counters) is cleared in stream order before its launch.  Two
 * calls that overlap on the GPU (different streams, or different host threads on one device)
 * race on it - serialise them.
 * ------------------------------------------------------------------------------------- */
VOID_API int void_spmm_i8_static_scratch(const void_spmm_args* args, int32_t n_split_rows,
                                         void_stream_t stream);

/* Measurement aid (no counterpart in the reference): launches an empty kernel with the grid, block size,
 * dynamic shared memory and launch attribute (programmatic stream serialisation) of an SpMM launch.  What
 * a stream of such launches costs per launch is the part of an SpMM launch's time that no kernel code can
 * remove; bench.py --workload floor reports it next to an SpMM over an empty A. */
VOID_API int void_launch_floor(int32_t grid, int32_t threads, int32_t smem_bytes, void_stream_t stream);

/* Second half of the sum over ranks in slot form (void_spmm_args.peer_slots): for the rows_owned tile rows this
 * GPU owns (global tile rows row0 ...), add the partial tiles the ranks stored - slots [rows_owned][chunk][n_ranks][panel of the
 * chunk][32][128] int32 with chunks of panels_per_item panels as in the SpMM launch, contrib[row] = bit mask of the
 * ranks that stored one - and apply the INT8 epilogue of
 * void/int_quant.py:516-540 with the WHOLE row's mean scale (row_scale, indexed by global tile row), per-column
 * scales, bias and activation; out = this GPU's rows of C, [rows_owned * 32, N].  Together with the stores of the
 * SpMM launches this replaces dist.all_reduce of the full result, void/distributed.py:252-267. */
VOID_API int void_reduce_slots(const void* slots, const uint8_t* contrib, int32_t n_ranks, int32_t rows_owned,
                               int32_t row0, int32_t n_panels, int32_t panels_per_item, const float* row_scale,
                               const float* col_scale,
                               float b_scale, const float* bias, int32_t act, void* out, int64_t ldc,
                               int32_t out_dtype, int32_t M, int32_t N, void_stream_t stream);

/* number of SMs of the current device (grid sizing on the host side) */
VOID_API int void_device_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif /* VOID_B200_H_ */
