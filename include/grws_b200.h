/*
 * grws_b200.h -- C ABI of libgrws_b200.so, the sm_100a replacement for Graph_RWS's native
 * extension `core_lib` (core/wrapper/bind.cpp:78-161).
 *
 * Conventions, all entry points:
 *   - plain pointers and sizes, no framework types; every array pointer is DEVICE memory unless
 *     its comment says "host";
 *   - the caller owns every buffer (inputs, outputs and scratch); nothing is allocated or freed
 *     inside, nothing synchronises with the host, all work is queued on `stream`
 *     (a cudaStream_t passed as void*), so calls are re-entrant and may come from several host
 *     threads on several streams, as the reference's sampler thread does
 *     (helper/engine.py:118-153);
 *   - the return value is GRWS_OK (0) or a negative grws_status; grws_last_error() returns the
 *     message of the calling thread's last failure.  The reference raises through TORCH_CHECK
 *     (core/wrapper/spmm_wrapper.cu:48-51,89-90); the Python shim turns a negative status into
 *     the same RuntimeError.
 *
 * BCSR layout (core/wrapper/convert_wrapper.cpp:27-180, data/bcsr.py:23-62):
 *   window_offset        int64 [W+1]   prefix sum of tiles per 16-row window
 *   original_col_indices int32 [T*8]   per window: sorted unique column ids, 8 per tile, -1 pad
 *   values_condensed     [T*16*8]      per tile row-major [16][8]; fp32, fp16 or bf16
 */
#ifndef GRWS_B200_H
#define GRWS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GRWS_TILE_ROWS 16
#define GRWS_TILE_COLS 8

typedef enum { GRWS_F32 = 0, GRWS_F16 = 1, GRWS_BF16 = 2 } grws_dtype;

typedef enum {
    GRWS_OK = 0,
    GRWS_ERR_INVALID = -1,      /* bad argument (null pointer, negative size, misalignment)   */
    GRWS_ERR_UNSUPPORTED = -2,  /* dtype / shape combination this build has no kernel for     */
    GRWS_ERR_CUDA = -3,         /* a CUDA runtime call or launch failed                        */
    GRWS_ERR_SCRATCH = -4,      /* caller-provided scratch or output buffer too small          */
    GRWS_ERR_DEVICE = -5        /* a kernel reported a failure through its status word         */
} grws_status;

/* SpMM kernel selection. AUTO picks TCGEN05 when the shape allows it, else WARP_MMA. */
typedef enum { GRWS_SPMM_AUTO = 0, GRWS_SPMM_WARP_MMA = 1, GRWS_SPMM_TCGEN05 = 2 } grws_spmm_algo;

const char *grws_last_error(void);
int grws_version(void);

/* ------------------------------------------------------------------------------------------
 * Forward SpMM  C[W*16, N] = A_bcsr * B[K, N].
 * Replaces spmm_tc_wrapper + tcspmm_base_kernel (core/wrapper/spmm_wrapper.cu:33-95,
 * core/include/spmm_tc.cuh:40-195).  Differences from the reference, all deliberate: every one
 * of the N columns is computed (the reference computes 8*warps_per_block of them), values and
 * B may be fp16/bf16 as well as fp32 (fp32 operands are rounded to TF32 like the reference,
 * spmm_tc.cuh:118-121,144-145), accumulation is fp32, there is no host synchronisation.
 * Column ids equal to -1 contribute nothing (spmm_tc.cuh:131-141); all others must be < K.
 *   num_tiles_bound : any upper bound on window_offset[W] known to the host without a sync,
 *                     e.g. the allocated tile count of `cols`;
 *   val_dtype must equal b_dtype; N % 8 == 0; ldb, ldc in elements, rows 16-byte aligned;
 *   algo : GRWS_SPMM_AUTO takes the tcgen05 kernel for fp16 / bf16 operands of width 128 or 256,
 *          and of widths 16 .. 120 when num_tiles_bound >= 512 (a narrow operand is multiplied
 *          as 128 features of which the missing ones are zeros and only N are written); every
 *          other case runs on the warp-MMA kernel.  GRWS_SPMM_TCGEN05 accepts N = 256 and every
 *          multiple of 8 up to 128;
 *   scratch : grws_spmm_scratch_bytes(...) bytes, contents need not be initialised.
 * The same entry point computes the backward product A^T * G when given the cached transposed
 * BCSR built by grws_bcsr_transpose_* (this replaces the reference's atomic scatter
 * spmm_transpose_wrapper + spmm_bcsr_transpose_atomic_kernel, spmm_wrapper.cu:109-152,
 * spmm_tc.cuh:211-270).
 * ------------------------------------------------------------------------------------------ */
size_t grws_spmm_scratch_bytes(int64_t num_windows, int64_t num_tiles_bound, int64_t N, int algo);

/* Which kernel `algo` resolves to for this dtype and width (GRWS_SPMM_WARP_MMA or _TCGEN05).
 * The tcgen05 kernel keeps a status word (int32) in the first bytes of `scratch`: 0 after a
 * clean run, otherwise the code of the wait that ran out (its waits on shared-memory barriers
 * are bounded, so a broken pipeline ends with a status instead of hanging the GPU). */
int grws_spmm_resolve_algo(int dtype, int64_t N, int algo);

int grws_spmm_fwd(const int64_t *window_offset, const int32_t *cols, const void *vals,
                  int val_dtype, const void *B, int b_dtype, int64_t ldb, void *C, int c_dtype,
                  int64_t ldc, int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N,
                  void *scratch, size_t scratch_bytes, int algo, void *stream);

/* ------------------------------------------------------------------------------------------
 * SpMM on a graph that is multiplied many times (full-graph training: the same BCSR every epoch).
 * The reference has no counterpart (its kernel maps one thread block to one window,
 * core/include/spmm_tc.cuh:48-50).  The tcgen05 kernel gives each persistent CTA a contiguous range
 * of tiles; grws_spmm_fwd finds the ranges at the start of every launch by a search over
 * `window_offset`, with equal tile counts.  A plan holds ranges computed once for a graph, with
 * equal numbers of pipeline stages (what a CTA's run time follows), so the slowest CTA finishes
 * earlier and the search is gone:
 *   grws_spmm_plan_bytes : size of the plan buffer for this shape on the current device;
 *   grws_spmm_plan_build : queues one small kernel that fills `plan` from `window_offset`; call it
 *                          again whenever `window_offset` changes;
 *   grws_spmm_fwd_planned: grws_spmm_fwd with the plan (null = none).  The plan is used by the
 *                          tcgen05 kernel only, and only if it was built for the same num_windows,
 *                          tile count, K class and N on a device of the same size; otherwise the
 *                          launch searches its ranges as grws_spmm_fwd does.  A plan built from
 *                          another graph of the same shape gives wrong results.
 * ------------------------------------------------------------------------------------------ */
size_t grws_spmm_plan_bytes(int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N);
int grws_spmm_plan_build(const int64_t *window_offset, int64_t num_windows, int64_t num_tiles_bound,
                         int64_t K, int64_t N, void *plan, size_t plan_bytes, void *stream);
int grws_spmm_fwd_planned(const int64_t *window_offset, const int32_t *cols, const void *vals,
                          int val_dtype, const void *B, int b_dtype, int64_t ldb, void *C, int c_dtype,
                          int64_t ldc, int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N,
                          void *scratch, size_t scratch_bytes, int algo, const void *plan,
                          size_t plan_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * Status of the tcgen05 SpMM launches.  The reference has no counterpart: its kernels cannot
 * report anything (errors are host-side TORCH_CHECKs, core/wrapper/spmm_wrapper.cu:48-51).
 * Every wait of the tcgen05 kernel on a shared-memory barrier is bounded; a launch whose wait
 * runs out stops its pipeline, leaves its output incomplete, writes the code of the wait into
 * the status word at the start of its scratch and into one word per device that keeps the worst
 * code since it was last cleared.  Launches never synchronise, so the status is read separately:
 *   grws_spmm_last_status : queues, on `stream`, a copy of the current device's word to
 *                           `out_status` (device or pinned host memory) and, if `reset`, clears
 *                           the word after the copy; no synchronisation;
 *   grws_spmm_check       : synchronises `stream`, reads the word, clears it when non-zero and
 *                           returns GRWS_ERR_DEVICE with a message naming the wait, else GRWS_OK.
 *                           Call it where the host synchronises anyway (end of an epoch);
 *   grws_spmm_set_wait_limit : the limit of one wait in SM clocks for launches made after the
 *                           call (0 restores the default of 3e9, about 1.5 s); a diagnostic
 *                           knob, process-wide.
 * The first SpMM call or status call on a device looks up the word's device address
 * (cudaGetSymbolAddress): make it before any stream capture.
 * ------------------------------------------------------------------------------------------ */
int grws_spmm_last_status(int *out_status, int reset, void *stream);
int grws_spmm_check(void *stream);
int grws_spmm_set_wait_limit(long long sm_clocks);

/* ------------------------------------------------------------------------------------------
 * Forward SpMM that allocates nothing and takes no scratch buffer.  It has no counterpart in
 * the reference.  It exists for callers that cannot provide device scratch: code that runs
 * inside another framework's memory pool and only receives its input and output buffers, a
 * serving loop whose device memory was fixed at start-up, a host that must not call cudaMalloc
 * at this point.  The kernel's scratch (status word, per-CTA split-window counters, fp32 partial tiles
 * of windows split between CTAs) lives in a fixed array inside the library instead:
 *   - GRWS_SPMM_STATIC_SCRATCH_BYTES (about 21 MB) per GPU that loads the library, held until
 *     the process exits; sized for N <= 256 on devices with up to 160 SMs -- a call that would
 *     need more returns GRWS_ERR_SCRATCH;
 *   - covers the tcgen05 kernel only: fp16 / bf16 operands, N = 128 or 256; anything else
 *     returns GRWS_ERR_UNSUPPORTED (use grws_spmm_fwd with caller scratch);
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call before any stream capture;
 *   - every call shares the array, which keeps the previous call's contents (the status word is
 *     cleared on the stream before each launch).  Calls that overlap on the GPU race on it:
 *     issue them on one stream, or otherwise order them;
 *   - the status word of a call lives inside the array, out of the caller's reach: a wait that ran
 *     out is reported through grws_spmm_last_status / grws_spmm_check.
 * Arguments as grws_spmm_fwd, without scratch and algo.
 * ------------------------------------------------------------------------------------------ */
#define GRWS_SPMM_STATIC_SCRATCH_BYTES (256 + 131072 + 32768 + 160 * 4 * 2 * 16 * 256 * 4)

int grws_spmm_fwd_static(const int64_t *window_offset, const int32_t *cols, const void *vals,
                         int val_dtype, const void *B, int b_dtype, int64_t ldb, void *C,
                         int c_dtype, int64_t ldc, int64_t num_windows, int64_t num_tiles_bound,
                         int64_t K, int64_t N, void *stream);

/* ------------------------------------------------------------------------------------------
 * CSR -> BCSR on the device, two phases so that the caller can allocate exact outputs.
 * Replaces csr_to_bcsr_cpu (core/wrapper/convert_wrapper.cpp:27-180; called from
 * data/bcsr.py:209-216) and produces bit-identical arrays: per window the sorted unique
 * column ids, 8 per tile, -1 padding, values [tile][16][8] with zeros where there is no edge,
 * the last duplicate of a (row, column) pair winning.
 *   count: writes window_offset [ceil(num_rows/16)+1]; the caller then reads its last entry
 *          (the tile count T) and allocates out_cols [T*8], out_vals [T*128];
 *   fill : must get the same scratch buffer, untouched since the count call.  num_tiles may be
 *          any bound >= T (nnz / 8 + number of windows always is), which saves the caller the
 *          read-back: the tiles past T are written empty (ids -1, values 0).
 * row_ptr int64 [num_rows+1], col_idx int32 [nnz] (0 <= id), values fp32 [nnz]; nnz < 2^31.
 * ------------------------------------------------------------------------------------------ */
size_t grws_csr_to_bcsr_scratch_bytes(int64_t num_rows, int64_t nnz);

int grws_csr_to_bcsr_count(int64_t num_rows, const int64_t *row_ptr, const int32_t *col_idx,
                           const float *values, int64_t nnz, int64_t *window_offset, void *scratch,
                           size_t scratch_bytes, void *stream);

int grws_csr_to_bcsr_fill(int64_t num_rows, int64_t nnz, const int64_t *window_offset,
                          int64_t num_tiles, int32_t *out_cols, void *out_vals, int val_dtype,
                          void *scratch, size_t scratch_bytes, void *stream);

/* The count phase for CSR arrays whose entry count the host knows only as a bound (per-step
 * builders that must not read a size back): only the first row_ptr[num_rows] entries of col_idx
 * and values exist, nnz_bound >= that count sizes the scratch (grws_csr_to_bcsr_scratch_bytes(
 * num_rows, nnz_bound)) and is what grws_csr_to_bcsr_fill must be given as nnz.
 * num_cols_bound: 0, or a number every column id is below; the builder then sorts keys with a
 * narrower column field (fewer radix passes: it matters for the small blocks of a sampled step). */
int grws_csr_to_bcsr_count_bounded(int64_t num_rows, const int64_t *row_ptr, const int32_t *col_idx,
                                   const float *values, int64_t nnz_bound, int64_t num_cols_bound,
                                   int64_t *window_offset, void *scratch, size_t scratch_bytes,
                                   void *stream);

/* The count phase straight from a hop's fixed-stride neighbour lists (this, with
 * grws_csr_to_bcsr_fill, replaces build_col_to_val_map_kernel + recompress_sampled_bcsr_kernel,
 * core/include/sampling.cuh:471-579,707-773): row i has the entries local[i*fanout + j] >= 0
 * with weights w[i*fanout + j]; -1 marks an empty slot.  Scratch as
 * grws_csr_to_bcsr_scratch_bytes(n_dst, n_dst*fanout); the fill call takes nnz = n_dst*fanout.
 * num_cols_bound as above (0, or the length of the hop's source list). */
int grws_block_build_count(const int32_t *local, const float *w, int64_t n_dst, int fanout,
                           int64_t num_cols_bound, int64_t *window_offset, void *scratch,
                           size_t scratch_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * All-gather of row shards over NVLink with the library's own kernels (the reference is
 * single-GPU: no counterpart).  Every rank owns a staging block and a control block in memory
 * that all ranks of the node can address (one symmetric allocation each, mapped into every
 * rank); `stages` and `ctrl` are DEVICE arrays of `world` pointers to them as this rank sees
 * them, this rank's own included (`my_stage` is that one again, as a host-side value).  The call
 * queues two kernels: one copies `local` (local_bytes, the rest of the stage_bytes zero-filled)
 * into this rank's staging block once every peer has read the previous exchange, the other copies
 * all ranks' staging blocks into `out` ([world][stage_bytes]) once every rank has published.
 * `state` is grws_peer_state_bytes() of zero-initialised local device memory that the calls of
 * one communicator share; the control blocks (grws_peer_ctrl_bytes() each) start zeroed too.
 * All ranks must make the same sequence of calls with the same stage_bytes.  The waits are
 * bounded by `wait_limit` SM clocks; a wait that runs out leaves a non-zero status in the
 * int32 word state[3] (1: peers still reading the previous exchange, 2: peers never published),
 * `out` is then undefined and the call returns all the same.  No host synchronisation.
 * ------------------------------------------------------------------------------------------ */
size_t grws_peer_ctrl_bytes(void);
size_t grws_peer_state_bytes(void);
int grws_peer_all_gather(const void *local, int64_t local_bytes, void *my_stage, int64_t stage_bytes,
                         const void *const *stages, void *const *ctrl, int world, int rank,
                         void *state, void *out, long long wait_limit, void *stream);
/* The push form of the same exchange: every rank owns an inbox of [world][stage_bytes] in symmetric
 * memory (`inboxes`: device array of `world` pointers); the call stores this rank's rows into slot
 * `rank` of every inbox once all ranks are done with the previous contents, and when its kernels
 * have run this rank's inbox holds the gathered operand -- until this rank's next call.  One pass
 * over the data instead of two, and stores over the links instead of loads. */
int grws_peer_all_gather_push(const void *local, int64_t local_bytes, int64_t stage_bytes,
                              void *const *inboxes, void *const *ctrl, int world, int rank,
                              void *state, long long wait_limit, void *stream);

/* ------------------------------------------------------------------------------------------
 * Row normalisation between the graph convolutions: y = LayerNorm(act(x)) * gamma + beta over the
 * C features of every row, act = identity or ReLU (relu_input != 0), and its backward pass.  The
 * reference goes through torch.nn.LayerNorm and a separate activation (models/model.py:117-121).
 * x, y, dy, dx: [rows, C] row-major and contiguous, gamma / beta [C], all of `dtype`; mean / rstd
 * [rows] fp32 (written by the forward call, read by the backward call); dgamma / dbeta [C] fp32.
 * C % 8 == 0, C <= 1024.  Deterministic (no atomics).  Backward scratch:
 * grws_layer_norm_scratch_bytes(C).
 * ------------------------------------------------------------------------------------------ */
size_t grws_layer_norm_scratch_bytes(int64_t C);
int grws_layer_norm_fwd(const void *x, const void *gamma, const void *beta, void *y, float *mean,
                        float *rstd, int64_t rows, int64_t C, int dtype, int relu_input, float eps,
                        void *stream);
int grws_layer_norm_bwd(const void *x, const void *gamma, const void *dy, const float *mean,
                        const float *rstd, void *dx, float *dgamma, float *dbeta, int64_t rows,
                        int64_t C, int dtype, int relu_input, void *scratch, size_t scratch_bytes,
                        void *stream);

/* ------------------------------------------------------------------------------------------
 * BCSR -> CSR of the transposed matrix (rows = the BCSR's column ids), the first half of
 * building the cached transposed BCSR that the backward product runs on.  The reference has
 * no such structure: its backward is an atomicAdd scatter over the forward graph
 * (core/include/spmm_tc.cuh:211-270, called from layers/layer.py:71-77).  Entries with a -1
 * column id, an id >= num_cols or a zero value are dropped, like spmm_tc.cuh:258,264.
 *   count: writes row_ptr_t int64 [num_cols+1]; the caller reads its last entry (nnz);
 *   fill : writes out_col int32 [nnz] (row ids of A) and out_val fp32 [nnz]; the order of the
 *          entries inside one row is unspecified (grws_csr_to_bcsr_* sorts them).
 * ------------------------------------------------------------------------------------------ */
size_t grws_bcsr_transpose_scratch_bytes(int64_t num_cols);

int grws_bcsr_transpose_count(const int64_t *window_offset, const int32_t *cols, const void *vals,
                              int val_dtype, int64_t num_windows, int64_t num_cols,
                              int64_t *row_ptr_t, void *scratch, size_t scratch_bytes, void *stream);

int grws_bcsr_transpose_fill(const int64_t *window_offset, const int32_t *cols, const void *vals,
                             int val_dtype, int64_t num_windows, int64_t num_cols,
                             const int64_t *row_ptr_t, int32_t *out_col, float *out_val,
                             void *scratch, size_t scratch_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * BCSR -> CSR of the same matrix (rows ascending in column id): the sampler walks CSR rows.
 * No counterpart in the reference, whose sampler reads the BCSR tiles directly
 * (core/include/sampling.cuh:188-394).  count writes row_ptr int64 [num_rows+1]; the caller
 * reads its last entry (nnz) and allocates out_col int32 [nnz], out_val fp32 [nnz] for fill.
 * ------------------------------------------------------------------------------------------ */
size_t grws_bcsr_to_csr_scratch_bytes(int64_t num_rows);

int grws_bcsr_to_csr_count(const int64_t *window_offset, const int32_t *cols, const void *vals,
                           int val_dtype, int64_t num_windows, int64_t num_rows, int64_t *row_ptr,
                           void *scratch, size_t scratch_bytes, void *stream);

int grws_bcsr_to_csr_fill(const int64_t *window_offset, const int32_t *cols, const void *vals,
                          int val_dtype, int64_t num_windows, int64_t num_rows,
                          const int64_t *row_ptr, int32_t *out_col, float *out_val, void *stream);

/* ------------------------------------------------------------------------------------------
 * One hop of neighbour sampling.  Replaces Phase 1 of sample_one_layer_internal
 * (core/wrapper/sampling_wrapper.cu:101-157, warp_centric_find_top_k_kernel,
 * core/include/sampling.cuh:65-448) with different semantics: the reference keeps, per 16-row
 * window, the top-K columns by edge weight; this samples, per frontier node, `fanout`
 * neighbours uniformly without replacement from a Philox4x32-10 stream keyed by
 * (seed, node, hop) -- counter {node, hop, j/2, 0}, key = seed, draw j = words (2(j&1)+1 :
 * 2(j&1)).  Degree <= fanout takes all neighbours in CSR order; otherwise Floyd's subset
 * algorithm with pick_j = floor(draw_j * (deg - fanout + j + 1) / 2^64).  One warp per node.
 *   nodes int32 [num_nodes] (-1 entries give an empty list); 1 <= fanout <= 256;
 *   out_nbr int32 [num_nodes*fanout] (-1 padding), out_w fp32 [num_nodes*fanout] (CSR values
 *   of the picked edges, 1.0 when values is NULL), out_cnt int32 [num_nodes] or NULL.
 * ------------------------------------------------------------------------------------------ */
int grws_sample_hop(const int64_t *row_ptr, const int32_t *col_idx, const float *values,
                    const int32_t *nodes, int64_t num_nodes, int fanout, uint64_t seed, uint32_t hop,
                    int32_t *out_nbr, float *out_w, int32_t *out_cnt, void *stream);

/* ------------------------------------------------------------------------------------------
 * Dedup + reindex of a hop.  Replaces prepare_windows_and_masks + the per-layer
 * reindex_bcsr call (core/wrapper/sampling_wrapper.cu:283-347, models/model.py:127-143) for
 * per-node sampling: the hop's source list is the destination nodes, in the given order,
 * followed by the sampled neighbours that are not destination nodes in ascending id order; the
 * local id of a node is its position in that list.
 *   out_src     int32 [n_dst + n_dst*fanout]  source list (the first out_counts[0] entries)
 *   out_local   int32 [n_dst*fanout]          local id of every sampled neighbour, -1 for empty
 *   out_row_ptr int64 [n_dst+1]               prefix sum of the valid entries per destination
 *   out_counts  int64 [2]                     {number of source nodes, number of sampled edges}
 * ------------------------------------------------------------------------------------------ */
size_t grws_dedup_scratch_bytes(int64_t n_dst, int fanout);

int grws_dedup_reindex(const int32_t *dst, int64_t n_dst, const int32_t *nbr, int fanout,
                       int32_t *out_src, int32_t *out_local, int64_t *out_row_ptr,
                       int64_t *out_counts, void *scratch, size_t scratch_bytes, void *stream);

/* Fixed-stride (local id, weight) lists -> compact CSR arrays of the hop's block, which
 * grws_csr_to_bcsr_* turns into the BCSR block (this replaces build_col_to_val_map_kernel +
 * recompress_sampled_bcsr_kernel, core/include/sampling.cuh:471-579,707-773). */
int grws_block_compact(const int32_t *local, const float *w, int64_t n_dst, int fanout,
                       const int64_t *row_ptr, int32_t *out_col, float *out_val, void *stream);

/* ------------------------------------------------------------------------------------------
 * All hops of a mini-batch in one call: the hop loop of bcsr_sample_all_layers_wrapper
 * (core/wrapper/sampling_wrapper.cu:365-438) without its per-layer host synchronisation
 * (sampling_wrapper.cu:339-344).  Per hop h (fanouts are consumed in the order given): sample the
 * frontier as grws_sample_hop does, build the source list as grws_dedup_reindex does, build the
 * hop's BCSR block from the lists.  Every buffer is sized by a bound the host computes from
 * (num_seeds, fanouts, pad_to) alone -- grws_sample_layers_sizes -- so no size is read back:
 *   n_dst[0] = num_seeds, n_src[h] = roundup(n_dst[h] * (1 + fanout[h]), pad_to),
 *   n_dst[h+1] = n_src[h], tiles_bound[h] = n_dst[h]*fanout[h]/8 + ceil(n_dst[h]/16).
 * The frontier of hop h+1 is the whole source list of hop h, padding entries (-1) included: they
 * sample nothing and become rows without entries.  Outputs per hop h (arrays of num_hops host
 * pointers to device memory):
 *   out_src[h]           int32 [n_src[h]]   frontier ++ new nodes in ascending id order ++ -1
 *   out_window_offset[h] int64 [ceil(n_dst[h]/16) + 1]
 *   out_cols[h]          int32 [tiles_bound[h]*8], out_vals[h] [tiles_bound[h]*128] of val_dtype;
 *                        tiles past window_offset's last entry are empty (-1 / 0)
 *   out_counts           int64 [num_hops*4] or NULL: {source nodes incl. padded frontier entries,
 *                        sampled edges, tiles, real frontier nodes} per hop, for reporting
 * seed_dev, when not NULL, is a device uint64 read by the kernels instead of `seed` (a seed that
 * changes between replays of a captured launch sequence).
 * ------------------------------------------------------------------------------------------ */
int grws_sample_layers_sizes(int64_t num_seeds, const int *fanouts, int num_hops, int64_t pad_to,
                             int64_t *n_dst, int64_t *n_src, int64_t *tiles_bound);

size_t grws_sample_layers_scratch_bytes(int64_t num_seeds, const int *fanouts, int num_hops,
                                        int64_t pad_to);

int grws_sample_layers(const int64_t *row_ptr, const int32_t *col_idx, const float *values,
                       const int32_t *seeds, int64_t num_seeds, const int *fanouts, int num_hops,
                       uint64_t seed, const uint64_t *seed_dev, int64_t pad_to, int val_dtype,
                       int32_t *const *out_src, int64_t *const *out_window_offset,
                       int32_t *const *out_cols, void *const *out_vals, int64_t *out_counts,
                       void *scratch, size_t scratch_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * Rows of a feature matrix that is sharded over the GPUs of one node, read from their owners over
 * NVLink with plain loads.  Replaces the reference's placement of large feature matrices in pinned
 * host memory with a CPU-side gather per step (helper/engine.py:135-147,
 * data/data_loader.py:1513-1564).  Rank r owns rows [r * rows_per_shard, (r+1) * rows_per_shard);
 * `shards` is a DEVICE array of `world` pointers to the ranks' blocks, each addressable from this
 * GPU (peer-mapped or local), rows src_stride_bytes apart.  out[i] = row ids[i] (row_bytes each,
 * packed); ids[i] < 0 gives a zero row.  row_bytes and src_stride_bytes are multiples of 16.
 * ------------------------------------------------------------------------------------------ */
int grws_gather_rows_sharded(const void *const *shards, int world, int64_t rows_per_shard,
                             int64_t row_bytes, int64_t src_stride_bytes, const int32_t *ids,
                             int64_t n, void *out, void *stream);

/* ------------------------------------------------------------------------------------------
 * Global -> local column ids by window lookup, pruning misses.  Replaces reindex_bcsr_cuda +
 * reindex_and_prune_kernel (core/wrapper/reindex_wrapper.cu:27-68, core/include/reindex.cuh:
 * 33-102) with identical integer arithmetic: window = col / tile_rows (C division, so -1 maps
 * to window 0); hit -> rank * tile_rows + col % tile_rows; miss -> 0 and that column of the
 * tile's values zeroed in place.
 * ------------------------------------------------------------------------------------------ */
int grws_reindex_bcsr(const int32_t *in_cols, void *values, int val_dtype,
                      const int32_t *active_windows, int64_t num_indices, int64_t num_active,
                      int tile_rows, int tile_cols, int32_t *out_cols, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GRWS_B200_H */
