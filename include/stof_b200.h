/*
 * stof_b200 -- C ABI of the B200 (sm_100a) kernels behind the STOF operator API.
 *
 * Every entry point takes plain device pointers, sizes, element strides and a CUDA
 * stream (passed as void*, a cudaStream_t; NULL = the legacy default stream).  The
 * caller owns every buffer.  Functions return 0 on success and a negative STOF_E_*
 * code otherwise; `stof_last_error()` then holds a message for the calling thread.
 * Nothing here aborts the process or traps the GPU.  Kernels that wait on hardware
 * barriers do so with a cycle budget and report through `status_dev` (a device int
 * the caller zero-initialises; 0 = ok, otherwise (barrier id << 8) | code).
 *
 * "Replaces" comments cite the interface of the reference implementation
 * (AD-pap899-SC25/SC25-STOF-AD, paths relative to its root) that an entry point stands in for.
 */
#ifndef STOF_B200_H
#define STOF_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STOF_OK 0
#define STOF_E_INVALID (-1)   /* bad argument (shape, alignment, null pointer, unsupported block size) */
#define STOF_E_CUDA (-2)      /* a CUDA runtime / driver call failed */
#define STOF_E_WORKSPACE (-3) /* workspace too small */
#define STOF_E_LIMIT (-4)     /* size beyond a stated maximum */

#define STOF_DTYPE_F16 0
#define STOF_DTYPE_F32 1

/* Library version (major*100 + minor) and the last error text of the calling thread. */
int stof_version(void);
const char* stof_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Mask -> block index compaction.
 * Replaces: get_sparse_storage(Mask, block_size_m, block_size_n), src/util/masks.py:125-184.
 *
 * Two phases, because the sizes of the outputs depend on the data:
 *   1. stof_mask_classify  : classifies every (block_m x block_n) tile of mask[0] as full / empty /
 *      partial, counts the non-zero elements of the WHOLE (batch, S, S) tensor, and writes the
 *      three row-pointer arrays.  `counts` (device, 4 x int64) receives
 *      {n_full, n_part, n_load, nnz_elements}.
 *   2. stof_mask_fill      : writes the column indices (ascending inside a row, `load` = merge of
 *      full and partial) and gathers the partial tiles as -10000 * (1 - m) in fp16.
 * `workspace` is scratch shared by both phases (size from stof_mask_workspace_bytes) and must stay
 * untouched between them.  mask_dtype is STOF_DTYPE_F16 or STOF_DTYPE_F32; the mask is a dense
 * row-major (batch, S, S) array; S must be a multiple of block_m and of block_n, block_n a multiple
 * of 8.  Index outputs are int32.
 * ------------------------------------------------------------------------------------------ */
size_t stof_mask_workspace_bytes(int seq_len, int block_m, int block_n);

int stof_mask_classify(const void* mask, int mask_dtype, int batch, int seq_len, int block_m, int block_n,
                       int* full_row_ptr, int* part_row_ptr, int* load_row_ptr, /* each S/block_m + 1 */
                       long long* counts, void* workspace, size_t workspace_bytes, void* stream);

int stof_mask_fill(const void* mask, int mask_dtype, int seq_len, int block_m, int block_n,
                   const int* full_row_ptr, const int* part_row_ptr, const int* load_row_ptr,
                   int* full_col_idx, int* part_col_idx, int* load_col_idx,
                   void* part_block_mask, /* fp16 (n_part, block_m, block_n); may be NULL when n_part == 0 */
                   const void* workspace, size_t workspace_bytes, void* stream);

/* Mask compaction for callers that must not allocate.
 * No counterpart in the reference: its get_sparse_storage builds Python lists and allocates freely.
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they need the block index: code
 * that runs between a framework's allocator hooks, a plugin callback that is only handed its inputs and
 * outputs, a latency-critical serving loop that has frozen its memory pool.  For them this single call
 * does both phases of the compaction with the scratch (one class byte per tile plus a 16-byte header)
 * in an array that is part of the library's device image instead of a workspace argument.  It calls no
 * cudaMalloc / cudaFree and no allocating library routine; the caller passes every input and output.
 *
 * Limits and rules:
 *  - (S / block_m) * (S / block_n) must not exceed 1,048,576 tiles (1 MiB of scratch; STOF_E_LIMIT
 *    otherwise -- fall back to stof_mask_classify / stof_mask_fill with your own workspace).  Each GPU
 *    that loads the library keeps that 1 MiB + 16 bytes resident until the process exits.
 *  - The outputs are sized by the caller before the counts are known: the three column-index arrays hold
 *    `col_capacity` entries each and `part_block_mask` holds `part_capacity` tiles; entries beyond a
 *    capacity are dropped, and `counts` ({n_full, n_part, n_load, nnz_elements}, device) tells the caller
 *    afterwards whether anything was.  Capacities of (S/block_m)*(S/block_n) never drop anything.
 *  - The first call on a device looks up the array's device address (one runtime query, cached per device).
 *    With the CUDA runtime's lazy module loading that query can be the moment the runtime loads the library's
 *    device image - the 1 MiB array included - onto that device, so this one call may take device memory and
 *    time that later calls do not; make it during set-up and outside any stream capture.  The cached address
 *    belongs to the device's primary context: after cudaDeviceReset() on that device it is stale and the entry
 *    point must not be used again in that process.
 *  - All calls share the one array and it keeps the previous call's bytes.  The call clears what has to
 *    start at zero itself, but two calls whose kernels overlap on the GPU (different streams, or several
 *    host threads) race on it: serialise them. */
int stof_mask_compact_static(const void* mask, int mask_dtype, int batch, int seq_len, int block_m, int block_n,
                             int* full_row_ptr, int* part_row_ptr, int* load_row_ptr,
                             int* full_col_idx, int* part_col_idx, int* load_col_idx, long long col_capacity,
                             void* part_block_mask, long long part_capacity,
                             long long* counts, void* stream);

/* ------------------------------------------------------------------------------------------
 * Block-masked multi-head attention, fp16 in / fp16 out, fp32 accumulation, head_dim 64.
 * Replaces: launch_block_attn_mask(...), src/ops/src/block_attn_mask_cuda.cu:6026-6316, as bound by
 *           block_attn_mask_gpu, src/ops/src/block_attn_mask.cpp:17-49.
 *
 * Two calls.  stof_block_attn_plan turns the block index (the full_* and part_* lists of
 * get_sparse_storage) into the kernel's own tiling.  A work item is a pair of 64-row halves of the
 * sequence (halves 2t and 2t + 1), each of which walks its own list of 64-wide key tiles - the tiles any
 * of its row blocks lists; the plan lays the two lists out step by step (tiles both halves list share a
 * step), with a code per 16 x 16 group and step (absent / full / partial tile i) and the order in which
 * the scheduler visits the items.  It depends on the index only, so one plan serves every call with that
 * index (every layer of an encoder).  The plan buffer is caller-owned scratch of
 * stof_block_attn_plan_bytes() bytes; the kernel checks that a plan was made for the sequence length and
 * block shape it is launched with and reports another one through status_dev.
 * stof_block_attn runs the attention.  For each row block only the listed column blocks take part; a
 * partial block adds its fp16 tile to the unscaled scores before the softmax scale, as the reference
 * kernel does.  A row without any listed key yields zeros.  `out` may alias `q` (the reference
 * overwrites q): an item's query rows are read completely before they are written.
 * Strides are in elements for (batch, head, row); the innermost (head_dim) stride is 1.  All base
 * pointers 16-byte aligned, strides multiples of 8 elements.  block_m, block_n in {16,32,64,128};
 * seq_len a multiple of both.  `num_warps` is accepted for signature compatibility and ignored.
 * ------------------------------------------------------------------------------------------ */
size_t stof_block_attn_plan_bytes(int seq_len, int block_m, int block_n);

int stof_block_attn_plan(const int* full_row_ptr, const int* full_col_idx,
                         const int* part_row_ptr, const int* part_col_idx,
                         int seq_len, int block_m, int block_n,
                         void* plan, size_t plan_bytes, int* status_dev, void* stream);

/* The same plan with the work items put together by the caller.  No counterpart in the reference
 * (its kernel works on one BLOCK_M row block per thread block).  Here `pairs` (device, 2 ints per item,
 * ceil(seq_len / 128) items) names the two 64-row halves of every item by their index seq_row / 64; the
 * second may be -1.  The two halves of an item work side by side, each on its own key tiles, so an item
 * takes as many steps as its longer list and loads every tile either half lists: a caller pairs halves
 * with equally long lists and, among those, halves whose lists agree (rows r and r + 2 of a dilated
 * mask, say).  Every half must appear in exactly one item: a half that is left out is never written,
 * which the plan does not check; an index outside [0, ceil(seq_len / 64)) sets *status_dev and the item
 * falls back to half 0 alone. */
int stof_block_attn_plan_paired(const int* full_row_ptr, const int* full_col_idx,
                                const int* part_row_ptr, const int* part_col_idx, const int* pairs,
                                int seq_len, int block_m, int block_n,
                                void* plan, size_t plan_bytes, int* status_dev, void* stream);

int stof_block_attn(const void* q, const void* k, const void* v, void* out,
                    int batch, int heads, int seq_len, int head_dim,
                    const long long q_strides[3], const long long k_strides[3],
                    const long long v_strides[3], const long long out_strides[3],
                    const int* part_row_ptr, const void* part_block_mask, const void* plan,
                    int block_m, int block_n, int num_warps, float softmax_scale,
                    int* status_dev, void* stream);

/* stof_block_attn with the deal of the work items to the thread blocks given by the caller.  No counterpart in the
 * reference (its kernels take one 64-row block per thread block from the launch grid,
 * src/ops/src/block_attn_mask_cuda.cu:6026-6316); here the kernel is persistent and a work item is one pair of 64-row halves
 * of one (batch, head).  By default the items are dealt round-robin, heaviest first; items with very different step counts
 * then leave some blocks with up to 10-20 % more steps than the average.  `schedule` (device, int32) lets the host balance
 * them, e.g. by a longest-processing-time assignment over the per-item step counts that the plan holds
 * (stof_b200/attention.py: attention_schedule):
 *   schedule[0] = G (thread blocks, 1 <= G <= 2 x SMs), schedule[1 .. G + 1] = offsets, then the item ids,
 *   id = (batch_index * heads + head_index) * ceil(seq_len / 128) + item_of_the_plan; block b works through
 *   ids[offset[b] .. offset[b + 1]) in that order.  Every item must appear exactly once (items left out are not computed).
 * `schedule_blocks` repeats G for validation on the host. */
int stof_block_attn_scheduled(const void* q, const void* k, const void* v, void* out,
                              int batch, int heads, int seq_len, int head_dim,
                              const long long q_strides[3], const long long k_strides[3],
                              const long long v_strides[3], const long long out_strides[3],
                              const int* part_row_ptr, const void* part_block_mask, const void* plan,
                              int block_m, int block_n, int num_warps, float softmax_scale,
                              const int* schedule, int schedule_blocks,
                              int* status_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * GEMM with fused epilogue: C[M,N] = epilogue(A[M,K] @ W[K,N] + bias[N]), fp16 in/out, fp32 accumulate.
 * Replaces: the Triton templates of src/triton_template/ (gemm_add_layernorm.py:77-144,
 *           gemm_gemm.py:99-174) and the cuBLAS + elementwise sequences of src/benchmk_end2end.py:73-86.
 *
 * A row-major with row stride lda, W row-major (K rows) with row stride ldw, C row-major with row
 * stride ldc; all in elements, multiples of 8; pointers 16-byte aligned; K, N multiples of 8.
 * epilogue: STOF_EPI_BIAS, _GELU_ERF, _GELU_TANH, _RESIDUAL (adds residual[M,N], row stride ldr), _RELU
 * (max(x, 0): the FFN activation of the T5 loops, src/benchmk_end2end.py:203,313).
 * bias may be NULL.
 * Two kernels serve the call: shapes with at least two 256 x 256 tiles per pair of multiprocessors run on
 * pairs of thread blocks (tcgen05 cta_group::2, clusters of two), smaller ones - and residual epilogues with
 * K <= 1024 below 16 such tiles per pair - on single blocks with 128 x 256 tiles; the results agree within
 * fp16 rounding.  The
 * environment variable STOF_B200_GEMM_PAIR = 0 / 1, read once per process, forces one of the two
 * (a testing aid).  GELU_ERF evaluates x * Phi(x) with a polynomial (|error| < 1.1e-4).
 * ------------------------------------------------------------------------------------------ */
#define STOF_EPI_BIAS 0
#define STOF_EPI_BIAS_GELU_ERF 1
#define STOF_EPI_BIAS_GELU_TANH 2
#define STOF_EPI_BIAS_RESIDUAL 3
#define STOF_EPI_BIAS_RELU 4

int stof_gemm_bias_act(const void* a, long long lda, const void* w, long long ldw, const void* bias,
                       const void* residual, long long ldr, void* c, long long ldc,
                       int m, int n, int k, int epilogue, int* status_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * GEMM with the LayerNorm in its epilogue:  c = LN(a @ w + bias + residual) * gamma + beta, rows normalised over
 * all n columns (biased variance, fp32 statistics taken on the fp32 sums, before any rounding to fp16).
 * Replaces: triton_matmul_bias_layernorm, src/triton_template/gemm_add_layernorm.py:77-144 (statistics inside the
 *           GEMM kernel), and matmul + bias + residual + F.layer_norm of src/benchmk_end2end.py:73-76, 83-86.
 * bias, residual, gamma, beta may be NULL (0 / 0 / 1 / 0).  For n a multiple of 256 up to 1024 and k <= 2048
 * this is ONE kernel (the n / 256 thread blocks of a row block form a cluster and exchange row statistics
 * through distributed shared memory); other shapes run stof_gemm_bias_act followed by
 * stof_bias_residual_layernorm in place (for long contractions that is the faster of the two, measured).
 * ------------------------------------------------------------------------------------------ */
int stof_gemm_bias_residual_layernorm(const void* a, long long lda, const void* w, long long ldw, const void* bias,
                                      const void* residual, long long ldr, const void* gamma, const void* beta, float eps,
                                      void* c, long long ldc, int m, int n, int k, int* status_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * Row LayerNorm with fused bias / residual add:  y = LN(x + bias + residual) * gamma + beta.
 * Replaces: triton_batched_bias_layernorm, src/triton_template/add_layernorm.py:19-107, and the
 *           normalisation half of triton_matmul_bias_layernorm (gemm_add_layernorm.py:113-123).
 * x, residual, y: (rows, hidden) fp16 with row strides in elements; bias/gamma/beta: fp16 (hidden) or
 * NULL (0 / 1 / 0).  Statistics in fp32, biased variance.  hidden a multiple of 8, at most 8192.
 * status_dev (device int, may be NULL): a warp whose row copy does not arrive within the wait budget writes
 * a STATUS_WAIT_TIMEOUT code there and leaves its remaining rows unwritten.
 * ------------------------------------------------------------------------------------------ */
int stof_bias_residual_layernorm(const void* x, long long ldx, const void* bias, const void* residual, long long ldr,
                                 const void* gamma, const void* beta, float eps, void* y, long long ldy,
                                 int rows, int hidden, int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STOF_B200_H */
