/* C ABI of the B200 implementation of the TP-invariant row-split path.
 *
 * One shared library (libtbik_b200.so) exports these entry points.  They take plain device
 * pointers, sizes and a CUDA stream; no torch types cross this boundary.  Every function
 * returns TBIK_OK (0) or a negative TBIK_ERR_* code and never throws; the message for the
 * last error of the calling thread is available from tbik_last_error().
 *
 * Each declaration names the reference interface it stands in for (paths are relative to the
 * reference project).
 */
#ifndef TBIK_H_
#define TBIK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ---------------------------------------------------------------------- */
#define TBIK_OK 0
#define TBIK_ERR_ARG (-1)    /* null pointer / bad handle / bad enum                         */
#define TBIK_ERR_SHAPE (-2)  /* sizes the path cannot take (K not a multiple of the leaf ...) */
#define TBIK_ERR_DTYPE (-3)  /* element type not supported                                    */
#define TBIK_ERR_ALIGN (-4)  /* pointer or stride alignment                                   */
#define TBIK_ERR_CUDA (-5)   /* a CUDA runtime / driver call failed                           */
#define TBIK_ERR_STATE (-6)  /* unregistered buffer, capacity exhausted, closed handle        */
#define TBIK_ERR_DEVICE (-7) /* a kernel gave up on a bounded wait and reported it            */

/* ---- element types --------------------------------------------------------------------- */
#define TBIK_DTYPE_BF16 0
#define TBIK_DTYPE_FP16 1
#define TBIK_DTYPE_FP32 2

/* Type of the tree nodes of the GEMM. */
#define TBIK_NODE_INPUT 0 /* nodes rounded to the operand type: the reference's arithmetic   */
#define TBIK_NODE_FP32 1  /* leaves and nodes stay fp32 (one fp32 add per node, same tree); C, of the operand type,
                             is the root rounded once                                                          */
#define TBIK_NODE_FP32_OUT_FP32 2 /* as above, but C is an fp32 matrix (ldc in fp32 elements) holding the unrounded
                             root: what a tensor-parallel rank hands to the cross-rank levels of the tree      */

typedef void* tbik_stream_t; /* a cudaStream_t */

/* Message of the last failing call made by this thread ("" if none). */
const char* tbik_last_error(void);

/* Library / ABI version: major * 1000 + minor. */
int tbik_version(void);

/* (T, F, L) of the reduction tree for a K extent and leaf width: T leaves, level 0 sums F
 * consecutive leaves, L levels in all (T = F * 2^(L-1)).
 * Replaces: src/tbik/tree_based_matmul.py:240-249 (TILE_K, FIRST_LEVEL_BLOCK, LEVEL_K). */
int tbik_tree_shape(int64_t K, int leaf, int* T, int* F, int* L);

/* C[M,N] = A[M,K] * W[N,K]^T with the K reduction done in the fixed tree order.
 *   A   row-major, row stride lda elements; W row-major [N,K] (the K-contiguous weight, i.e.
 *       the reference's B = weight.t() without the transpose), row stride ldw; C row stride ldc.
 *   dtype       TBIK_DTYPE_BF16 or TBIK_DTYPE_FP16 (operands and C)
 *   leaf        leaf width in elements, multiple of 64 (the reference uses 256)
 *   node_dtype  TBIK_NODE_INPUT: the reference's arithmetic (every node rounded to the operand type).
 *               TBIK_NODE_FP32 / TBIK_NODE_FP32_OUT_FP32: nothing is rounded below the root.  The tree (shape and
 *               order) is the same function of (K, leaf), so batch- and TP-invariance hold exactly as before, but the
 *               bits are not the reference's; accuracy against fp64 improves by an order of magnitude.  With fp32
 *               nodes the leaf may be long (K / 8, say): fewer accumulator drains.  The tree's stack then lives in
 *               tensor memory only: at most 3 levels on the full-rate 128-column tilings (7 / 15 on the 64- / 32-column
 *               ones), no K-slabs; deeper trees are refused -- use a wider leaf.
 * A and W must be 16-byte aligned with lda, ldw multiples of 8.  M == 0 or N == 0 is a no-op.
 * The kernel is enqueued on `stream`.  This entry point uses no scratch memory and allocates
 * nothing: it picks among the tilings whose tree stack fits on chip (128-column tiles: trees of up to
 * 7 levels, K <= 64 * 2 * leaf); deeper trees are rejected here and need tbik_gemm_ws.
 * Replaces: matmul_tp_persistent / matmul_kernel_tp_persistent,
 *           src/tbik/tree_based_matmul.py:50-187 and :190-274. */
int tbik_gemm(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
              int dtype, int leaf, int node_dtype, tbik_stream_t stream);

/* Scratch bytes tbik_gemm_ws wants for these sizes on the current device (0 if none).
 * No counterpart in the reference (its kernel keeps the whole stack in registers). */
size_t tbik_gemm_workspace_bytes(int M, int N, int64_t K, int leaf);

/* As tbik_gemm, with a caller-owned scratch buffer (16-byte aligned device memory, not shared with a
 * concurrently running call).  The buffer must be ZERO-FILLED ONCE before its first use (cudaMemset): its first
 * 16 KiB hold arrival counters that every completed call leaves at zero again, so the same buffer serves call
 * after call without further clearing; everything behind them may hold anything.  (If tbik_gemm_status ever
 * reports a kernel that gave up, clear the buffer again.)  The scratch serves the 256-column tilings (their
 * accumulators fill tensor memory, so the upper levels of the tree stack are kept in registers and shared memory
 * and, for levels touched at most once every four leaves, in this buffer), trees deeper than the on-chip stack,
 * and the K-slab roots of decode-sized calls (below).  With scratch the automatic choice at large M is the 256x256
 * CTA-pair tile (the fastest: a third less operand traffic per flop than 256x128); without it, 256x128.
 * Same bits as tbik_gemm.
 * Replaces: the same reference functions as tbik_gemm. */
int tbik_gemm_ws(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 int dtype, int leaf, int node_dtype, void* workspace, size_t workspace_bytes, tbik_stream_t stream);

/* K-slabs.  When C has too few tiles to give every SM one (decode-sized M), tbik_gemm_ws cuts K into 2, 4, 8 or 16
 * slabs, each a whole subtree of the reduction tree, and runs every (tile, slab) pair as its own work item of ONE
 * launch.  Slab s stores its subtree root in the workspace and counts its arrival at the tile; the CTA that arrives
 * last adds the roots pairwise in slab order in the element type and writes C (which CTA that is depends on timing,
 * the sum it forms does not).  That is the arithmetic the reference applies across tensor-parallel ranks
 * (per-rank tree of K / tp, then the rank-pair tree: src/tbik/tree_based_matmul.py:240-249 with
 * mini_allreduce/tbik_kernel/csrc/allreduce/custom_all_reduce.cuh:203-234), applied inside one GPU, so the bits do
 * not change.  tbik_gemm_workspace_bytes includes the room for the roots and the counters.  tbik_gemm_slabs runs one
 * explicit (tiling 1..6, slabs = power of two <= min(16, T / F)) combination so that tests can prove the invariance;
 * tbik_gemm_slabs_workspace_bytes gives its scratch need (0 for an invalid combination or when none is needed).
 * The functions themselves have no counterpart in the reference. */
size_t tbik_gemm_slabs_workspace_bytes(int M, int N, int64_t K, int leaf, int tiling, int slabs);
int tbik_gemm_slabs(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                    int dtype, int leaf, int node_dtype, int tiling, int slabs, void* workspace, size_t workspace_bytes,
                    tbik_stream_t stream);

/* The schedule tbik_gemm_ws would run for these sizes on the current device with `workspace_bytes` of scratch and
 * at most `max_ctas` CTAs (0 = one per SM): out[0] = tiling (codes of tbik_gemm_ex), out[1] = K-slabs, out[2] = CTAs,
 * out[3] = 1 if the variant with the deeper on-chip stack is used.  A function of the sizes only; nothing is
 * launched.  Without a visible GPU it answers for 148 SMs.  No counterpart in the reference. */
int tbik_gemm_plan(int M, int N, int64_t K, int leaf, int max_ctas, size_t workspace_bytes, int out[4]);

/* As tbik_gemm_ws, with the schedule exposed: at most `max_ctas` CTAs (0 = one per SM) and
 * `tiling` 0 = automatic, 1 = 128x128 tile per CTA, 2 = 256x128 per CTA pair, 3 = 128x256 per CTA,
 * 4 = 256x256 per CTA pair, 5 = 128x64 per CTA, 6 = 128x32 per CTA (an explicit tiling runs without K-slabs).
 * The result does not depend on either; the entry point exists so that
 * tests can prove that. */
int tbik_gemm_ex(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 int dtype, int leaf, int node_dtype, int max_ctas, int tiling, void* workspace,
                 size_t workspace_bytes, tbik_stream_t stream);

/* tbik_gemm_ws for callers that have no way to hand over device memory of their own: a host
 * runtime that binds this C ABI without a device allocator, or a serving engine that has already
 * given all free HBM to its KV cache, where a cudaMalloc at this point would fail or stall.  The
 * scratch is a fixed array inside the library image (tbik_gemm_static_scratch_bytes() bytes, 32 MiB;
 * each GPU that loads the library keeps it until the process exits).  The call performs no
 * allocation of any kind.  It runs the schedule tbik_gemm_ws would pick if that one's scratch fits the
 * array, else the best full-rate schedule that fits; sizes for which none fits (trees of more than about
 * twelve levels at thousands of rows) are refused with TBIK_ERR_SHAPE and a message naming both numbers.
 * Same bits as tbik_gemm_ws.
 * The first call on each device looks up the array's device address; make that first call outside
 * any stream capture (two host threads may race on it harmlessly: both find the same address).  All
 * calls on a device share the one array, so two calls that can overlap on the GPU (different streams)
 * race on it -- serialise them.  The array keeps whatever the previous call left behind.  What must
 * start at zero are the arrival counters at its head: they are zero when the library is loaded and
 * every completed call puts them back to zero.  Everything else is written before it is read within a
 * call (the rows of K-slab roots are padded to a multiple of 8 columns and the pad is written too).
 * This entry point has no counterpart in the reference. */
int tbik_gemm_static(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                     int dtype, int leaf, int node_dtype, tbik_stream_t stream);

/* Capacity in bytes of the scratch built into the library for tbik_gemm_static.
 * No counterpart in the reference. */
size_t tbik_gemm_static_scratch_bytes(void);

/* 1 if tbik_gemm_static would run these sizes on the current device, 0 if it would refuse them (a question
 * about sizes only: nothing is launched, no pointer is needed).  No counterpart in the reference. */
int tbik_gemm_static_accepts(int M, int N, int64_t K, int leaf);

/* Reads (and clears) the device-side status of the GEMM kernels on the current device:
 * out[0] != 0 means a kernel gave up on a bounded wait (out[1] = block, out[2] = role).
 * out[3] = SM clock cycles CTA 0 of the most recent launch spent in its main loop (for utilisation
 * figures that do not depend on the clock the GPU happened to run at).  Synchronises with the device.  No counterpart in the reference (its waits are unbounded). */
int tbik_gemm_status(uint32_t out[4]);

/* ---- cross-GPU all-reduce over IPC-registered buffers --------------------------------------- */
typedef void* tbik_ar_t;

/* Keys of tbik_ar_configure. */
#define TBIK_AR_CFG_SCRATCH_BYTES 1     /* bytes available after the signal area of each meta buffer */
#define TBIK_AR_CFG_ONESHOT_MAX_BYTES 2 /* messages up to this size use the one-shot schedule (0 = built-in) */
#define TBIK_AR_CFG_MAX_BLOCKS 3        /* upper bound on CTAs per launch (0 = built-in)               */
#define TBIK_AR_CFG_WAIT_LIMIT_NS 4     /* bound of one cross-GPU barrier wait                          */
#define TBIK_AR_CFG_THREADS 5           /* threads per CTA, a multiple of 32 in [32, 512] (0 = built-in) */
#define TBIK_AR_CFG_PUSH_MIN_BYTES 6    /* messages from this size on use the push schedule (0 = built-in, 1 = all two-shot sizes) */
#define TBIK_AR_CFG_PUSH_CHUNKS 7       /* chunks the push schedule cuts a message into, 1..64 (0 = built-in) */
#define TBIK_AR_CFG_VEC_PACKS 8         /* 16-byte packs per load / store instruction: 1, or 2 = 256-bit accesses (0 = built-in) */
#define TBIK_AR_CFG_LOADS_IN_FLIGHT 9   /* 16-byte packs a thread requests before it uses the first, 1..32 (0 = built-in) */
#define TBIK_AR_CFG_CLUSTER_PAIRS 11     /* 1 (default): CTAs are launched as clusters of two, so that beside a GEMM made of CTA pairs the all-reduce takes whole SM pairs; 0: plain launch */
#define TBIK_AR_CFG_TRACE 10            /* 1: every launch records per-CTA phase time stamps (tbik_ar_trace); 0: off      */

/* Size in bytes of the signal (flag) area at the start of every rank's meta buffer.
 * Replaces: meta_size, mini_allreduce/tbik_kernel/csrc/allreduce/custom_all_reduce.cu:148-150. */
size_t tbik_ar_meta_size(void);

/* Creates a communicator.  signals[i] = address, in this process, of rank i's meta buffer (signal
 * area followed by scratch), zero-filled by its owner before the addresses were exchanged.
 * rank_data = caller-owned device table (64 bytes per registered buffer).  The object owns no
 * device memory.  world must be 1, 2, 4, 6 or 8.
 * Replaces: init_custom_ar, custom_all_reduce.cu:14-27 and the CustomAllreduce constructor,
 *           custom_all_reduce.cuh:360-373. */
int tbik_ar_create(void* const* signals, int world, int rank, void* rank_data, size_t rank_data_bytes,
                   int full_nvlink, tbik_ar_t* out);

/* Replaces: dispose, custom_all_reduce.cu:144-146 (closes the IPC handles the object opened). */
int tbik_ar_destroy(tbik_ar_t comm);

/* Tuning / capacity knobs (see TBIK_AR_CFG_*).  No counterpart in the reference, whose limits are
 * compile-time constants (custom_all_reduce.cuh:20, 494-506). */
int tbik_ar_configure(tbik_ar_t comm, int key, int64_t value);

/* Registers one buffer: ptrs[i] = address, in this process, of rank i's copy.
 * Replaces: register_buffer, custom_all_reduce.cu:152-160 / custom_all_reduce.cuh:411-420. */
int tbik_ar_register_buffer(tbik_ar_t comm, void* const* ptrs);

/* out = tree-sum over ranks of inp, ((0+1)+(2+3))+((4+5)+(6+7)), adds in the element type.
 * If reg_buffer != NULL, inp is first copied (on `stream`) into reg_buffer, which must be a
 * registered buffer of at least numel*elsize bytes; otherwise inp itself must be registered (or
 * the stream is capturing, in which case inp is queued for tbik_ar_register_graph_buffers).
 * numel*elsize must be a multiple of 16.  Collective: every rank calls it in the same order.
 * Replaces: tree_all_reduce, custom_all_reduce.cu:100-142 / tree_allreduce, custom_all_reduce.cuh:523-573. */
int tbik_ar_tree_allreduce(tbik_ar_t comm, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer,
                           size_t reg_buffer_bytes, tbik_stream_t stream);

/* Tree all-reduce of a message that a producer kernel wrote IN PLACE inside a registered buffer: the message is
 * the numel elements that start byte_offset bytes into the buffer registered at reg_base (same offset on every
 * rank; a multiple of 16).  No staging copy.  This is how the row-split layer overlaps its two halves: the GEMM
 * writes row blocks of its partial result into the registered buffer, and each block is reduced, on a second
 * stream, while the GEMM computes the next one.
 * Replaces: the same reference functions as tbik_ar_tree_allreduce, minus the copy at custom_all_reduce.cu:112-114. */
int tbik_ar_tree_allreduce_within(tbik_ar_t comm, const void* reg_base, size_t byte_offset, void* out, int64_t numel,
                                  int dtype, tbik_stream_t stream);

/* Tree all-reduce of fp32 contributions with ONE rounding at the end: out[numel] (out_dtype: TBIK_DTYPE_BF16 or
 * TBIK_DTYPE_FP16, 16-byte aligned) = round(rank-pair tree sum, in fp32, of every rank's numel floats at
 * reg_base + byte_offset).  It finishes a tree whose nodes stay fp32 (tbik_gemm_ex with TBIK_NODE_FP32_OUT_FP32
 * writes each rank's subtree root there): same tree as the TP = 1 launch with TBIK_NODE_FP32, hence the same bits.
 * reg_base must be a registered buffer (tbik_ar_register_buffer); byte_offset a multiple of 32; numel a multiple
 * of 8.  Collective.  No counterpart in the reference, whose nodes are always rounded to the operand type. */
int tbik_ar_tree_allreduce_rounding(tbik_ar_t comm, const void* reg_base, size_t byte_offset, void* out, int64_t numel,
                                    int out_dtype, tbik_stream_t stream);

/* The row-split layer as a pipeline: out[M, N] (contiguous) = tree-all-reduce over ranks of (A * W^T), computed
 * block of rows by block of rows.  Block i's GEMM (tbik_gemm_ws arithmetic) writes its partial rows into the
 * registered buffer at reg_base on `main_stream`; its tree all-reduce runs on `side_stream` with at most
 * `comm_ctas` CTAs while the GEMM of block i + 1 occupies the other SMs; the layer's last all-reduce gets the
 * whole GPU.  The call enqueues everything (kernels, event records and waits) and returns; `main_stream` ends
 * up waiting for the last all-reduce, so work enqueued on it afterwards sees the complete result.  Cutting
 * the rows into blocks cannot change a bit: no sum ever joins two rows.  block_rows[0 .. num_blocks) are the
 * rows of each block (they add up to M; multiples of 256 keep the GEMM tiles whole; a short last block keeps the
 * one all-reduce that nothing hides short).  Collective: every rank calls it in the same order with the same sizes.  Not
 * for use under stream capture.
 * Replaces: the sequence matmul_tp_persistent -> tree_all_reduce_sum in the patched forward,
 *           src/patch/patch_tp_invariant.py:31-34 (and the staging copy at custom_all_reduce.cu:112-114). */
int tbik_ar_row_split_layer(tbik_ar_t comm, const void* A, const void* W, void* out, int M, int N, int K, int64_t lda,
                            int64_t ldw, int dtype, int leaf, void* reg_base, size_t reg_bytes, void* workspace,
                            size_t workspace_bytes, const int* block_rows, int num_blocks, int comm_ctas,
                            tbik_stream_t main_stream, tbik_stream_t side_stream);

/* As above with the non-tree arithmetic: fp32 accumulation in rank order, one final rounding.
 * Replaces: all_reduce, custom_all_reduce.cu:57-98 / allreduce, custom_all_reduce.cuh:462-521. */
int tbik_ar_allreduce(tbik_ar_t comm, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer,
                      size_t reg_buffer_bytes, tbik_stream_t stream);

/* CUDA-graph support: inputs seen while a stream was capturing wait for their peers' addresses.
 * _count gives their number n; _meta writes n IPC handles (64 bytes each) and n offsets;
 * _register_graph_buffers takes, per rank, that rank's handles and offsets and fills the slots.
 * Replaces: get_graph_buffer_ipc_meta / register_graph_buffers, custom_all_reduce.cu:162-181 and
 *           custom_all_reduce.cuh:384-451. */
int tbik_ar_graph_meta_count(tbik_ar_t comm, int* n);
int tbik_ar_graph_meta(tbik_ar_t comm, void* handles_out, int64_t* offsets_out);
int tbik_ar_register_graph_buffers(tbik_ar_t comm, const void* const* handles, const int64_t* const* offsets);

/* Host-visible status of the communicator's kernels, readable at any time without synchronising:
 * out[0] 0 = healthy, 1 = a barrier wait ran out; out[1..6] = rank, block, peer, expected epoch,
 * value seen, barrier id.  No counterpart in the reference (custom_all_reduce.cuh:182,186 spin forever). */
int tbik_ar_status(tbik_ar_t comm, uint32_t out[8]);

/* Phase time stamps of the most recent all-reduce launch (needs TBIK_AR_CFG_TRACE = 1; synchronise the stream
 * first): for each of its CTAs eight GPU-timer values in nanoseconds -- [0] kernel entry, [1] after the first
 * cross-GPU barrier, [2] after the reduce phase, [3] after the middle barrier (two-shot only), [4] exit.  `out`
 * has room for 8 * max_blocks values; *blocks receives the number of CTAs recorded.  This is how the phases of a
 * multi-rank kernel are timed without a profiler.  No counterpart in the reference. */
int tbik_ar_trace(tbik_ar_t comm, uint64_t* out, int max_blocks, int* blocks);

#ifdef __cplusplus
}
#endif
#endif /* TBIK_H_ */
