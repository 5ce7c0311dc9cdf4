/*
 * flash_colreduce_b200 -- C ABI of the sm_100a column-reduction library.
 *
 * The library computes, for queries Q (B,H,M,D) and keys K (B,H,N,D),
 *
 *     P[b,h,i,:] = softmax_j( Q[b,h,i,:] . K[b,h,j,:] * scale  (+ right-aligned causal mask) )
 *     R[b,h,j]   = reduce_i P[b,h,i,j]            reduce in {sum, mean, max}
 *
 * without materialising the (B,H,M,N) matrix.  Every entry point takes plain
 * pointers and sizes; device pointers are raw CUDA addresses, `stream` is a
 * `cudaStream_t` passed as `void*`.  All launches are asynchronous on that
 * stream and the library never synchronises, except where a function says so.
 *
 * Every function returning `int` returns an fcr_status; a human-readable
 * message for the calling thread's last failure is available from
 * fcr_last_error().  No C++ exception crosses this boundary.
 *
 * Reference interfaces replaced (paths inside z-lab/flash-colreduce v0.2.2):
 *   flash_colreduce/flash.py:277-308  `_flash_colreduce`   -> fcr_colreduce
 *   flash_colreduce/flash.py:144-274  `_flash_colreduce_kernel` (Triton) -> the kernels behind fcr_colreduce
 *   flash_colreduce/flash.py:377-385  mean divisor + cast  -> fused into fcr_colreduce; fcr_finalize for sharded runs
 */
#ifndef FLASH_COLREDUCE_B200_H_
#define FLASH_COLREDUCE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fcr_status {
  FCR_OK = 0,
  FCR_ERR_BAD_ARG = 1,        /* null pointer, negative size, inconsistent problem */
  FCR_ERR_UNSUPPORTED = 2,    /* shape / dtype / stride the sm_100a kernels cannot take */
  FCR_ERR_WORKSPACE = 3,      /* workspace missing, misaligned or smaller than fcr_workspace_bytes() */
  FCR_ERR_DEVICE_TIMEOUT = 4, /* a bounded device-side wait expired; see fcr_read_device_status */
  FCR_ERR_CUDA = 5,           /* a CUDA runtime / driver call failed */
  FCR_ERR_NCCL = 6            /* NCCL could not be loaded or one of its calls failed */
} fcr_status;

typedef enum fcr_dtype { FCR_F16 = 0, FCR_BF16 = 1, FCR_F32 = 2 } fcr_dtype;
typedef enum fcr_reduction { FCR_SUM = 0, FCR_MEAN = 1, FCR_MAX = 2 } fcr_reduction;

/*
 * One column-reduction problem.  Strides are in ELEMENTS, in (B,H,rows,D)
 * order, exactly the four numbers `tensor.stride()` returns; the innermost
 * stride must be 1 and the other three must be multiples of 16 bytes (8
 * 16-bit or 4 fp32 elements) -- a TMA tensor-map requirement.
 *
 * Replaces the argument list of `_flash_colreduce_kernel`
 * (flash_colreduce/flash.py:145-167: pointers, scale, eight strides, H, M, N,
 * D, REDUCTION, CAUSAL).
 */
typedef struct fcr_problem {
  int32_t B, H, M, N, D;
  int64_t q_strides[4];
  int64_t k_strides[4];
  int32_t in_dtype;      /* fcr_dtype of q and k: FCR_F16, FCR_BF16 (D <= 256) or FCR_F32 (D <= 128, multiplied as TF32) */
  int32_t reduction;     /* fcr_reduction */
  int32_t is_causal;     /* 0 / 1 */
  float scale;           /* softmax scale applied to q.k (the reference's default is 1/sqrt(D)) */
  /*
   * Causal alignment: query row i attends keys j <= i + causal_offset.
   * A negative value selects the reference's right alignment max(N - M, 0)
   * (flash_colreduce/flash.py:202, naive.py:21).  A row-sliced shard of a
   * larger problem passes the offset of its first row explicitly.
   */
  int64_t causal_offset;
  /*
   * Divisor rule for FCR_MEAN (flash_colreduce/flash.py:377-384): the rule is
   * evaluated with these "whole problem" row/key counts.  0 selects M / N of
   * this problem.
   */
  int32_t mean_M, mean_N;
} fcr_problem;

/* Launch plan derived on the host from a problem and an SM count. */
typedef struct fcr_plan {
  int32_t d_pad;            /* row width the kernels run at, in 2-byte units: 64, 128 or 256 (zero-filled by TMA) */
  int32_t rows_per_block;   /* stationary rows a CTA owns: 256 */
  int32_t m_pad, n_pad;     /* M and N rounded up to 128 */
  int32_t row_blocks;       /* rows pass: blocks of 256 query rows per head */
  int32_t col_blocks;       /* columns pass: blocks of 256 key columns per head */
  int32_t row_splits;       /* rows pass: splits of the key range per row block */
  int32_t col_splits;       /* columns pass: splits of the query range per column block */
  int32_t row_items, col_items; /* work items per pass = B*H*blocks*splits */
  int32_t row_ctas, col_ctas;   /* persistent CTAs launched per pass */
  int32_t head_group;       /* heads whose work items are interleaved (causal: evens out the tail of the grid) */
  int32_t short_items;      /* bit 0 / 1: the rows / columns pass uses the buffering for items of few tiles */
  int64_t causal_offset;    /* resolved offset */
  int64_t valid_scores;     /* B*H*sum_i valid(i): the unit the throughput metric counts */
  /* workspace layout, byte offsets from the workspace base */
  int64_t off_status;       /* int32[256] device status words (word 0: first failure code) */
  int64_t off_neg_lse;      /* float[B*H][m_pad]: minus the base-2 log-sum-exp of each query row */
  int64_t off_part_m;       /* float[row_splits][B*H][m_pad] running maxima (row_splits > 1) */
  int64_t off_part_l;       /* float[row_splits][B*H][m_pad] running sums   (row_splits > 1) */
  int64_t off_part_out;     /* float[col_splits][B*H][n_pad] column partials (col_splits > 1) */
  int64_t workspace_bytes;
  /* Key streaming (M <= 128 and at least 8 key tiles, the decode shapes): both passes keep the one
   * query tile of a head in shared memory and stream its key tiles through a deep ring.  The key
   * tiles of a head are cut into key_chunks equal chunks, one work item each; the rows pass leaves
   * row_splits = 4 * key_chunks partial (max, sum) states per row, the columns pass none. */
  int32_t key_stream;       /* 1 when the key-streaming kernels run this problem */
  int32_t key_chunks;       /* work items per head and pass */
  /* Score cache (key streaming with M <= 16): the rows pass also writes the raw fp32 scores, 4*M bytes
   * per key against the 2*D bytes of the key itself, and the columns are reduced from that array by
   * a plain kernel instead of a second sweep over K: the keys are read from HBM once. */
  int64_t off_scores;       /* float[B*H][M][n_pad] raw scores Q.K^T (score_cache only); the last region of the
                             * workspace and optional: a workspace of only off_scores bytes is accepted, the
                             * columns pass then sweeps K a second time */
  int32_t score_cache;      /* 1 when the columns are reduced from cached scores */
  int32_t static_schedule;  /* 1: work items are dealt round-robin (item, item + CTAs, ...) and nothing in the workspace has
                             * to be cleared before the kernels (small problems and the key-streaming kernels);
                             * 0: CTAs draw items from a counter, which one cudaMemsetAsync per call clears */
} fcr_plan;

/* Library version string, e.g. "0.1.0". */
const char* fcr_version(void);

/* Message describing the last failure on the calling thread ("" if none). */
const char* fcr_last_error(void);

/*
 * Pure host function: validates `problem` and fills `plan` for a device with
 * `num_sms` streaming multiprocessors (pass 0 to query the current CUDA
 * device).  Replaces the grid computation of flash_colreduce/flash.py:287.
 */
int fcr_plan_problem(const fcr_problem* problem, int32_t num_sms, fcr_plan* plan);

/*
 * Pure host function: decodes work item `item` of pass 1 (rows pass: Q tiles
 * stationary, K tiles streamed) or pass 2 (columns pass: K tiles stationary,
 * Q tiles streamed) with the same routine the kernels run.  out[10] receives
 * {head, split, chunk_lo, chunk_hi, row0_a, tile_lo_a, tile_hi_a, row0_b,
 * tile_lo_b, tile_hi_b}: 128-row streamed tiles [tile_lo, tile_hi) are
 * multiplied against the stationary tile starting at row0.  This is the
 * counterpart of the per-program loop bounds of flash_colreduce/flash.py:201-207.
 * For a key-streaming plan both passes report {head, chunk, key_tile_lo,
 * key_tile_hi, 0, key_tile_lo, key_tile_hi, m_pad, key_tile_lo, key_tile_lo}:
 * key tiles [lo, hi) of the head against its single query tile; tile t of the
 * item is folded by warpgroup (t - key_tile_lo) mod 4, and the rows pass
 * stores that warpgroup's state in partial slot 4 * chunk + warpgroup.
 */
int fcr_plan_item(const fcr_problem* problem, const fcr_plan* plan, int32_t pass, int32_t item,
                  int32_t* out);

/*
 * Bytes of device workspace fcr_colreduce needs for `problem` (0 on error).
 * The reference allocates its fp32 accumulator itself
 * (flash_colreduce/flash.py:286); here the caller owns every allocation.
 */
size_t fcr_workspace_bytes(const fcr_problem* problem, int32_t num_sms);

/*
 * The operator.  q, k: device pointers to the first element of the (B,H,*,D)
 * tensors described by `problem`.  out: device pointer to a contiguous
 * (B,H,N) tensor of `out_dtype`.  workspace: device memory, 256-byte aligned,
 * at least fcr_workspace_bytes() long; its contents need not be initialised.
 * Results are deterministic: no atomics, fixed summation order.
 *
 * With reduction == FCR_MEAN the divisor of flash_colreduce/flash.py:377-384
 * is applied in fp32 before the single rounding to `out_dtype`.
 *
 * Replaces `_flash_colreduce` (flash_colreduce/flash.py:277-308) together
 * with the tail of `flash_colreduce` (flash.py:377-385).
 *
 * Every wait inside the kernels is bounded (about one second).  A kernel whose
 * wait expires gives up, leaves `out` unspecified and records a status code in
 * the workspace and in a per-device mailbox in mapped host memory; the NEXT
 * call of fcr_colreduce / fcr_colreduce_static on that device (or
 * fcr_poll_device_status at any time) then returns FCR_ERR_DEVICE_TIMEOUT
 * without launching, once, and clears the mailbox.  No synchronisation is
 * involved.  The first call on a device allocates the mailbox (64 bytes of
 * pinned host memory, the library's only allocation) and opts the kernels in
 * to their shared-memory size: make it before any stream capture begins.
 */
int fcr_colreduce(const fcr_problem* problem, const void* q, const void* k, void* out,
                  int32_t out_dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The operator without a caller-supplied workspace and without any allocation.
 * (No counterpart in the reference, which allocates through PyTorch,
 * flash_colreduce/flash.py:286.)
 *
 * Meant for hosts that cannot call cudaMalloc where this library runs: a
 * plugin invoked from another runtime's enqueue hook, a process that handed
 * its whole device-memory budget to one arena at start-up, or C code that has
 * no route to the framework allocator that owns the device.  The scratch
 * memory the kernels need (status words, per-row log-sum-exp, split partials)
 * is a fixed FCR_STATIC_SCRATCH_BYTES array in device global memory inside the
 * library image: every GPU that loads the library holds that much until the
 * process exits.
 *
 * - q, k, out, out_dtype, stream: exactly as for fcr_colreduce; the caller
 *   still owns inputs and output.
 * - A problem whose required scratch exceeds FCR_STATIC_SCRATCH_BYTES is
 *   rejected with FCR_ERR_WORKSPACE and a message naming both numbers.  The
 *   required scratch is fcr_workspace_bytes() for every problem but the decode
 *   shapes with a score cache (fcr_plan.score_cache): the cache is optional
 *   here as it is for fcr_colreduce, so for those the limit applies to
 *   fcr_plan.off_scores, and the cache is used when all of
 *   fcr_plan.workspace_bytes fits the array.
 * - The first call on each device looks up the array's device address (with
 *   that device current) and caches it; make that first call before any
 *   stream capture begins.
 * - All calls share the one array and it keeps whatever the previous call left
 *   in it.  The call clears the words that must start at zero on `stream`
 *   itself, so back-to-back calls on one stream are fine; two calls that can
 *   overlap on the GPU (different streams, or different host threads on
 *   different streams) race on the array and must be serialised by the caller.
 * - Performs no cudaMalloc / cudaFree and uses no allocating library routine
 *   (tracing, if enabled with fcr_trace_enable, creates CUDA events: leave it off).
 *   It does not create the status mailbox either; it uses the one an earlier
 *   fcr_colreduce call on the device created, if any.  Without a mailbox an
 *   expired device-side wait is visible through fcr_read_device_status_static.
 */
#define FCR_STATIC_SCRATCH_BYTES (8u << 20)
int fcr_colreduce_static(const fcr_problem* problem, const void* q, const void* k, void* out,
                         int32_t out_dtype, void* stream);

/*
 * Tail of a sharded run: `acc` holds fp32 column sums (or maxima) of shape
 * (B,H,N) that were produced with reduction FCR_SUM / FCR_MAX and combined
 * across shards; this applies the mean divisor (for FCR_MEAN) for a whole
 * problem of M rows and N keys and casts to `out_dtype`.
 * Replaces flash_colreduce/flash.py:377-385 for that case.
 */
int fcr_finalize(const float* acc, void* out, int32_t out_dtype, int32_t B, int32_t H, int32_t M,
                 int32_t N, int32_t reduction, int32_t is_causal, void* stream);

/*
 * ---- Several GPUs: one process (rank) per GPU ----------------------------
 * The reference has no multi-GPU path; these entry points have no counterpart
 * in it.  Heads are independent, and so are the query rows of a head, so the
 * work is sharded without any exchange of Q, K or scores: a rank computes
 * fp32 partial column vectors for its heads / rows, the partials are combined
 * by ONE all-reduce (sum, or max for FCR_MAX) over NCCL, and the mean divisor
 * of flash_colreduce/flash.py:377-384 and the cast come last.  NCCL is loaded
 * at run time (libnccl.so.2, the copy already in the process if there is one).
 *
 * fcr_shard says what a rank computes: heads [head_lo, head_hi) of the B*H
 * heads and, of each of them, the query rows [row_lo[r], row_hi[r]) for
 * r < n_ranges.  fcr_plan_shards fills it: with heads >= world the heads are
 * partitioned (one range: all rows; needs_reduce = 0); otherwise world / heads
 * ranks share a head and rank g of a head takes row chunks g and
 * 2 * ranks_per_head - 1 - g of 2 * ranks_per_head chunks of whole 128-row
 * tiles (zig-zag: equal causal work); ranks left over get no heads and only
 * take part in the all-reduce.
 */
typedef struct fcr_shard {
  int32_t rank, world;
  int32_t head_lo, head_hi;
  int32_t n_ranges;
  int32_t row_lo[2], row_hi[2];
  int32_t needs_reduce;     /* rows of a head are spread over several ranks */
} fcr_shard;

int fcr_plan_shards(int32_t heads, int32_t M, int32_t world, int32_t rank, fcr_shard* out);

/*
 * Communicator: rank 0 obtains FCR_NCCL_ID_BYTES bytes from fcr_comm_unique_id
 * and hands them to every rank by whatever means the application has; every
 * rank then calls fcr_comm_init with its own device current.  The handle is an
 * ncclComm_t; an application that already has one may pass its own instead.
 */
#define FCR_NCCL_ID_BYTES 128
int fcr_comm_unique_id(void* id_out);
int fcr_comm_init(const void* id, int32_t world, int32_t rank, void** comm_out);
int fcr_comm_destroy(void* comm);

/*
 * The sharded operator.  `local` describes the tensors this rank holds: B = 1,
 * H = head_hi - head_lo heads, ALL M rows and N keys of them (q, k, strides,
 * dtype as for fcr_colreduce), and the whole problem's reduction, mask and
 * scale.  acc: device fp32 (total_heads, N), scratch for the partial vectors;
 * out: device (total_heads, N) of out_dtype, the full result on every rank.
 * workspace: at least fcr_sharded_workspace_bytes(local, shard), 256-byte
 * aligned.  comm may be NULL when shard->world == 1.  Everything is queued on
 * `stream`: a memset of acc, fcr_colreduce's kernels per row range, one small
 * fold kernel per range, ncclAllReduce, the finalize kernel; no host
 * synchronisation.
 */
size_t fcr_sharded_workspace_bytes(const fcr_problem* local, const fcr_shard* shard);
int fcr_colreduce_sharded(const fcr_problem* local, const fcr_shard* shard, int32_t total_heads, const void* q,
                          const void* k, float* acc, void* out, int32_t out_dtype, void* workspace,
                          size_t workspace_bytes, void* comm, void* stream);

/*
 * Synchronises `stream` and reads the device status words of a workspace
 * used by fcr_colreduce.  Returns FCR_OK if no bounded wait expired, else
 * FCR_ERR_DEVICE_TIMEOUT with details in fcr_last_error(); `code_out` (may be
 * NULL) receives the raw first status word.
 */
int fcr_read_device_status(const void* workspace, void* stream, int32_t* code_out);

/* The same for the built-in scratch array that fcr_colreduce_static uses on the current device. */
int fcr_read_device_status_static(void* stream, int32_t* code_out);

/*
 * Looks at the current device's status mailbox without synchronising anything:
 * FCR_OK when no kernel of an earlier call reported an expired wait, else
 * FCR_ERR_DEVICE_TIMEOUT (details in fcr_last_error(), raw code in `code_out`,
 * which may be NULL); the mailbox is cleared, so a failure is reported once.
 * A failure of a kernel that is still running or queued is seen only after it
 * has happened: poll after the work is known to be done, or rely on the check
 * the next fcr_colreduce call makes.
 */
int fcr_poll_device_status(int32_t* code_out);

/* Number of kernels this library has launched in the process so far (all threads). */
int64_t fcr_launch_count(void);

/*
 * Self-test of the bounded waits, for the calling thread's later
 * fcr_colreduce calls: `wait_limit_cycles` > 0 replaces the one-second bound
 * of every device-side wait (in SM clock cycles), and `skip_ring_load` >= 0
 * makes the first CTA of each pass kernel leave out its skip_ring_load-th
 * streamed-tile load, so that the waits on that tile expire: the kernels then
 * give up in an orderly way (no trap, no fault; tensor memory is released) and
 * the call's failure is reported as described at fcr_colreduce.  (0, -1)
 * restores normal operation.  The decode (key-streaming) kernels ignore
 * skip_ring_load.
 */
int fcr_self_test_hooks(int64_t wait_limit_cycles, int32_t skip_ring_load);

/*
 * Tracing (the reference has none; its benchmark times whole calls on the
 * host, benchmarks/run.py:59-83).  While enabled for the calling thread, each
 * fcr_colreduce call records CUDA events on its stream before the rows pass,
 * between the passes and after the last kernel (at most 256 calls are kept;
 * enabling resets the count).  fcr_trace_read synchronises on call `index`
 * and returns the device time of its rows pass (plus the split combine, if
 * any) and of its columns pass (plus the final reduction, if any).
 */
int fcr_trace_enable(int32_t on);
int32_t fcr_trace_count(void);
int fcr_trace_read(int32_t index, float* rows_ms, float* cols_ms);

/*
 * Row-wise top-k over a contiguous (rows, n) score array of dtype `dtype`
 * (FCR_F16, FCR_BF16 or FCR_F32), e.g. the (B*H, N) output of fcr_colreduce:
 * for every row the positions of its k largest scores, in ascending position
 * order, as int32 (index_bits = 32) or int64 (index_bits = 64) into
 * `indices` (rows, k), and, when `values` is not null, the scores at those
 * positions into `values` (rows, k) of the same dtype.  Among scores equal to
 * the k-th largest the lowest positions win; NaN orders above +inf.  This is
 * the selection step of the token-pruning use the reference's README.md:9
 * names; the reference has no counterpart (it returns the scores).  One
 * launch on `stream`, no workspace, no allocation, no host synchronisation.
 */
int fcr_topk(const void* scores, int32_t dtype, int32_t rows, int32_t n, int32_t k, void* indices,
             int32_t index_bits, void* values, void* stream);

/*
 * Row-wise threshold selection over the same kind of array: for every row the
 * positions whose score is greater than `threshold` (compared in fp32), in
 * ascending order, into `indices` (rows, n) -- only the first counts[row]
 * entries of a row are written -- and their number into `counts` (rows).
 * The other selection rule of a pruning consumer; no counterpart in the
 * reference.  One launch on `stream`, no workspace, no host synchronisation.
 */
int fcr_select_above(const void* scores, int32_t dtype, int32_t rows, int32_t n, float threshold,
                     void* indices, int32_t index_bits, int32_t* counts, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_COLREDUCE_B200_H_ */
