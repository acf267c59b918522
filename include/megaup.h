/*
 * megaup.h - C ABI of libmegaup.so, the sm_100a implementation of the two
 * fused Ulysses exchange GEMMs and of the symmetric-memory runtime under them.
 *
 * The reference project (mega_up 0.3.0) is pure Python over the CuTe DSL and
 * has no C ABI; each entry point below names the Python seam of the reference
 * it stands behind (file:line in the reference tree).
 *
 * Conventions
 *   - every function returns MUP_OK (0) or a negative MUP_ERR_* code and
 *     never throws; mup_last_error() gives the message of the calling
 *     thread's last failure;
 *   - pointers are raw device addresses (tensor.data_ptr()); the caller keeps
 *     the memory alive for as long as a plan that was given it exists;
 *   - `stream` is a cudaStream_t passed as void*; nothing here creates a
 *     stream or synchronises one;
 *   - launch calls allocate nothing; plan creation allocates host memory only;
 *   - all data is BF16, accumulation FP32, one rounding to BF16.
 *
 * Device-side failures (a bounded wait that ran out) do not fault the GPU:
 * the kernel writes a code into the status word the plan was given and ends
 * normally. Status word layout: code << 24 | detail, code one of MUP_ST_*.
 */
#ifndef MEGAUP_H_
#define MEGAUP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MUP_ABI_VERSION 1

#define MUP_OK 0
#define MUP_ERR_BAD_ARG (-1)
#define MUP_ERR_CUDA (-2)
#define MUP_ERR_UNSUPPORTED (-3)
#define MUP_ERR_DRIVER (-4)
#define MUP_ERR_DEVICE_STATUS (-5)

#define MUP_ST_OK 0
#define MUP_ST_PRODUCER_SLOT_TIMEOUT 1
#define MUP_ST_MMA_FULL_TIMEOUT 2
#define MUP_ST_MMA_ACC_TIMEOUT 3
#define MUP_ST_EPILOGUE_TIMEOUT 4
#define MUP_ST_PULL_READY_TIMEOUT 5
#define MUP_ST_SMEM_MISALIGNED 6
#define MUP_ST_FLAG_TIMEOUT 7
#define MUP_ST_ITEM_FEED_TIMEOUT 8

typedef struct mup_peer_write_plan mup_peer_write_plan;
typedef struct mup_pull_plan mup_pull_plan;
typedef struct mup_arena mup_arena;

/* ---- library ------------------------------------------------------------ */

int mup_abi_version(void);
const char *mup_last_error(void);

/* Whether `device` can run the kernels (compute capability 10.x).
 * Replaces mega_up/ops.py:272-278 (_check_runtime_device). */
int mup_device_supported(int device, int *supported);

/* The shape rule of the exchanged width: up in {2,4,8}, width > 0,
 * width % up == 0, width % 256 == 0, (width / up) % 128 == 0. Returns 0 when
 * supported, else the 1-based index of the first violated clause.
 * Replaces mega_up/runtime.py:32-57 (unsupported_shape_reason). */
int mup_shape_rule(int64_t width, int up);

/* First N tile visited by `rank`: ceil(rank * n_tiles / up) mod n_tiles.
 * Replaces mega_up/kernels/peer_write_gemm.py:977-993 (peer_n_rotation). */
int mup_peer_n_rotation(int rank, int up, int n_total, int tile_n);

/* The work-item list the library would run for a problem, without touching a
 * GPU (host arithmetic only): `slots` CTAs (cta_group 1) or CTA pairs
 * (cta_group 0 or 2) that are resident at once run items i, i + slots, ... in
 * list order. Item encoding: bits 0-13 row tile (128 * cta_group rows), bits
 * 14-25 first column / 64, bits 26-28 columns / 64 - 1. Writes at most
 * `capacity` items, the full count, the widest item in columns and the
 * critical path the library's time model predicts (SM cycles). mode 0 =
 * peer-write (each rank starts every row at its own column block), 1 = pull.
 * Plays the part of the reference's tile scheduler parameters
 * (mega_up/kernels/peer_write_gemm.py:775-781, headshard_pull_gemm.py:1227-1268),
 * which it fixes at compile time. Any output pointer may be NULL. */
int mup_schedule_preview(int mode, int rows, int n, int k, int up, int rank, int cta_group, int slots,
                         uint32_t *items, int capacity, int *count, int *max_item_cols,
                         double *model_cycles);

/* Plans created by the calling thread after this call launch at most
 * `max_ctas` CTAs (0 lifts the limit), leaving the other SMs to kernels of
 * other streams. The kernels need their whole grid resident at once (the pull
 * workers of every CTA own a share of the first tickets), so a caller that runs
 * them next to other work reserves room this way. Plays the part of the
 * `max_active_ctas` argument of the reference's compile_headshard_pull_gemm
 * (mega_up/kernels/headshard_pull_gemm.py:2440-2777). */
int mup_set_max_active_ctas(int max_ctas);

/* ---- status word ---------------------------------------------------------- */

/* One 64-byte block of pinned, device-mapped host memory. `host_ptr` is read
 * by the CPU, `device_ptr` is what plans and flag kernels are given. */
int mup_status_create(uint32_t **host_ptr, void **device_ptr);
int mup_status_destroy(uint32_t *host_ptr);

/* ---- symmetric-memory arena ---------------------------------------------- */

/* Device-local physical allocation (cuMemCreate) of at least `bytes`, rounded
 * up to the allocation granularity, mapped read/write into this process and
 * zero-filled, exported as a POSIX file descriptor that another process on
 * the node can import. Replaces symm_mem.empty / empty_strided_p2p at
 * mega_up/runtime.py:72-91. */
int mup_arena_create(int device, uint64_t bytes, mup_arena **out);
/* Map a peer's exported allocation into this process with read/write access
 * from `device`. Replaces symm_mem.rendezvous + handle.get_buffer at
 * mega_up/runtime.py:94-105, :618-625. The fd stays owned by the caller. */
int mup_arena_import(int device, int fd, uint64_t mapped_bytes, mup_arena **out);
int mup_arena_info(const mup_arena *arena, void **device_ptr, uint64_t *mapped_bytes, int *fd);
int mup_arena_destroy(mup_arena *arena);

/* ---- slot hand-off flags -------------------------------------------------- */

/* All-peer barrier on `stream`, replacing torch's symmetric-memory
 * handle.barrier(channel=0) (mega_up/runtime.py:108-112). Every rank owns an
 * array of `up` uint32 flags; rank r publishes `epoch` into entry r of every
 * peer's array with a system-scope release store, then waits (bounded by
 * timeout_ns) until every entry of its own array has reached `epoch`.
 * `peer_flags[p]` is the address, in this process, of rank p's array. Epochs
 * must increase by one per barrier on every rank. On timeout the kernel
 * writes MUP_ST_FLAG_TIMEOUT into the status word and ends normally. */
int mup_flag_barrier(void *const *peer_flags, int up, int rank, uint32_t epoch,
                     void *status_device_ptr, uint64_t timeout_ns, void *stream);

/* ---- hand-off folded into the kernels ----------------------------------------- */

/* Sync points form one sequence that every rank walks through in the same
 * order (a stand-alone mup_flag_barrier is "signal e, then wait e"). The
 * *_synced launches below fold the two halves into the kernels around them:
 * the kernel waits for `wait_epoch` before it first touches memory the
 * hand-off protects (0: no wait) and, once all of its CTAs have finished the
 * work `signal_epoch` stands for, raises that epoch at every peer (0: no
 * signal). This replaces the two barrier kernels per operation of the
 * reference's protocol (mega_up/runtime.py:264, :281, :415, :421).
 * `done_counter` is a zero-initialised device uint64 that only ever grows;
 * pass its expected value before the launch in `done_before` and read the
 * value it will have afterwards from `done_after`. */
typedef struct mup_sync {
  void *const *peer_flags; /* [up] flag arrays as in mup_flag_barrier */
  int up;
  int rank;
  uint32_t wait_epoch;
  uint32_t signal_epoch;
  void *done_counter;
  uint64_t done_before;
  uint64_t done_after; /* out */
  void *status_device_ptr;
  uint64_t timeout_ns;
} mup_sync;

/* ---- peer-write GEMM ------------------------------------------------------- */

/* Bind out = bf16(A[rows,k] @ W[n,k]^T + bias) whose column block p lands in
 * slot_ptrs[p], a dense [rows, n/up] BF16 matrix (this rank's receive slot in
 * rank p's arena). Replaces make_peer_write_launch
 * (mega_up/kernels/peer_write_gemm.py:2697-2930). cta_group: 1 or 2 selects
 * the tcgen05 CTA pairing, 0 lets the library choose. */
int mup_peer_write_plan_create(mup_peer_write_plan **out, int device, int rows, int n, int k,
                               int up, int rank, const void *weight, const void *bias,
                               void *const *slot_ptrs, int cta_group, void *status_device_ptr,
                               uint64_t timeout_ns);
/* Launch on `stream` for input `a` ([rows, k] BF16, 16-byte aligned).
 * Replaces PeerWriteLaunch.__call__ (peer_write_gemm.py:2677-2694). */
int mup_peer_write_launch(mup_peer_write_plan *plan, const void *a, void *stream);
/* As mup_peer_write_launch; the first store into a peer slot waits for
 * sync->wait_epoch (the owners have copied the previous result out) and the
 * last CTA to finish its stores signals sync->signal_epoch. sync == NULL
 * behaves like mup_peer_write_launch. */
int mup_peer_write_launch_synced(mup_peer_write_plan *plan, const void *a, void *stream,
                                 mup_sync *sync);
/* Any output pointer may be NULL. tile_n is the width of an output tile the
 * widest work item the library chose for this problem (64 .. 512 columns);
 * n_rotation is the first column of the first item in 256-column blocks. */
int mup_peer_write_plan_info(const mup_peer_write_plan *plan, int *grid_ctas, int *cta_group,
                             int *n_rotation, int *smem_bytes, int *tile_n);
/* Cycle tracing (no counterpart in the reference, which has no built-in tracing):
 * give the plan a zeroed device buffer of grid_ctas * 16 uint64 and every launch
 * records, per CTA, {start clock, end clock, MMA cycles waiting for operands,
 * MMA cycles waiting for a free accumulator, TMA-producer cycles waiting for a
 * free stage, epilogue cycles waiting for an accumulator, start ns, end ns,
 * end ns of the CTA's pull workers, tickets they copied} (unused slots stay 0).
 * NULL switches tracing off (the default). */
int mup_peer_write_plan_set_trace(mup_peer_write_plan *plan, void *trace_buffer);
int mup_peer_write_plan_destroy(mup_peer_write_plan *plan);

/* ---- head-shard pull GEMM --------------------------------------------------- */

/* Shape of a pull ticket for shard rows of `shard_elems` BF16 (host arithmetic
 * only): `*rows` rows of one peer shard per ticket, or, when a single row
 * exceeds a ticket, `*segments` equal column segments of one row. Describes what
 * the reference tabulates in _vector_pull_rows_per_ticket / _pull_column_chunks
 * (headshard_pull_gemm.py:166-198) for its own kernel. */
int mup_pull_ticket_shape(int shard_elems, int *rows, int *segments);
/* Bytes of zero-initialised device workspace a pull plan for `rows` needs. */
uint64_t mup_pull_workspace_bytes(int rows);

/* Bind dy[t, p*k/up + c] = peer_arena_ptrs[p][(rank*peer_rows + t)*k/up + c]
 * followed by out = bf16(dy[rows,k] @ W[n,k]^T + bias). `dy` ([rows,k]) and
 * `out` ([rows,n]) are caller-owned BF16 buffers; `workspace` holds the
 * ticket cursor and the per-panel ready counts and is only ever incremented,
 * so launches need no reset in between. Replaces compile_headshard_pull_gemm
 * (mega_up/kernels/headshard_pull_gemm.py:2440-2777). */
int mup_pull_plan_create(mup_pull_plan **out, int device, int rows, int n, int k, int up, int rank,
                         int peer_rows, const void *weight, const void *bias,
                         void *const *peer_arena_ptrs, void *dy, void *out_buf, void *workspace,
                         int cta_group, void *status_device_ptr, uint64_t timeout_ns);
/* Replaces CompiledHeadShardPullGemm.__call__ (headshard_pull_gemm.py:2407-2428). */
int mup_pull_launch(mup_pull_plan *plan, void *stream);
/* As mup_pull_launch; the pull workers wait for sync->wait_epoch (the peers
 * have staged their shards) before their first peer load, and the last pull
 * warp to run out of tickets signals sync->signal_epoch (this rank will not
 * read a peer arena again), typically long before the GEMM itself ends. */
int mup_pull_launch_synced(mup_pull_plan *plan, void *stream, mup_sync *sync);
/* After a device-side failure the counters are inconsistent: zero the
 * workspace on `stream` and restart the launch ordinal. Replaces
 * CompiledHeadShardPullGemm.reset_workspace (headshard_pull_gemm.py:2393-2405). */
int mup_pull_plan_reset(mup_pull_plan *plan, void *stream);
int mup_pull_plan_info(const mup_pull_plan *plan, int *grid_ctas, int *cta_group,
                       uint64_t *launches, int *smem_bytes, int *tile_n);
/* Same tracing switch as mup_peer_write_plan_set_trace. */
int mup_pull_plan_set_trace(mup_pull_plan *plan, void *trace_buffer);
int mup_pull_plan_destroy(mup_pull_plan *plan);

/* ---- head-shard pull GEMM without any allocation ---------------------------- */

/* Largest `rows` the built-in scratch of mup_pull_gemm_noalloc can serve. */
#define MUP_NOALLOC_MAX_ROWS 262144

/* One-call variant of the pull GEMM for callers that cannot allocate device
 * memory at the point of the call: code running under a memory pool that is
 * already fully committed, inside a framework's "no allocator calls here"
 * region (for example while another component owns the caching allocator), or
 * a host that may only hand over buffers it was given. It has no counterpart
 * in the reference, whose pull always allocates its cursor and ready counts.
 *
 * Same computation as mup_pull_plan_create + mup_pull_launch: it fills `dy`
 * ([rows,k]) from the `up` staged peer arenas and writes
 * out = bf16(dy @ W^T + bias) to `out_buf` ([rows,n]); the caller still
 * passes every input and output. What differs is the scratch (ticket cursor,
 * one claim word per pull warp and the per-panel ready counts): it is a fixed array inside the library's device
 * image, about 24 KB per GPU, held by every GPU that loads the library until
 * the process exits. The call performs no cudaMalloc/cudaFree, creates no
 * plan object and calls no allocating library routine.
 *
 * Limits and rules:
 *   - rows <= MUP_NOALLOC_MAX_ROWS, otherwise MUP_ERR_BAD_ARG with a message
 *     naming the limit (use the plan API with your own workspace instead);
 *   - the first call on a device performs a one-time set-up for that device
 *     (it resolves the scratch array's device address and sets kernel
 *     attributes); make that first call before starting any stream capture;
 *   - all calls on one GPU share the scratch, which keeps the last call's
 *     contents; each call clears the part it uses on `stream` before the
 *     kernel. Two calls that overlap on the GPU (different streams without an
 *     ordering between them) race on it: serialise them. */
int mup_pull_gemm_noalloc(int device, int rows, int n, int k, int up, int rank, int peer_rows,
                          const void *weight, const void *bias, void *const *peer_arena_ptrs,
                          void *dy, void *out_buf, int cta_group, void *status_device_ptr,
                          uint64_t timeout_ns, void *stream);

/* ---- layout copies ----------------------------------------------------------- */

/* dst row i = src row index[i] (index == NULL: identity), rows of
 * `row_elems` BF16 (a multiple of 8), both 16-byte aligned. Replaces the
 * index_select copies at mega_up/runtime.py:330-335 and :367-372. */
int mup_gather_rows(void *dst, const void *src, const int64_t *index, int64_t rows,
                    int64_t row_elems, void *stream);

/* mup_gather_rows with the hand-off folded in: every block waits for
 * sync->wait_epoch before it reads or writes, the last block to finish
 * signals sync->signal_epoch. */
int mup_gather_rows_synced(void *dst, const void *src, const int64_t *index, int64_t rows,
                           int64_t row_elems, void *stream, mup_sync *sync);

/* Batched source-major <-> batch-major regroup of dense rows:
 * dst[(b*up + r)*seq + s] = src[(r*batch + b)*seq + s]   when to_batch_major,
 * dst[(r*batch + b)*seq + s] = src[(b*up + r)*seq + s]   otherwise.
 * Replaces the permuted copy_ at mega_up/runtime.py:272-280 and :399-414. */
int mup_regroup_rows(void *dst, const void *src, int up, int batch, int64_t seq,
                     int64_t row_elems, int to_batch_major, void *stream);

/* Diagnostic (no counterpart in the reference): one thread issues `iters`
 * dependent 8-byte loads from `zeros` (at least 2 KiB of zero-filled device
 * memory, local or a mapped peer arena) and writes the elapsed nanoseconds to
 * out_ns[0] (device memory): elapsed / iters is the load round-trip time, over
 * NVLink when `zeros` belongs to a peer. */
int mup_probe_load_latency(const void *zeros, int iters, uint64_t *out_ns, void *stream);

/* mup_regroup_rows with the hand-off folded in (see mup_gather_rows_synced). */
int mup_regroup_rows_synced(void *dst, const void *src, int up, int batch, int64_t seq,
                            int64_t row_elems, int to_batch_major, void *stream, mup_sync *sync);

#ifdef __cplusplus
}
#endif

#endif /* MEGAUP_H_ */
