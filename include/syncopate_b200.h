/*
 * syncopate_b200 — C ABI of the B200 (sm_100a) backend for Syncopate's chunk-centric overlapped
 * operators.  Plain C: pointers, sizes and PODs only; every function returns 0 on success or a
 * negative SYN_ERR_* code (see syn_strerror).  No exception crosses this boundary.
 *
 * The library sits behind Syncopate's Python front end: plans are built and lowered on the host
 * (build_*_plan -> CommGenerator.plan_signals / generate_code_for_plan ->
 * lower_comm_plan_to_raw_schedules) and the per-rank wave offsets / shapes / signal indices / peer
 * ranks produced by RawSchedule.gen_*_lists() (syncopate/interface/tile_schedule.py:90-145) are
 * handed to the kernels below as HOST arrays; the library copies them into kernel parameters.
 *
 * Threading: a syn_ctx belongs to one host thread of one process (one process per GPU).
 * Device pointers are CUDA device pointers of the current device unless stated otherwise.
 * `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 */
#ifndef SYNCOPATE_B200_H
#define SYNCOPATE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SYN_MAX_WORLD 8
#define SYN_MAX_WAVES 64
#define SYN_MAX_COMM_OPS 64
#define SYN_NUM_COUNTERS (SYN_MAX_WAVES + SYN_MAX_COMM_OPS + 2)

/* ------------------------------------------------------------------ error codes */
#define SYN_OK 0
#define SYN_ERR_INVALID (-1)       /* bad argument (NULL, negative size, unsupported block, ...) */
#define SYN_ERR_SHAPE (-2)         /* schedule entry out of bounds or not a multiple of the block */
#define SYN_ERR_CUDA (-3)          /* a CUDA runtime / driver call failed (syn_last_cuda_error) */
#define SYN_ERR_TIMEOUT_FLAG (-4)  /* device: a signal flag never reached its value */
#define SYN_ERR_TIMEOUT_MBAR (-5)  /* device: an intra-kernel pipeline wait ran out */
#define SYN_ERR_TIMEOUT_COUNTER (-6)
#define SYN_ERR_RENDEZVOUS (-7)    /* peers did not show up at the rendezvous in time */
#define SYN_ERR_UNSUPPORTED (-8)
#define SYN_ERR_TOO_LARGE (-9)     /* more waves / ops / bytes than the fixed limits above */

const char* syn_strerror(int code);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* syn_last_cuda_error(void);
/* Library version and the SM architecture it was compiled for (always "sm_100a"). */
const char* syn_version(void);

/* ------------------------------------------------------------------ schedules
 * One lowered RawSchedule (syncopate/interface/tile_schedule.py:65-171), flattened wave-major.
 * All arrays are HOST memory, int32, in ELEMENTS of the scheduled tensor (not tiles):
 *   offsets[w*ndim + d], shapes[w*ndim + d]   gen_block_offset_lists / gen_block_shape_lists
 *   signals[w]       flag index the wave waits on (consumer) or sets when complete (producer), -1 = none
 *   target_ranks[w]  peer that owns / receives the wave's data, -1 or own rank = local (may be NULL)
 *   dst_offsets[w*ndim + d]  offsets on the peer side (may be NULL = same as offsets)
 * ndim = 2 for GEMM (M, N) and 4 for attention (Z, H, Q, KV).
 */
typedef struct syn_schedule {
  int32_t num_waves;
  int32_t ndim;
  const int32_t* offsets;
  const int32_t* shapes;
  const int32_t* signals;
  const int32_t* target_ranks;
  const int32_t* dst_offsets;
} syn_schedule;

/* ------------------------------------------------------------------ GEMM
 * C[M,N] = A[M,K] * B[N,K]^T, 16-bit inputs, fp32 accumulation in tensor memory, 16-bit output.
 * Replaces the Triton persistent GEMM templates (syncopate/computation/gemm/template.py:21-159
 * consumer, :224-351 producer; local_code.py:18-107 un-fused).  Tile order = waves in array order,
 * grouped raster with GROUP_SIZE_M inside each wave (template.py:10-18, :103-136).
 */
#define SYN_DTYPE_F16 0
#define SYN_DTYPE_BF16 1

typedef struct syn_gemm_args {
  const void* a; /* [M, K] row-major, leading dimension lda (elements) */
  const void* b; /* [N, K] row-major (K-major weights), leading dimension ldb */
  void* c;       /* [M, N] row-major, leading dimension ldc */
  int32_t M, N, K;
  int32_t lda, ldb, ldc;
  int32_t dtype;        /* SYN_DTYPE_* */
  int32_t block_m;      /* 128 (0 = default) */
  int32_t block_n;      /* 64..256, multiple of 16 (0 = choose to minimise tail quantisation) */
  int32_t block_k;      /* 64 (0 = default) */
  int32_t group_size_m; /* grouped-raster height, 0 = 8 */
  int32_t num_sms;      /* persistent grid size, 0 = all SMs of the device */
  /* Signal flags (uint64 words, device memory).  A wave with signals[w] >= 0 starts only once
   * signal_ptr[signals[w]] >= signal_value (consumer), or sets it to signal_value after its last
   * tile is stored (producer; needs counter_ptr: uint32[num_waves], zero before the first call;
   * every call leaves it zero again). */
  const uint64_t* consumer_signal_ptr;
  uint64_t* producer_signal_ptr;
  uint32_t* producer_counter_ptr;
  uint64_t signal_value;   /* value waited for / written; 0 = 1 */
  uint64_t timeout_ns;     /* bound of every device-side wait; 0 = 2 s */
  int32_t* status;         /* device int32[4] {code, wave, flag, block}; may be NULL */
  /* Optional device uint32[2], zero before the first call (every call leaves it zero): when given,
   * CTAs take tiles from a grid-wide counter as they become free instead of round-robin, which
   * hides the stall of the CTAs that reach a wave before its flag is up. */
  uint32_t* sched_counter;
  /* Optional device uint64[2 + 3 * num_waves] of %globaltimer stamps (ns) for the non-overlapped-time
   * breakdown: [0] earliest CTA start (initialise to UINT64_MAX), [1] latest CTA end (0); per wave w:
   * [2+3w] earliest flag-wait begin (UINT64_MAX), [3+3w] latest flag-wait end (0), [4+3w] summed wait
   * over CTAs (0).  A wave waits either for its consumer flag (before its first load) or, in GEMM +
   * reduce-scatter, for the flags of the staged partial sums it adds (w then counts the waves the
   * kernel walks: those of src_sched with the locally kept one cut into its row pieces). */
  uint64_t* trace;
  /* Optional device scratch, 256-byte aligned, its first 256 bytes zero before the first call (every
   * call leaves them zero): lets the CTA-pair kernel cut the few tiles left over after the last full
   * persistent round along K over all CTA pairs (fp32 partial tiles in the scratch, summed in a
   * fixed order) instead of giving them a round of their own.  256 + 74 * 256 * 256 * 4 bytes
   * (about 19.4 MB) always suffice; with less, fewer shapes qualify. */
  void* workspace;
  size_t workspace_bytes;
} syn_gemm_args;

/* Un-fused / flag-gated persistent GEMM on one GPU.  `sched` may be NULL (one wave = whole C);
 * `producer_sched` is the RawSchedule of C when the GEMM feeds communication (may be NULL).
 * When both are given they must describe the same tile order (same shapes), as in the reference's
 * dual-role kernels (syncopate/computation/transform/transformer.py:1086-1116).
 * `sched` may also have ndim = 3 with axes (M, N, K), the consumer form of all-to-all + GEMM
 * (tests/test_all2all_gemm.py:83-110 builds exactly these waves): every wave covers all of C and one
 * range of K (multiples of 64, disjoint, together all of K), A's columns of that range being valid
 * once signal_ptr[signals[w]] >= signal_value.  Every tile then accumulates over the ranges in
 * wave order, waiting for a range's flag before its first load from it (at most 16 ranges; not
 * together with producer_sched). */
int syn_gemm(const syn_gemm_args* args, const syn_schedule* sched, const syn_schedule* producer_sched,
             void* stream);

/* Same operation as syn_gemm in its producer role, for callers that cannot allocate device memory
 * (a process whose GPU memory is wholly owned by its own pool, a latency-critical step that must
 * not hit cudaMalloc's device-wide synchronisation, a plugin in a host that forbids allocation
 * after start-up).  It has no counterpart in the reference.  args->producer_counter_ptr is
 * ignored: the per-wave tile counters live in a 256-byte device array inside the library (every
 * GPU that loads the library holds one until exit), so at most SYN_MAX_WAVES (64) waves are
 * accepted (SYN_ERR_TOO_LARGE beyond).  No cudaMalloc / cudaFree / allocating routine is called.
 * The first call on each device looks up the array's device address; make that first call outside
 * any stream capture.  Each call zeroes the array on `stream` before launching.  All calls on a
 * device share the array: two calls that may overlap on the GPU (different streams) race. */
int syn_gemm_noalloc(const syn_gemm_args* args, const syn_schedule* sched, const syn_schedule* producer_sched,
                     void* stream);

/* The same GEMM in its consumer role with the schedule given in closed form (the reference's
 * Mod1DSchedule, syncopate/interface/tile_schedule.py:214-266: what SimplifiedSchedule reduces the
 * schedule of a ring or swizzled direct all-gather to): num_waves equal blocks of `stride` rows
 * (axis 0) or columns (axis 1), block w at (starting_offset + w * stride) mod (stride * num_waves),
 * the first resident and block w > 0 waiting for flag w - 1 of args->consumer_signal_ptr. */
int syn_gemm_mod1d(const syn_gemm_args* args, int num_waves, int stride, int starting_offset, int axis, void* stream);

/* Smallest persistent-grid tail for an M x N output on `num_sms` SMs: returns the block_n the
 * library would choose for block_n = 0. */
int syn_gemm_pick_block_n(int M, int N, int num_sms);

/* ------------------------------------------------------------------ symmetric memory
 * Replaces the NVSHMEM symmetric heap of the reference's CommContext
 * (syncopate/communication/comm_runtime/communication_context.py:31-76: nvshmem_create_tensors
 * returns the peer-mapped views of every rank's buffer).  One process per GPU; every rank calls
 * the same sequence of syn_symm_alloc with the same sizes.  Buffers are cudaMalloc'ed, exported
 * with CUDA IPC and opened by every peer, so that kernels address a peer's copy through plain
 * pointers over NVLink.  Handles are exchanged through small files in `rendezvous_dir` (a
 * directory all ranks of the box can reach, e.g. under /dev/shm or /tmp).
 */
typedef struct syn_ctx syn_ctx;

/* View of one symmetric buffer from this rank: ptrs[r] addresses rank r's copy (ptrs[rank] is
 * local).  Tests on one GPU may fill it by hand with local pointers to emulate several ranks. */
typedef struct syn_symm {
  int32_t world;
  int32_t rank;
  void* ptrs[SYN_MAX_WORLD];
} syn_symm;

int syn_ctx_create(int rank, int world, int device, const char* rendezvous_dir, syn_ctx** out);
/* Unmaps peers, frees local buffers, removes this rank's rendezvous files.  Never blocks on peers:
 * call it on every rank after a syn_barrier and a synchronisation of the streams in use, so that no
 * peer's kernel or copy still touches a buffer that is being freed. */
int syn_ctx_destroy(syn_ctx* ctx);
/* Collective: allocates `bytes` (zero-filled) on every rank and fills `out` with all ranks' pointers.
 * Waits at most `timeout_s` seconds for the peers (0 = 120 s) and returns SYN_ERR_RENDEZVOUS after. */
int syn_symm_alloc(syn_ctx* ctx, size_t bytes, int timeout_s, syn_symm* out);
int syn_symm_free(syn_ctx* ctx, void* local_ptr);
/* Loads the code of every kernel of the library on the current device and waits for the device.
 * syn_ctx_create calls it.  With lazy module loading the first launch of a kernel may wait for the
 * kernels that are running on the device; a kernel that waits for a peer (a reduce wave, a barrier)
 * must never be what such a first launch waits for, so the loading is done once, up front. */
int syn_preload(void);
/* Device-side barrier over all ranks on `stream` (replaces nvshmem_barrier_all_on_stream, e.g.
 * tests/test_ag_gemm_gen.py:53): a one-block kernel raises this rank's slot on every peer and waits,
 * bounded by timeout_ns (0 = 2 s), for all slots.  Errors surface through syn_ctx_status. */
int syn_barrier(syn_ctx* ctx, void* stream, uint64_t timeout_ns);
/* Device int32[4] status block of the context {code, wave, flag, block}; kernels given it record
 * the first timed-out wait there.  syn_ctx_status synchronises `stream`, reads and clears it and
 * returns 0 or the SYN_ERR_TIMEOUT_* code; out4 (host, may be NULL) receives the four words. */
int32_t* syn_ctx_status_ptr(syn_ctx* ctx);
int syn_ctx_status(syn_ctx* ctx, void* stream, int32_t* out4);

/* Stream-ordered flag operations (replace _set_signal_cuda / _wait_eq_cuda of the reference's
 * op interpreter, communication_context.py:145-160): one-thread kernels that store `value` with
 * system-scope release, or wait (bounded) until *flag >= value; a wait that runs out records
 * {SYN_DEV_TIMEOUT_FLAG, -1, tag, -1} in `status` (device int32[4], may be NULL). */
int syn_flag_set(uint64_t* flag, uint64_t value, void* stream);
/* Copy-engine transfer between (peer-mapped) device pointers, the CopyEngineOp of the reference's
 * interpreter (communication_context.py:129-143). */
int syn_memcpy_async(void* dst, const void* src, size_t bytes, void* stream);
int syn_flag_wait(const uint64_t* flag, uint64_t value, uint64_t timeout_ns, int32_t* status, int tag,
                  void* stream);
/* Stream-ordered wait until *flag >= value as a stream memory operation: needs no SM, so it is not
 * starved by a persistent kernel that fills the GPU (which syn_flag_wait's one-thread kernel can
 * be).  Unbounded by itself: use it only for flags that a bounded kernel raises on every path.
 * SYN_ERR_UNSUPPORTED when the driver offers no such operation. */
int syn_flag_wait_stream(const uint64_t* flag, uint64_t value, void* stream);

/* ------------------------------------------------------------------ fused operators
 * The flag value of one fused call is `gemm.signal_value` (an epoch that the caller increases by
 * one per call; flags are never reset, waits are `>=`).  `counters` is device uint32
 * [SYN_NUM_COUNTERS], zero before the first call and left zero by every call (per-wave tile counts,
 * per-copy CTA counts, and the two words of the dynamic tile scheduler).
 */

/* All-gather + GEMM (replaces kernel_gemm_consumer + the copy-engine / SM-copy program,
 * syncopate/computation/gemm/template.py:21-159, tests/test_ag_gemm_gen.py:44-77, and the direct
 * remote read of template_ag.py:43-187).  gemm.a is this rank's copy of the gathered buffer
 * [M, K] with its own shard in place; `a_sched` is the RawSchedule of that buffer (ndim 2, blocks
 * [rows, K]).  For every wave whose target rank is another rank, the comm warps of all CTAs pull
 * the block from its owner's copy (a.ptrs[owner], owner = row offset / rows per rank) into
 * gemm.a and raise recv_flags[signals[w]]; GEMM tiles of the wave's rows (all N columns) start
 * once that flag is up.  recv_flags = gemm.consumer_signal_ptr (local). */
typedef struct syn_ag_gemm_args {
  syn_gemm_args gemm;
  syn_symm a;
  uint32_t* counters;
} syn_ag_gemm_args;
int syn_ag_gemm(const syn_ag_gemm_args* args, const syn_schedule* a_sched, void* stream);

/* GEMM + reduce-scatter (replaces kernel_gemm_producer + ring_reduce_tma and the direct remote
 * reduce, syncopate/computation/gemm/template.py:224-351, tests/test_gemm_rs.py:22-72,
 * template_rs.py:37-209).  The partial product C = A * B^T [M, N] is never stored whole: the tiles
 * of wave w (rows of `src_sched`, the RawSchedule of the partial-C buffer) go, as 16-bit values,
 * straight from the epilogue into the target rank's staging slab stage.ptrs[target] +
 * ((epoch & 1) * world + rank) * slab, and once the wave's last tile has landed
 * recv_flags.ptrs[target][remote_signals[w]] is raised.  A target may get its slab in several waves
 * (row pieces).  `dst_sched` is the RawSchedule of the receive buffer (target = sending rank,
 * signal = local flag; rows and columns are its last two axes): the rows kept here are cut into
 * the row pieces that the senders' waves arrive in, and each piece becomes one wave that waits for
 * the flags of exactly its rows from every other rank, adds the staged partial sums to its own
 * accumulators in fp32 (fixed order: ascending sender rank as first met in `dst_sched`) and writes
 * `out` [M / world, N].  Every other rank must send every piece exactly once.  gemm.c is unused
 * and may be NULL. */
typedef struct syn_gemm_rs_args {
  syn_gemm_args gemm;
  syn_symm stage;               /* 16-bit [2, world, M / world, N] on every rank */
  syn_symm recv_flags;          /* uint64 flags on every rank */
  const int32_t* remote_signals; /* host int32[num_waves of src_sched], -1 = none */
  void* out;                    /* [M / world, N] */
  int32_t ldo;                  /* 0 = N */
  uint32_t* counters;
  /* Optional transport by somebody else (copy engines): with `send_buf` set, the tiles of a wave
   * for another rank are stored into the LOCAL buffer send_buf[target][M / world][N] (16 bit, at the
   * wave's rows inside the slab) and the LOCAL flag send_flags[w] (w = the wave's index in
   * `src_sched`) is raised to the epoch when the wave is complete; the kernel then writes nothing
   * to a peer.  The caller moves each wave's rows to stage.ptrs[target] + ((epoch & 1) * world +
   * rank) * slab and raises recv_flags.ptrs[target][remote_signals[w]] (syn_ce_run below does this
   * on side streams).  A kernel that gives up on a timed-out wait still raises every send flag, so
   * such a stream cannot be left waiting; the error is in the status block. */
  void* send_buf;
  uint64_t* send_flags;         /* device uint64[num_waves of src_sched] */
  /* Optional device uint64[row pieces of the locally kept slab, in row order]: out_flags[g] is
   * raised (locally) to the epoch once piece g of `out` is complete, so that somebody else can
   * pass the reduced rows on while the kernel still runs (GEMM + all-reduce = this operator plus an
   * all-gather of the reduced slabs; the reference runs a library all-reduce per slice behind the
   * producer GEMM instead, tests/test_gemm_ar_collective.py:97-160). */
  uint64_t* out_flags;
  /* 0: the tiles of the own slab wait for the staged partial sums and add them in the epilogue
   * (one kernel).  1: the kernel stores the own partial sum like any other (16 bit) and a reduce
   * pass launched behind it on the same stream waits for the flags, adds the staged slabs with
   * coalesced loads and raises out_flags; the own partial sum is then rounded to 16 bits before
   * the fp32 sum, like those of the other ranks.  N must be a multiple of 8. */
  int32_t reduce_pass;
  int32_t reserved;
} syn_gemm_rs_args;
int syn_gemm_rs(const syn_gemm_rs_args* args, const syn_schedule* src_sched, const syn_schedule* dst_sched,
                void* stream);

/* A copy-engine program: the host-side form of a rank's CopyEngineOp / IntraNodeSignal /
 * WaitIntraNodeSignal records (syncopate/communication/comm_runtime/operations.py:9-69, interpreted
 * by communication_context.py:129-160) with every address resolved.  Step i runs on stream
 * streams[step.stream % num_streams], in array order per stream:
 *   wait_flag != NULL : stream waits until *wait_flag >= value (syn_flag_wait_stream: needs no SM)
 *   bytes > 0         : cudaMemcpyAsync(dst, src, bytes) (peer-mapped pointers allowed)
 *   set_flag != NULL  : *set_flag = value, ordered after the copy (syn_flag_set); with `flag_stream`
 *                       the write goes to that stream, behind an event recorded after the copy, so
 *                       that the copy stream runs its copies back to back
 * One call issues the whole program from C, so a program of a few dozen steps costs a few dozen
 * driver calls and nothing else. */
typedef struct syn_ce_step {
  const uint64_t* wait_flag;
  void* dst;
  const void* src;
  size_t bytes;
  uint64_t* set_flag;
  int32_t stream;
  int32_t reserved;
} syn_ce_step;
int syn_ce_run(const syn_ce_step* steps, int num_steps, void* const* streams, int num_streams, void* flag_stream,
               uint64_t value);

/* ------------------------------------------------------------------ attention
 * Flash-attention forward over a wave schedule (replaces the TLX kernel
 * _attn_fwd_ws_pipelined_pingpong and its host wrapper, syncopate/computation/attn/template.py:47-436,
 * and the un-fused local_code.py).  q [Z, Hq, Sq, D], k / v [Z, Hkv, Skv, D], o [Z, Hq, Sq, D] with
 * arbitrary element strides for (z, h, s) and D = 128 contiguous (so BHSD and BSHD layouts and
 * slices of a stacked [3, ...] buffer all work); 16-bit inputs, fp32 softmax, 16-bit output.
 * Hq must be a multiple of Hkv (grouped-query heads share a KV head).
 *
 * `sched` has ndim = 4 with axes (Z, H, Q, KV) in tokens, as the reference's wave metadata
 * (tests/test_all2all_attn_transform.py:58-117, tests/test_double_ring_ag_attn.py:60-81): a wave
 * covers the (z, h, q) box and attends to keys [kv_off, kv_off + kv_len); Q and KV offsets and
 * lengths must be multiples of 128.  A wave with signals[w] >= 0 starts only once
 * signal_ptr[signals[w]] >= signal_value.  A query row visited by several waves ends with the
 * log-sum-exp merge of its partial results; `lse` [Z, Hq, Sq] receives log2-domain LSE values.
 * `causal`: key j is visible to query i iff kv_pos(j) <= q_pos(i), positions being
 * q_pos[tile] + row and kv_pos[block] + col (device int32 arrays per 128 rows / keys; NULL =
 * the index itself).  Key blocks with no visible key are skipped.
 * `visit` is device int32 [Z, Hq, Sq] scratch, zero before the first call; `epoch` must be positive
 * and increase from call to call (rows not visited by a call keep their old contents).
 */
typedef struct syn_attn_args {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  int32_t* visit;
  int32_t Z, Hq, Hkv, Sq, Skv, D;
  int64_t q_strides[3]; /* elements: z, h, s */
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t o_strides[3];
  float sm_scale;
  int32_t causal;
  const int32_t* q_pos;
  const int32_t* kv_pos;
  int32_t dtype;
  int32_t num_sms;
  int32_t epoch;
  const uint64_t* signal_ptr;
  uint64_t signal_value; /* 0 = 1 */
  uint64_t timeout_ns;   /* 0 = 2 s */
  int32_t* status;
  const struct syn_attn_plan* plan; /* NULL, or a work-balanced ownership made by syn_attention_plan for
                                       exactly these shapes, waves, positions and num_sms */
  const struct syn_attn_push* push; /* NULL, or the producer role: finished rows go to their destination ranks */
} syn_attn_args;

/* Producer role of the attention kernel (replaces the reference's per-wave tile counter that raises
 * COMPUTE_DONE for a communication program to push the finished slab,
 * syncopate/computation/attn/template.py:47-361 with the producer epilogue of
 * computation/transform/transformer.py:882-903, driven as in tests/test_attn_all2all_transform.py:182-215).
 * Here the kernel pushes by itself: when a 128-row query tile has had its LAST visit (syn_attn_plan
 * visits), its final rows are not stored to `o` but staged in shared memory and sent with TMA
 * stores into the destination rank's buffer dst.ptrs[dst_rank], a [Z, dst_rows, dst_heads, 128]
 * tensor with element strides dst_strides (z, s, h), at row dst_row0 + (row - q_begin) and head
 * head_offset + h; when every tile of a slab has landed, flags.ptrs[dst_rank][flag] is raised to
 * the call's signal_value.  Needs a plan (fixed ownership lists), Sq a multiple of 128, slabs that
 * start and end on 128-row boundaries and cover every query row exactly once, at most 64 units
 * per CTA; tiles that no wave visits are not sent.  Earlier visits of a tile still merge through
 * `o` (local), which therefore must be a private buffer of the rank. */
typedef struct syn_attn_push_slab {
  int32_t q_begin, q_rows; /* query rows [q_begin, q_begin + q_rows) of the kernel's output */
  int32_t dst_rank;
  int32_t dst_row0;        /* destination row of q_begin */
  int32_t flag;            /* -1 = none */
} syn_attn_push_slab;
typedef struct syn_attn_push {
  int32_t num_slabs;       /* at most SYN_MAX_WORLD */
  const syn_attn_push_slab* slabs; /* host array */
  syn_symm dst;
  int64_t dst_strides[3];  /* elements: z, s, h */
  int32_t dst_rows, dst_heads;
  int32_t head_offset;
  syn_symm flags;
  uint32_t* counters;      /* device uint32[SYN_MAX_WORLD], zero before the first call (left zero by every call) */
} syn_attn_push;

/* Which CTA owns which unit of query rows for a whole launch (fixed ownership is what makes the
 * merge over waves lock-free).  Without a plan ownership is arithmetic (unit id modulo grid, or
 * balanced pairs for causal runs); that leaves CTAs unevenly loaded when each holds only a few
 * units of different length.  A plan assigns units longest-first to the least loaded CTA, the
 * weight of a unit being the key blocks it visits over all waves.  The reference balances the same
 * work dynamically with a tile counter and a lock per query tile
 * (syncopate/computation/attn/template.py:80-121, :339-349). */
#define SYN_ATTN_PLAN_MAX_GRID 160
#define SYN_ATTN_PLAN_MAX_UNITS 2048
typedef struct syn_attn_plan {
  int32_t grid;       /* CTAs the plan was made for */
  int32_t unit_rows;  /* query rows per unit (128 or 256) */
  int32_t num_units;  /* Z * Hq * ceil(Sq / unit_rows) */
  uint16_t start[SYN_ATTN_PLAN_MAX_GRID + 1]; /* CTA c owns units[start[c] .. start[c + 1]) */
  uint16_t units[SYN_ATTN_PLAN_MAX_UNITS];    /* unit id = (z * Hq + h) * units_per_head + index */
  /* visits[2 * unit + t]: in how many waves query tile t (0 / 1) of the unit takes part (has a
   * visible key block); what tells the producer role of syn_attention a tile's last visit. */
  uint8_t visits[2 * SYN_ATTN_PLAN_MAX_UNITS];
} syn_attn_plan;

/* Fills `out` for the launch that `args` + `sched` describe (pointers to tensors are not used).
 * `q_pos_host` / `kv_pos_host` are host copies of args->q_pos / args->kv_pos (NULL where those are
 * NULL).  Host work proportional to units x waves x key blocks: call once per configuration and
 * keep the result.  SYN_ERR_TOO_LARGE when there are more units than the plan holds (arithmetic
 * ownership balances such launches well enough). */
int syn_attention_plan(const syn_attn_args* args, const syn_schedule* sched, const int32_t* q_pos_host,
                       const int32_t* kv_pos_host, syn_attn_plan* out);

/* One 2-D strided copy for the kernel's comm warps: `rows` rows of `row_bytes` bytes from
 * bufs[src_buf].ptrs[src_rank] + src_offset (pitch src_pitch) to bufs[dst_buf].ptrs[dst_rank] +
 * dst_offset (pitch dst_pitch); one end must be this rank.  When it has landed,
 * flags.ptrs[flag_rank][flag] is raised to signal_value (flag < 0: nothing).  Addresses, pitches
 * and row_bytes must be multiples of 16.  This is the N-D box form of the reference's SMCopyOp
 * (syncopate/communication/comm_runtime/operations.py:20-33) cut into 2-D pieces. */
typedef struct syn_copy_op {
  int32_t src_rank, dst_rank;
  int32_t src_buf, dst_buf;
  uint64_t src_offset, dst_offset;
  uint64_t src_pitch, dst_pitch;
  uint32_t rows, row_bytes;
  int32_t flag_rank, flag;
  /* SMCopyOp.reduce_op (operations.py:31, executed by tma_persistent_copy.py:129-169 in the
   * reference): 0 = plain copy; 1 = dst += src for 16-bit elements of type `dtype` (SYN_DTYPE_*),
   * performed as vector reductions at the memory that owns dst, so reducing copies from several
   * ranks into the same bytes may overlap in time; every addition rounds to the element type.
   * Only syn_copy executes reducing copies (the kernels' comm warps move bytes and do not add). */
  int32_t reduce;
  int32_t dtype;
} syn_copy_op;

typedef struct syn_attn_comm {
  int32_t num_ops;
  const syn_copy_op* ops;  /* host array, executed in order, each op spread over all CTAs */
  int32_t num_bufs;
  syn_symm bufs[4];
  syn_symm flags;          /* uint64 flag arrays */
  uint32_t* counters;      /* device uint32[SYN_MAX_COMM_OPS], zero before the first call */
} syn_attn_comm;

/* Stand-alone SM copy: executes `comm->ops` in order on `num_sms` CTAs (0 = all) and raises each
 * op's flag when it has landed; pushes (dst on a peer) and pulls alike.  Replaces the reference's
 * persistent copy kernels for SMCopyOp records (comm_runtime/tma_persistent_copy.py:114-171). */
int syn_copy(const syn_attn_comm* comm, int num_sms, uint64_t signal_value, uint64_t timeout_ns, int32_t* status,
             void* stream);

/* `comm` may be NULL (data already in place; flags, if any, raised by somebody else). */
int syn_attention(const syn_attn_args* args, const syn_schedule* sched, const syn_attn_comm* comm, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SYNCOPATE_B200_H */
