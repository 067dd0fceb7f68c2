/*
 * C ABI of the sm_100a advantage library (libpuff_advantage_sm100.so).
 *
 * Plain pointers and sizes only: no torch types, no C++ types, no exceptions.
 * Every entry point returns 0 on success, a negative PUFF_ERR_* code when an
 * argument is rejected before anything is launched, or a positive cudaError_t
 * value when the CUDA runtime reports a failure.  Nothing here falls back to
 * the CPU: without an sm_100 device every launch returns an error.
 *
 * The recurrence (one [horizon] row per segment, walked backwards, A starts 0):
 *     nn    = 1 - dones[t+1]
 *     rho   = min(importance[t], rho_clip);   c = min(importance[t], c_clip)
 *     delta = rho * (rewards[t+1] + gamma*values[t+1]*nn - values[t])
 *     A     = delta + gamma*lambda*c*A*nn;     advantages[t] = A
 * for t = horizon-2 ... 0.  advantages[:, horizon-1] is never written.
 */
#ifndef PUFF_ADVANTAGE_H_
#define PUFF_ADVANTAGE_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes (negative: rejected before launch) ---------------------- */
#define PUFF_OK                 0
#define PUFF_ERR_NULL          -1   /* a required pointer is NULL                 */
#define PUFF_ERR_SHAPE         -2   /* negative num_segments / horizon            */
#define PUFF_ERR_VARIANT       -3   /* unknown variant                            */
#define PUFF_ERR_ALIGN         -4   /* a pointer is not 4-byte aligned            */
#define PUFF_ERR_ALIAS         -5   /* advantages / seg_abs_sum overlap an input  */
#define PUFF_ERR_ARCH          -6   /* current device is not compute capability 10.x */
#define PUFF_ERR_DRIVER        -7   /* cuTensorMapEncodeTiled unavailable / failed */
#define PUFF_ERR_DEVICE_WAIT   -8   /* a bounded in-kernel wait gave up (see _device_status) */
#define PUFF_ERR_WORKSPACE     -9   /* scratch / workspace too small or missing   */
#define PUFF_ERR_SIZE         -10   /* size beyond what the entry point supports  */
#define PUFF_ERR_DEVICE_BOUNDS -11  /* debug builds (PUFF_DEBUG_BOUNDS): a kernel formed an out-of-range index (see _device_status) */

/* ---- kernel variants ----------------------------------------------------- */
#define PUFF_VARIANT_AUTO       0   /* pick from (num_segments, horizon, alignment): a bit-exact serial kernel,
                                     * except for few long rows (num_segments < 24 x SM count and horizon >= 512)
                                     * with gamma*lambda*c_clip <= 1, which take the scan kernel and its error bar */
#define PUFF_VARIANT_SERIAL     1   /* one thread per row, reference operation order: bit-exact */
#define PUFF_VARIANT_SCAN       2   /* affine-pair scan along the horizon: |a-b| <= max(1e-6, 1e-5|b|) */
#define PUFF_VARIANT_GENERIC    3   /* serial, direct global loads; any alignment, any horizon  */

/* Kernel actually used by the last launch of the calling thread (tests/bench). */
#define PUFF_KERNEL_NONE        0
#define PUFF_KERNEL_TMA2D       1   /* serial, 2-D TMA tiles, 128B-swizzled shared memory */
#define PUFF_KERNEL_BULK1D      2   /* serial, 1-D bulk-copied dense row tiles             */
#define PUFF_KERNEL_SCAN        3
#define PUFF_KERNEL_GENERIC     4

/*
 * The advantage op on DEVICE buffers, asynchronous on `cuda_stream`.
 *
 * Replaces the reference launcher compute_puff_advantage_cuda
 * (pufferlib/extensions/cuda/pufferlib.cu:53-82) and its kernel
 * puff_advantage_kernel (cu:41-51) / puff_advantage_row_cuda (cu:7-20);
 * argument meaning follows cu:53-55 with gamma..c_clip already narrowed to
 * float as at cu:70-73.  All five arrays are row-major contiguous
 * [num_segments, horizon] fp32 on the current device.
 *
 * seg_abs_sum (nullable, [num_segments] fp32, device): when non-NULL the same
 * kernel also writes sum_t |advantages[s, t]| over t = 0..horizon-2, the
 * quantity `advantages.abs().sum(axis=1)` of pufferl.py:359 computes from a
 * zero-initialised buffer.
 *
 * Differences from the reference launcher, all deliberate: runs on the
 * caller's stream instead of the legacy default stream (cu:64); 64-bit
 * offsets (cu:48 overflows int at 2^31 elements); num_segments == 0 or
 * horizon < 2 return PUFF_OK without a launch (cu:62 launches a 0-block grid,
 * which is a CUDA error); no allocation, no host synchronisation.
 *
 * Every wait inside the kernels is bounded.  A wait that gives up records
 * PUFF_ERR_DEVICE_WAIT in a per-device status word and the kernel returns with
 * part of the output unwritten; this asynchronous entry point cannot report
 * that.  A caller that needs to know polls puff_advantage_sm100_device_status
 * at its own synchronisation points (the synchronous _host entry point does it
 * itself and returns the code).
 *
 * The first call on each device (from any entry point of this header) queries
 * the device once and raises the kernels' shared-memory limits; make it during
 * set-up, before a stream is being captured.  Later calls only encode tensor
 * maps on the host and launch.
 */
int puff_advantage_sm100_launch(const float* values, const float* rewards,
                                const float* dones, const float* importance,
                                float* advantages, float* seg_abs_sum,
                                float gamma, float lambda, float rho_clip, float c_clip,
                                long long num_segments, long long horizon,
                                int variant, void* cuda_stream);

/*
 * puff_advantage_sm100_launch with option flags.
 *
 * PUFF_FLAG_ZERO_LAST_COLUMN: the op owns the whole output and also writes
 * advantages[:, horizon-1] = 0, so `advantages` may be uninitialised memory.
 * This is the contract change that lets the trainer drop the `torch.zeros`
 * fill in front of every call (pufferl.py:352-353: one extra 4 B/element write
 * pass and one launch per minibatch); the 9-argument reference contract, which
 * leaves that column alone, stays on puff_advantage_sm100_launch (flags = 0).
 */
#define PUFF_FLAG_ZERO_LAST_COLUMN 1u
int puff_advantage_sm100_launch_ex(const float* values, const float* rewards,
                                   const float* dones, const float* importance,
                                   float* advantages, float* seg_abs_sum,
                                   float gamma, float lambda, float rho_clip, float c_clip,
                                   long long num_segments, long long horizon,
                                   int variant, unsigned flags, void* cuda_stream);

/*
 * The same op on HOST buffers (pinned memory recommended), synchronous.
 *
 * Stands where the reference's host-tensor path stands: the Python wrapper's
 * `.cpu()` route (pufferl.py:666-678) and compute_puff_advantage_cpu
 * (pufferlib/extensions/pufferlib.cpp:75-85), i.e. "the caller holds host
 * memory".  Rows are cut into blocks that are copied in, processed and copied
 * out on rotating streams so that both PCIe directions and the kernel overlap.
 * h_advantages[:, horizon-1] is left untouched.  The device staging workspace
 * is allocated on first use and cached per device; puff_advantage_sm100_host_release
 * frees it.  Bytes moved: 16*S*H host->device, 4*S*(H-1) (+4*S) device->host.
 * Returns PUFF_ERR_DEVICE_WAIT (and clears the status word) when a bounded wait
 * inside one of its kernels gave up: the output is then incomplete.
 */
int puff_advantage_sm100_host(const float* h_values, const float* h_rewards,
                              const float* h_dones, const float* h_importance,
                              float* h_advantages, float* h_seg_abs_sum,
                              float gamma, float lambda, float rho_clip, float c_clip,
                              long long num_segments, long long horizon,
                              int variant, int device);
int puff_advantage_sm100_host_release(int device);
/* The copies of puff_advantage_sm100_host without its kernels: same blocks,
 * same streams, same bytes in both directions, nothing computed (h_advantages
 * receives whatever the staging buffers hold).  For benchmarks: the time the
 * host-buffer path cannot go below on a given machine. */
int puff_advantage_sm100_host_copies_only(const float* h_values, const float* h_rewards,
                                          const float* h_dones, const float* h_importance,
                                          float* h_advantages, float* h_seg_abs_sum,
                                          long long num_segments, long long horizon, int device);

/*
 * Prioritised-replay weights from the fused per-segment sums, on DEVICE
 * buffers, asynchronous on `cuda_stream`.  Replaces the eager torch sequence
 * of pufferl.py:359-361:
 *     w = nan_to_num(seg_abs_sum ** alpha, 0, 0, 0)
 *     p = (w + 1e-6) / (sum(w) + 1e-6)
 * split in two launches so that a sharded caller can all-reduce the sum in
 * between:
 *   _weights : writes weights[s] and the fp64 total sum(w) into *total_w
 *              (deterministic two-level reduction through `scratch`).
 *   _probs   : writes probs[s] = (weights[s] + 1e-6) / (*total_w + 1e-6).
 * scratch: device memory, at least puff_priorities_sm100_scratch_bytes(S)
 * bytes, 8-byte aligned, owned by the caller; no allocation happens here.
 */
size_t puff_priorities_sm100_scratch_bytes(long long num_segments);
int puff_priorities_sm100_weights(const float* seg_abs_sum, float* weights,
                                  double* total_w, float alpha,
                                  long long num_segments,
                                  void* scratch, size_t scratch_bytes,
                                  void* cuda_stream);
int puff_priorities_sm100_probs(const float* weights, const double* total_w,
                                float* probs, long long num_segments,
                                void* cuda_stream);

/*
 * The same two steps for segments sharded over several GPUs, with the exchange
 * of the weight total done by the kernels themselves instead of a collective
 * library call between them.  (The reference never shards this op: its DDP
 * ranks own private buffers, pufferl.py:913-939, and the only torch.distributed
 * calls near it are 1-element all-reduces for logging, pufferl.py:708-714.
 * This is the layout of the multi-GPU benchmark: contiguous row blocks per
 * rank, one process per GPU or one process driving several.)
 *
 * A puff_exchange is one rank's end of the exchange: a mailbox of a few hundred
 * bytes in that rank's device memory that every other rank can store into.
 *   _create   allocates it on the current device (set-up time; this is the only
 *             allocation) and, when handle_out is non-NULL, fills it with
 *             PUFF_EXCHANGE_HANDLE_BYTES bytes that identify the mailbox to
 *             other PROCESSES on the same machine (a CUDA IPC handle).
 *   _connect  takes the handles of all `world` ranks, indexed by rank, as one
 *             array of world * PUFF_EXCHANGE_HANDLE_BYTES bytes (exchange them
 *             with whatever the host program has: torch.distributed, MPI, a
 *             file) and maps the peers' mailboxes.
 *   _connect_pointers  the same for ranks that live in ONE process: device
 *             pointers from puff_exchange_sm100_mailbox(), indexed by rank
 *             (peer access between the devices must be enabled by the caller).
 *   _set_wait_ns  the bound of the in-kernel wait (default 2 s).
 *   _destroy  synchronises the device and frees everything.  Call it only after
 *             every rank has finished its last exchange (a host-side barrier):
 *             a peer whose kernel still stores into a freed mailbox would fault.
 *
 *   puff_priorities_sm100_weights_push   weights[s] as puff_priorities_sm100_weights,
 *             then the local fp64 total is stored into every rank's mailbox
 *             (plain stores over NVLink to peer-mapped memory, fence, flag);
 *             one launch: the CTA that finishes last adds the per-CTA sums in
 *             index order and pushes.
 *   puff_priorities_sm100_probs_gathered  waits until all `world` totals of the
 *             current round sit in this rank's own mailbox, adds them in rank
 *             order (identical on every rank), writes the global total to
 *             *total_w (nullable) and probs[s] = (weights[s] + 1e-6) / (total + 1e-6).
 * Every rank must issue the same sequence of _weights_push / _probs_gathered
 * pairs, each rank on one stream.  A rank with num_segments == 0 still takes
 * part.  The wait is bounded: when a peer's total has not arrived in time the
 * kernel records PUFF_ERR_DEVICE_WAIT in the device status word
 * (puff_advantage_sm100_device_status) and returns without writing probs.
 */
#define PUFF_EXCHANGE_HANDLE_BYTES 64
typedef struct puff_exchange puff_exchange;
int puff_exchange_sm100_create(int rank, int world, void* handle_out, puff_exchange** exchange);
int puff_exchange_sm100_connect(puff_exchange* exchange, const void* all_handles);
int puff_exchange_sm100_connect_pointers(puff_exchange* exchange, void* const* mailboxes);
void* puff_exchange_sm100_mailbox(puff_exchange* exchange);
int puff_exchange_sm100_set_wait_ns(puff_exchange* exchange, unsigned long long wait_ns);
int puff_exchange_sm100_destroy(puff_exchange* exchange);
int puff_priorities_sm100_weights_push(const float* seg_abs_sum, float* weights, float alpha,
                                       long long num_segments, void* scratch, size_t scratch_bytes,
                                       puff_exchange* exchange, void* cuda_stream);
int puff_priorities_sm100_probs_gathered(const float* weights, double* total_w, float* probs,
                                         long long num_segments, puff_exchange* exchange,
                                         void* cuda_stream);

/*
 * Minibatch gather and advantage normalisation, on DEVICE buffers, asynchronous
 * on `cuda_stream`.  Replaces the eager torch sequence of pufferl.py:363,
 * 373-375 and 408-409 for the sampled segment indices idx[mb_segments]:
 *     mb_prio     = (num_segments * prio_probs[idx]) ** -anneal_beta   [mb_segments]
 *     mb_values   = values[idx]                                        [mb_segments, horizon]
 *     mb_returns  = advantages[idx] + mb_values
 *     mb_adv_raw  = advantages[idx]
 *     mb_adv_norm = mb_prio[:, None] * (mb_adv_raw - mean) / (std + 1e-8)
 * with mean and the unbiased std taken over all gathered elements (fp64
 * accumulation through `scratch`, fixed order).  idx is int64 on the device; an
 * index outside [0, num_segments) yields zero rows in all four outputs and
 * mb_prio = 0 (its zeros still count in mean and std), and raises the flag that
 * puff_minibatch_sm100_bad_index() returns (and clears) after synchronising.
 * scratch: at least puff_minibatch_sm100_scratch_bytes(mb_segments) bytes,
 * 8-byte aligned, caller-owned.
 *
 * _gather_ex takes the N of `(N * prio_probs[idx]) ** -beta` separately, as
 * prio_segments >= num_segments: a caller whose segments are sharded over
 * several GPUs passes its local rows as num_segments (the bound of idx) and
 * the global segment count, over which prio_probs was normalised, as
 * prio_segments.  _gather is _gather_ex with prio_segments = num_segments.
 */
size_t puff_minibatch_sm100_scratch_bytes(long long mb_segments);
int puff_minibatch_sm100_gather(const float* advantages, const float* values,
                                const float* prio_probs, const long long* idx,
                                float* mb_values, float* mb_returns, float* mb_adv_raw,
                                float* mb_adv_norm, float* mb_prio, float anneal_beta,
                                long long num_segments, long long horizon,
                                long long mb_segments, void* scratch, size_t scratch_bytes,
                                void* cuda_stream);
int puff_minibatch_sm100_gather_ex(const float* advantages, const float* values,
                                   const float* prio_probs, const long long* idx,
                                   float* mb_values, float* mb_returns, float* mb_adv_raw,
                                   float* mb_adv_norm, float* mb_prio, float anneal_beta,
                                   long long num_segments, long long prio_segments,
                                   long long horizon, long long mb_segments,
                                   void* scratch, size_t scratch_bytes, void* cuda_stream);
int puff_minibatch_sm100_bad_index(void);

/*
 * Rollout writer, on DEVICE buffers, asynchronous on `cuda_stream`: one
 * environment step of rows [row_begin, row_begin + num_rows) into column
 * `column` of the [num_segments, horizon] experience buffers.  Replaces
 * pufferl.py:275 (clamp of the rewards to [-reward_clip, reward_clip];
 * reward_clip <= 0 disables it) and :294-296 (rewards, terminals = done as
 * 0/1 float, values).  step_dones is one byte per row (torch.bool).
 */
int puff_rollout_sm100_write(float* rewards, float* terminals, float* values,
                             const float* step_rewards, const unsigned char* step_dones,
                             const float* step_values, long long row_begin,
                             long long num_rows, long long column,
                             long long num_segments, long long horizon,
                             float reward_clip, void* cuda_stream);

/*
 * puff_priorities_sm100_weights for callers that cannot supply scratch.
 * (No counterpart in the reference, which allocates freely through torch.)
 *
 * Some hosts of this library have no way to allocate device memory at the
 * point of the call: a C or FFI caller inside a trainer whose GPU memory is
 * already fully owned by the policy, the experience buffers and the
 * framework's caching allocator, or a wrapper that holds no allocator handle
 * at all.  There cudaMalloc can fail, and even when it works it stalls the
 * device between minibatches.  This variant takes the same inputs and outputs
 * as puff_priorities_sm100_weights but keeps its partial sums in a fixed array
 * inside the library image (4 KB per GPU that loads the library, held until
 * the process exits), and calls no allocation routine of CUDA or any other
 * library.
 *
 * Limits and rules:
 *  - num_segments <= PUFF_NOALLOC_MAX_SEGMENTS, otherwise PUFF_ERR_SIZE and
 *    nothing is launched.
 *  - The first call on each device looks up the array's device address (that
 *    device must be current, as for every launch here).  Make that first call
 *    during set-up, before any stream capture is started.
 *  - All calls on a device share the one array.  Calls are safe back to back
 *    on one stream; two calls that can overlap on the GPU (different streams
 *    without an ordering between them) race on it and must be serialised by
 *    the caller.  Nothing needs clearing between calls: each call overwrites
 *    every entry it later reads.
 * Results are identical to puff_priorities_sm100_weights.
 */
#define PUFF_NOALLOC_MAX_SEGMENTS 524288LL
int puff_priorities_sm100_weights_noalloc(const float* seg_abs_sum, float* weights,
                                          double* total_w, float alpha,
                                          long long num_segments, void* cuda_stream);

/* ---- introspection ------------------------------------------------------- */
/* Human-readable text for a return code of any entry point above. */
const char* puff_advantage_sm100_strerror(int code);
/* PUFF_KERNEL_* used by the calling thread's most recent _launch. */
int puff_advantage_sm100_last_kernel(void);
/* Number of kernels this library has launched in this process so far. */
long long puff_advantage_sm100_launch_count(void);
/* Synchronises the current device and returns (then clears) the device-side
 * status word: 0, or PUFF_ERR_DEVICE_WAIT when a bounded wait inside a kernel
 * gave up.  The asynchronous launch path never calls it; callers do, at their
 * own synchronisation points. */
int puff_advantage_sm100_device_status(void);
/* Writes `value` into the current device's status word from the host (a plain
 * copy, nothing is launched): lets tests of a caller's error handling see
 * PUFF_ERR_DEVICE_WAIT without making any kernel wait.  Returns 0 or a
 * cudaError_t. */
int puff_advantage_sm100_inject_status(int value);
/* Tuning knobs for tests and sweeps (process-wide; value -1 restores the
 * automatic choice; returns the previous value, or PUFF_ERR_VARIANT for an
 * unknown knob).  The initial values come from the environment variables named
 * beside each knob, read once. */
#define PUFF_TUNE_FORCE_KERNEL  0   /* PUFF_ADV_FORCE_KERNEL: a PUFF_KERNEL_* to use whenever it applies */
#define PUFF_TUNE_STAGES        1   /* PUFF_ADV_STAGES: ring depth of the single-warp tma2d kernel (2, 3, 4) */
#define PUFF_TUNE_WS_STAGES     2   /* PUFF_ADV_WS: 0 = single-warp tma2d, N = warp-specialised with N stages */
#define PUFF_TUNE_CTAS_PER_SM   3   /* PUFF_ADV_CTAS_PER_SM: cap on resident CTAs per SM of the tma2d kernels */
#define PUFF_TUNE_LOAD_GROUP    4   /* PUFF_ADV_GROUP: chunks whose loads the warp-specialised producer issues together */
#define PUFF_TUNE_SCAN_THREADS  5   /* PUFF_ADV_SCAN_THREADS: threads per row of the scan kernel (power of two, 32..1024; default by row count and horizon) */
#define PUFF_TUNE_RESERVE_SMS   6   /* PUFF_ADV_RESERVE_SMS: SMs the persistent (warp-specialised) grids leave free for other streams' kernels */
#define PUFF_TUNE_TILE_ROWS     7   /* PUFF_ADV_TILE_ROWS: cap on the rows per tile of the bulk1d kernels (4, 8, 16, 32) */
#define PUFF_TUNE_PDL           8   /* PUFF_ADV_PDL: 0 = launch without programmatic stream serialization, 2 = only the advantage kernels with it */
#define PUFF_TUNE_SCAN_WIDE     9   /* PUFF_ADV_SCAN_WIDE: 0 = the scan kernel always takes four columns per thread and pass */
#define PUFF_TUNE_B1_WARP_TEAMS 10  /* PUFF_ADV_B1_WARP_TEAMS: 0 = the one-stage bulk1d kernel always works with one tile per CTA, never one per warp */
#define PUFF_TUNE_COUNT        11
int puff_advantage_sm100_set_tuning(int knob, int value);
/* Library version, "major.minor". */
const char* puff_advantage_sm100_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PUFF_ADVANTAGE_H_ */
