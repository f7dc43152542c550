/* b200amp.h: C ABI of the B200 (sm_100a) mixed-precision AdamW optimizer step.
 *
 * The library replaces one path of cuda-transformer: the AMP optimizer step
 * that FastGPT::optimizer_step (cuda/gpt_fast.cu:438-450) runs every training
 * step. Every entry point takes plain pointers, sizes and a stream, returns an
 * int status (0 = ok) and never calls exit(): the reference's launchers print
 * and exit(1) on a CUDA error (cuda/common.h:10-20); a caller that wants that
 * behaviour wraps the status (compat/fast_shim.h does).
 *
 * Two families of entry points:
 *
 *   compat  (…_f32)  same arguments and in/out behaviour as the reference's
 *                    launchers in cuda/kernels/fast.h:136-166: fp32 gradient
 *                    arena, unscaled IN PLACE, partial[512] owned by the caller.
 *   native  (…_f16)  the gradient arena is fp16 and read-only (2 B/param in
 *                    pass 1, 28 B/param in pass 2); the unscale is folded into
 *                    both passes, the finalize into the tail of pass 1. A range
 *                    of the arena (a ZeRO-1 shard) is addressed by passing the
 *                    shard's pointers plus its global offset.
 *
 * Ownership: the caller owns every device buffer, as in the reference
 * (cuda/common.h:51-127). The ops allocate nothing; the only exceptions are
 * b200amp_lr_on_gpu (8 bytes, as cuda/kernels/scaler.cu:100-110 does) and the
 * graph helpers (the graph objects themselves).
 *
 * Streams: everything is enqueued on the stream given, without a host sync,
 * and can be captured into a CUDA graph (changing scalars live in the step
 * state in device memory, cuda/graph.h:4-8).
 */
#ifndef B200AMP_H
#define B200AMP_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported with default visibility; everything else in the library is hidden. */
#if defined(__GNUC__)
#define B200AMP_API __attribute__((visibility("default")))
#else
#define B200AMP_API
#endif

/* A cudaStream_t, passed as an opaque pointer so this header needs no CUDA headers. */
typedef void *b200amp_stream;

/* ---------------------------------------------------------------- status codes */
enum
{
    B200AMP_OK = 0,
    B200AMP_ERR_ARG = 1,        /* null pointer, bad size, misaligned pointer, table too long */
    B200AMP_ERR_CUDA = 2,       /* a CUDA runtime call or a launch failed; b200amp_last_error() has the text */
    B200AMP_ERR_DEVICE = 3,     /* the current device is not compute capability 10.x */
    B200AMP_ERR_LIMIT = 4       /* a size beyond a stated maximum of the entry point */
};

/* Text of the last error on the calling thread ("" if none). */
B200AMP_API const char *b200amp_last_error(void);
/* Library version, "major.minor.patch". */
B200AMP_API const char *b200amp_version(void);
/* B200AMP_OK if the current device can run the kernels (compute capability 10.x). */
B200AMP_API int b200amp_device_check(void);

/* ---------------------------------------------------------------- types
 * Bit-compatible with the reference's structs (cuda/kernels/fast.h:104-133,
 * 153-158): 15 x 4 bytes = 60 B, 11 x 4 bytes = 44 B, and 24 B with padding.
 * sizeof(b200amp_step_state) is also the reference's checkpoint ABI
 * (cuda/checkpoint.cu:102-103). */
typedef struct b200amp_step_state
{
    float loss_scale;       /* S, multiplies dlogits at the start of backward */
    float inv_scale;        /* 1 / S of THIS step */
    int good_steps;         /* finite steps in a row since S last changed */
    int found_inf;          /* this step's gradients held an inf or NaN: the step is skipped */
    int skipped;            /* steps skipped so far */
    int step;               /* steps so far, skipped ones included (drives the lr schedule) */
    int adam_t;             /* AdamW steps taken (skipped steps do not count) */
    float lr;               /* of this step */
    float grad_norm;        /* of the unscaled gradients, before clipping */
    float clip_coef;        /* min(1, clip / (norm + 1e-6)) */
    float step_size;        /* lr / (1 - beta1^t) */
    float bc2_sqrt;         /* sqrt(1 - beta2^t) */
    float decay;            /* 1 - lr * weight_decay */
    float loss;             /* written by the caller's forward pass; carried, never read here */
    int n_valid;            /* written by the caller's forward pass; carried, never read here */
} b200amp_step_state;

typedef struct b200amp_schedule
{
    float lr, min_lr;
    int warmup_steps, max_steps;
    float beta1, beta2;
    float weight_decay;
    float grad_clip;
    int growth_interval;    /* finite steps in a row before S doubles (2000 in the reference) */
    int dynamic_scale;      /* 0: S never changes */
    int decay_steps;        /* 0: cosine after warmup; > 0: WSD */
} b200amp_schedule;

typedef struct b200amp_tensor_info
{
    long long offset;       /* first element of the tensor in the arena */
    long long count;
    int decay;              /* 1: weight decay applies (>= 2-D weights), 0: it does not */
} b200amp_tensor_info;

/* Set-up check of a HOST copy of the tensor table (the kernels read the device copy and, like the
 * reference's, trust it): 1..B200AMP_MAX_TENSORS entries, offsets multiples of 4 and ascending,
 * counts positive, no entry reaching into the next, and, when n > 0, none past the n elements of
 * the arena. The reference builds its table in code (cuda/gpt_fast.cu:105-115) and checks nothing;
 * a table that arrives from a file or another program should go through this once. Host only:
 * no CUDA call. */
B200AMP_API int b200amp_check_tensor_table(const b200amp_tensor_info *host_table, int ntensors, long long n);

#define B200AMP_NORM_BLOCKS 512     /* partial[] length of the compat path (cuda/kernels/fast.h:150) */
#define B200AMP_MAX_TENSORS 1024    /* longest tensor table (cuda/kernels/fast.h:163) */

/* ---------------------------------------------------------------- compat entry points */

/* Replaces initial_state (cuda/kernels/scaler.cu:21-29). Host only: a zeroed
 * state with loss_scale = scale, inv_scale = 1/scale, clip_coef = decay = 1. */
B200AMP_API int b200amp_initial_state(float scale, b200amp_step_state *out);

/* Replaces begin_step (cuda/kernels/scaler.cu:31-35,173-177):
 * found_inf = 0, inv_scale = 1 / loss_scale. st is a device pointer. */
B200AMP_API int b200amp_begin_step(b200amp_step_state *st, b200amp_stream s);

/* Replaces unscale_and_norm (cuda/kernels/scaler.cu:39-66,179-184).
 * grads[n] fp32 is multiplied by st->inv_scale in place; st->found_inf is set
 * to 1 if any result is not finite; partial[512] receives fp32 sums of squares
 * whose total is the squared norm. n > 0 and n % 4 == 0; grads 16-byte aligned. */
B200AMP_API int b200amp_unscale_and_norm_f32(float *grads, long long n, b200amp_step_state *st, float *partial,
                                 b200amp_stream s);

/* Replaces finalize_step (cuda/kernels/scaler.cu:115-171,186-192): norm, clip
 * coefficient, lr of this step, skip decision, loss-scale backoff/growth, bias
 * corrections, history[step % history_len] = state (history may be null), step++.
 * cfg is a HOST pointer, read before the call returns (the reference passes it by value). */
B200AMP_API int b200amp_finalize_step(b200amp_step_state *st, const float *partial, const b200amp_schedule *cfg,
                          b200amp_step_state *history, int history_len, b200amp_stream s);

/* Replaces adamw_multi (cuda/kernels/adamw_multi.cu:20-108): one launch over the
 * flat arena; does nothing when st->found_inf is set. grads are the UNSCALED fp32
 * gradients. params_x (fp16, may be null) receives the rounded-to-nearest copy of
 * the new parameters. n > 0, n % 4 == 0, every tensor offset a multiple of 4,
 * 1 <= ntensors <= 1024; tensors and st are device pointers. */
B200AMP_API int b200amp_adamw_multi_f32(float *params, void *params_x, const float *grads, float *m, float *v, long long n,
                            const b200amp_tensor_info *tensors, int ntensors, const b200amp_step_state *st,
                            float beta1, float beta2, float eps, b200amp_stream s);

/* Replaces lr_on_gpu (cuda/kernels/scaler.cu:95-110): the lr of 0-based step,
 * computed on the device in double. Synchronous; allocates and frees 8 bytes. */
B200AMP_API int b200amp_lr_on_gpu(int step, const b200amp_schedule *cfg, double *out);

/* Replaces cast_to_x of the fp16 build (cuda/kernels/fused.cu:285-292,319-323):
 * out[i] = fp16(in[i]), round to nearest even. Used to initialise the fp16
 * weight arena. Any n >= 0; pointers need only their natural alignment. */
B200AMP_API int b200amp_cast_to_x(void *out_f16, const float *in, long long n, b200amp_stream s);

/* ---------------------------------------------------------------- native entry points
 * The fp16 gradient arena holds loss-scaled gradients, as the backward pass
 * leaves them; it is never written. n % 8 == 0 and every pointer 32-byte
 * aligned (16 for the fp16 arenas). The workspace is device memory of
 * b200amp_workspace_bytes() bytes, zeroed once with b200amp_workspace_init();
 * after that the kernels keep it consistent themselves (the ticket counter
 * resets itself, so graph replays need no memset). */
B200AMP_API size_t b200amp_workspace_bytes(void);
B200AMP_API int b200amp_workspace_init(void *workspace, b200amp_stream s);

/* Pass 1 on [grads16, grads16 + n): sum of squares of the unscaled gradients
 * (g * 1/st->loss_scale) and the inf/NaN flag. Reads 2 B/param, writes nothing
 * but the workspace: on return of the kernel the first two doubles of the
 * workspace are {sum of squares, flag (0.0 or 1.0)}. The summation order depends
 * on n only (fixed virtual grid), never on the launch, so a replay gives the
 * same bits. No reference counterpart takes fp16 gradients; the arithmetic is
 * that of cuda/kernels/scaler.cu:39-66 on float(fp16 gradient). */
B200AMP_API int b200amp_pass1_f16(const void *grads16, long long n, const b200amp_step_state *st, void *workspace,
                      b200amp_stream s);

/* Pass 1 for callers that cannot allocate device memory and have none to spare for a
 * workspace (everything was handed to their own arenas at start-up, or they run inside
 * another framework's memory pool, or cudaMalloc's device-wide synchronisation is not
 * acceptable in their step loop). This entry point has no counterpart in the reference.
 * Same arithmetic and summation order as b200amp_pass1_f16, so the same bits; the scratch
 * is a 37,920-byte array inside the library image (each GPU that loads the library holds it
 * until the process exits). On return of the stream work sums_out[0..1] (DEVICE memory,
 * caller-owned, 8-byte aligned) hold {sum of squares, flag as 0.0 / 1.0}.
 *   - Calls cudaMalloc / cudaFree or any allocating routine: never.
 *   - n at most 4,294,967,296 elements; larger n returns B200AMP_ERR_LIMIT (use
 *     b200amp_pass1_f16 with your own workspace).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress). Make that first call outside any stream capture.
 *   - All calls on a device share the one array: two calls whose GPU work overlaps (different
 *     streams, no ordering between them) race on it. Serialise them. */
B200AMP_API int b200amp_pass1_f16_static(const void *grads16, long long n, const b200amp_step_state *st,
                                         double *sums_out, b200amp_stream s);

/* The step before the path: the bridge from the reference's fp32 gradient arena to the fp16
 * arena. grads32[n] holds loss-scaled fp32 gradients as the reference's backward pass leaves
 * them (cuda/gpt_fast.cu:455-457, cuda/kernels/gemm_common.cuh:11). One sweep writes
 * grads16 = fp16(grads32) (round to nearest even; out-of-range values become inf and skip the
 * step), computes pass 1 on exactly those fp16 values (workspace as b200amp_pass1_f16), and,
 * if clear_source != 0, zeroes grads32 in place, which replaces the reference's per-step
 * grads.zero memset. With cfg != null the finalize runs in the same launch (cfg, history and
 * history_len as b200amp_pass1_finalize_f16); with cfg == null only {sum, flag} are
 * published, as b200amp_pass1_f16 does. n % 8 == 0; grads32 32-byte, grads16 16-byte aligned. */
B200AMP_API int b200amp_cast_pass1_f32(float *grads32, void *grads16, long long n, int clear_source,
                                       b200amp_step_state *st, void *workspace, const b200amp_schedule *cfg,
                                       b200amp_step_state *history, int history_len, b200amp_stream s);

/* Finalize from nranks pairs {sum of squares, flag} laid out rank after rank
 * (device memory, e.g. the output of an all-gather of every rank's first 16
 * workspace bytes). Pairs are added in rank order, so every rank computes the
 * same bits. Also sets st->inv_scale = 1/loss_scale (of this step) and
 * st->found_inf. Otherwise cuda/kernels/scaler.cu:131-170. */
B200AMP_API int b200amp_finalize_sums(b200amp_step_state *st, const double *sums, int nranks, const b200amp_schedule *cfg,
                          b200amp_step_state *history, int history_len, b200amp_stream s);

/* Pass 1 and the finalize in ONE launch (the last block to finish runs the
 * finalize), for an arena held by one GPU. */
B200AMP_API int b200amp_pass1_finalize_f16(const void *grads16, long long n, b200amp_step_state *st, void *workspace,
                               const b200amp_schedule *cfg, b200amp_step_state *history, int history_len,
                               b200amp_stream s);

/* Pass 2 on a range of the arena: clip, AdamW on master/m/v (fp32, updated in
 * place), fp16 weight cast. Reads 14 B/param, writes 14 B/param. All array
 * pointers address the FIRST ELEMENT OF THE RANGE; arena_offset is that
 * element's index in the whole arena (0 for an unsharded arena) and is what
 * the tensor table is searched with. weights16 may be null. Does nothing when
 * st->found_inf is set. Arithmetic per element: cuda/kernels/adamw_multi.cu:20-29,75-89
 * with g = float(fp16 gradient) * st->inv_scale. */
B200AMP_API int b200amp_pass2_f16(float *master, float *m, float *v, const void *grads16, void *weights16, long long n,
                      long long arena_offset, const b200amp_tensor_info *tensors, int ntensors,
                      const b200amp_step_state *st, float beta1, float beta2, float eps, b200amp_stream s);

/* Pass 2 with the decay flags handed over as a kernel parameter instead of a table in device
 * memory. Only a CHANGE of the decay flag matters to the update, so the tensor table reduces to
 * runs of equal flag (a GPT layout: 8 runs per layer + 3): b200amp_decay_runs_build merges a HOST
 * copy of the table (checked as b200amp_check_tensor_table does) into at most B200AMP_MAX_RUNS
 * runs, or returns B200AMP_ERR_LIMIT when there are more (then use b200amp_pass2_f16). The
 * kernel then needs no shared memory and no table-loading prologue. Same arithmetic and the same
 * bits as b200amp_pass2_f16; `runs` is a HOST pointer, read before the call returns. No
 * reference counterpart beyond cuda/kernels/adamw_multi.cu:55-69 (the per-vector table search
 * this replaces). */
#define B200AMP_MAX_RUNS 256
typedef struct b200amp_decay_runs
{
    unsigned int first4[B200AMP_MAX_RUNS];  /* first element of run k, divided by 4 */
    int nruns;
    int flag0;                              /* decay flag of run 0; run k has flag0 ^ (k & 1) */
} b200amp_decay_runs;
B200AMP_API int b200amp_decay_runs_build(const b200amp_tensor_info *host_table, int ntensors,
                                         b200amp_decay_runs *out);
B200AMP_API int b200amp_pass2_f16_runs(float *master, float *m, float *v, const void *grads16, void *weights16,
                                       long long n, long long arena_offset, const b200amp_decay_runs *runs,
                                       const b200amp_step_state *st, float beta1, float beta2, float eps,
                                       b200amp_stream s);

/* ---------------------------------------------------------------- ZeRO-1 with the collectives folded in
 * For R = 1, 2, 4 or 8 GPUs of one NVLink box, with every rank's fp16 gradient arena, fp16
 * weight arena and pair table addressable from every rank (one process with peer access on, or
 * one process per GPU with the buffers mapped through CUDA IPC / symmetric memory: the pointers
 * below are ordinary device pointers of the CALLING process). The reference has no multi-GPU
 * code; per element these are pass 1 and pass 2 above. All remote accesses are plain 128-bit
 * loads and stores, or cudaMemcpyAsync in the ..._ce forms; nothing uses multicast.
 *
 * Ordering between the ranks (gradients of all ranks ready -> rs_pass1; all pairs written ->
 * finalize; all weights written -> the next forward pass) is either the caller's (the plain
 * entry points: a one-process host puts events between the ranks' streams) or the library's
 * (the ..._sync entry points and b200amp_zero1_barrier, below). */

/* Reduce-scatter + pass 1. grads16_by_rank[r] (HOST array of nranks device pointers) is the
 * start of THIS rank's slice in rank r's gradient arena. The slice is averaged over the ranks
 * (fp32 sum in rank order, * 1/nranks, one rounding to fp16) into reduced16 (local, n
 * elements); the squared norm and inf/NaN flag of those stored values go to the workspace
 * (first 16 bytes, as b200amp_pass1_f16) and, if pair_table_by_rank is not null, into entry
 * my_rank of every rank's pair table (pair_table_by_rank[r]: nranks pairs of doubles). */
B200AMP_API int b200amp_rs_pass1_f16(const void *const *grads16_by_rank, int nranks, int my_rank, void *reduced16,
                                     long long n, const b200amp_step_state *st, void *workspace,
                                     double *const *pair_table_by_rank, b200amp_stream s);

/* The same reduction in parts, for a caller that reduces a slice piece by piece (for instance
 * while the next piece is still on its way into a local staging buffer). The slice's norm is
 * summed over a fixed partition into virtual blocks (b200amp_pass1_partition); one call reduces
 * the elements of the virtual blocks vblock_first .. vblock_first + vblock_count - 1 and keeps
 * their partial sums in the workspace. The pointers still address the start of the slice. The
 * call with last_part != 0 must come last on the stream: it adds ALL partials of the slice and
 * writes the pairs, so the calls together give the bits of b200amp_rs_pass1_f16. */
B200AMP_API int b200amp_rs_pass1_f16_part(const void *const *grads16_by_rank, int nranks, int my_rank,
                                          void *reduced16, long long n, int vblock_first, int vblock_count,
                                          int last_part, const b200amp_step_state *st, void *workspace,
                                          double *const *pair_table_by_rank, b200amp_stream s);

/* The fixed partition pass 1 sums over: a range of n elements has *vblocks virtual blocks of
 * *elements_per_vblock elements (the last may be shorter). A function of n alone. Host only. */
B200AMP_API int b200amp_pass1_partition(long long n, int *vblocks, long long *elements_per_vblock);

/* Pass 2 + all-gather. As b200amp_pass2_f16 on the rank's slice, with the fp16 weights stored
 * to weights16_by_rank[r] for every r (HOST array of nranks device pointers: the start of this
 * rank's slice in rank r's weight arena, the rank's own arena included). */
B200AMP_API int b200amp_pass2_ag_f16(float *master, float *m, float *v, const void *reduced16,
                                     void *const *weights16_by_rank, int nranks, long long n, long long arena_offset,
                                     const b200amp_tensor_info *tensors, int ntensors, const b200amp_step_state *st,
                                     float beta1, float beta2, float eps, b200amp_stream s);

/* ---- ordering between one-process-per-GPU ranks, owned by the library
 * Each rank owns one block of B200AMP_ZERO1_SYNC_BYTES bytes of device memory that every rank
 * has mapped, zeroed with b200amp_zero1_sync_init before any rank's first step (the ranks agree
 * on that on the host, once). A rank announces a phase of the step in flight by storing the
 * step's number into its word of every rank's block; a rank waits by polling its own block. The
 * step's number lives in the block and is advanced on the device, so a step is the same
 * sequence of launches every time. Waits compare for equality and a step number is never 0, so
 * words still zero from the set-up never match and the 32-bit counter may wrap. Phases: 0 gradients ready, 1 pairs written, 2 weights
 * written.
 * Every wait is bounded (wait_limit polls; 0 = the default, several seconds). A wait that runs
 * out records (phase + 1) | missing_rank << 8 in the block's error word, sets bit 1 of
 * b200amp_device_error, and the kernel returns without doing its work; kernels launched after
 * it see the error word and return at once, the finalize sets found_inf = 1 so that pass 2
 * changes nothing, and the step counter is not advanced. Nothing traps or spins for ever. After
 * a reported give-up the optimizer's state is not to be trusted: restore a checkpoint, zero
 * every rank's block and workspace again, and go on. */
#define B200AMP_ZERO1_SYNC_BYTES 1024
typedef struct b200amp_zero1_sync
{
    void *block_by_rank[8];     /* block_by_rank[r]: rank r's block, a device pointer of the calling process */
    unsigned int wait_limit;    /* polls before a wait gives up; 0 = default */
} b200amp_zero1_sync;
enum
{
    B200AMP_SYNC_SIGNAL = 1,    /* announce the phase to every rank */
    B200AMP_SYNC_WAIT = 2,      /* wait for every rank's announcement of the phase */
    B200AMP_SYNC_ADVANCE = 4,   /* the step is over on this rank: advance its step counter */
    B200AMP_SYNC_STAMP = 8      /* record the step in flight where the copy engines read it (b200amp_rs_push_f16_ce) */
};
B200AMP_API int b200amp_zero1_sync_init(void *block, b200amp_stream s);
/* Synchronous read of a rank's own block: the number of the last step it completed (counts up from 0 and
 * wraps from 2^32 - 1 to 1), and the error word (0 = none). */
B200AMP_API int b200amp_zero1_sync_read(const void *block, unsigned int *steps_done, unsigned int *error);
/* One small kernel: `what` is a combination of the three flags above, applied to `phase` of the
 * step in flight. The step's last launch is (phase 2, SIGNAL | WAIT | ADVANCE): enqueued after
 * pass2_ag, it tells every rank that this rank's weights have landed and returns when every
 * rank's have landed here. */
B200AMP_API int b200amp_zero1_barrier(const b200amp_zero1_sync *sync, int nranks, int my_rank, int phase, int what,
                                      b200amp_stream s);
/* b200amp_rs_pass1_f16 that orders itself: every CTA announces this rank's gradients (phase 0)
 * and waits for every rank's before it loads anything; the last CTA announces the pairs it has
 * written (phase 1). */
B200AMP_API int b200amp_rs_pass1_f16_sync(const void *const *grads16_by_rank, int nranks, int my_rank,
                                          void *reduced16, long long n, const b200amp_step_state *st,
                                          void *workspace, double *const *pair_table_by_rank,
                                          const b200amp_zero1_sync *sync, b200amp_stream s);
/* b200amp_finalize_sums that first waits (phase 1) for every rank's pair; sums is this rank's
 * pair table. */
B200AMP_API int b200amp_finalize_sums_sync(b200amp_step_state *st, const double *sums, int nranks, int my_rank,
                                           const b200amp_schedule *cfg, b200amp_step_state *history,
                                           int history_len, const b200amp_zero1_sync *sync, b200amp_stream s);

/* ---- copy-engine forms: same results bit for bit, but the bytes that cross NVLink are moved by
 * cudaMemcpyAsync on copy streams of the library instead of by loads and stores of the kernels,
 * piece by piece, overlapped with the kernels (which then touch local memory only). With both
 * directions of the links busy the copy engines move 771-776 GB/s per direction between two
 * B200s where SM-issued loads reach 664 and stores 704.
 * rs: staging16 is a local buffer of (nranks - 1) * n fp16 values; the peers' slices are pulled
 * into it while earlier pieces are reduced. With sync != null the call starts with the phase-0
 * exchange and its last piece announces phase 1 (as b200amp_rs_pass1_f16_sync); with sync == null
 * the caller has ordered the ranks. ag: every piece of fp16 weights is pushed into the peers'
 * arenas while pass 2 runs on the next piece; the call returns with s waiting for the last push.
 * pieces: 1..64. Work enqueued on s before the call is complete before the first copy starts.
 * The streams and events are created on the first call on a device and kept (these two calls
 * allocate); one host thread per device may use them. */
B200AMP_API int b200amp_rs_pass1_f16_ce(const void *const *grads16_by_rank, int nranks, int my_rank, void *staging16,
                                        void *reduced16, long long n, int pieces, const b200amp_step_state *st,
                                        void *workspace, double *const *pair_table_by_rank,
                                        const b200amp_zero1_sync *sync, b200amp_stream s);
B200AMP_API int b200amp_pass2_ag_f16_ce(float *master, float *m, float *v, const void *reduced16,
                                        void *const *weights16_by_rank, int nranks, int my_rank, long long n,
                                        long long arena_offset, const b200amp_tensor_info *tensors, int ntensors,
                                        const b200amp_step_state *st, float beta1, float beta2, float eps, int pieces,
                                        b200amp_stream s);
/* Reduce-scatter by push, in two calls per rank. Writes use a link that is busy in both directions
 * better than reads do, so here every rank WRITES: b200amp_rs_push_f16_ce copies slice q of this
 * rank's gradient arena (grads16: the start of the arena; slices of n elements) into row my_rank of
 * rank q's staging buffer (staging_by_rank[q]: nranks rows of n fp16 values, mapped in this
 * process), in `pieces` pieces (at most 16), each followed on the same copy stream by a 4-byte
 * copy of the step number into rank q's flag block. b200amp_rs_pass1_f16_pushed then reduces the
 * owner's rows piece by piece (own_slice16: this rank's slice in its own arena; staging16: its own
 * staging buffer), each launch waiting, bounded, for its piece of every peer; the last piece
 * writes the pairs and announces phase 1. No phase-0 exchange is needed. Same bits as
 * b200amp_rs_pass1_f16. The gradient arena may be overwritten once the step's finalize has run. */
B200AMP_API int b200amp_rs_push_f16_ce(const void *grads16, void *const *staging_by_rank, int nranks, int my_rank,
                                       long long n, int pieces, const b200amp_zero1_sync *sync, b200amp_stream s);
B200AMP_API int b200amp_rs_pass1_f16_pushed(const void *own_slice16, const void *staging16, int nranks, int my_rank,
                                            void *reduced16, long long n, int pieces, const b200amp_step_state *st,
                                            void *workspace, double *const *pair_table_by_rank,
                                            const b200amp_zero1_sync *sync, b200amp_stream s);
/* cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, s): a copy-engine transfer between any two
 * device pointers of the calling process, a peer's mapped memory included. */
B200AMP_API int b200amp_copy_async(void *dst, const void *src, long long bytes, b200amp_stream s);

/* The whole step for an arena held by one GPU: b200amp_pass1_finalize_f16 then
 * b200amp_pass2_f16 (two launches). */
B200AMP_API int b200amp_step_f16(float *master, float *m, float *v, const void *grads16, void *weights16, long long n,
                     const b200amp_tensor_info *tensors, int ntensors, b200amp_step_state *st, void *workspace,
                     const b200amp_schedule *cfg, b200amp_step_state *history, int history_len,
                     float beta1, float beta2, float eps, b200amp_stream s);

/* ---------------------------------------------------------------- CUDA-graph helpers
 * Replace CudaGraph::{capture,launch} and its destructor (cuda/graph.h:14-30,
 * cuda/graph.cu:17-41): begin puts s in thread-local capture mode, the caller
 * enqueues the step, end instantiates. */
typedef struct b200amp_graph b200amp_graph;
B200AMP_API int b200amp_graph_begin_capture(b200amp_stream s);
B200AMP_API int b200amp_graph_end_capture(b200amp_stream s, b200amp_graph **out);
B200AMP_API int b200amp_graph_launch(b200amp_graph *g, b200amp_stream s);
B200AMP_API int b200amp_graph_destroy(b200amp_graph *g);

/* ---------------------------------------------------------------- tuning hooks
 * Launch-shape knobs for measurement (blocks per SM, variant); not part of the
 * reference's surface. Unknown keys return B200AMP_ERR_ARG. Results never depend on them.
 * Process-wide and unsynchronised: set them before other threads launch work. */
B200AMP_API int b200amp_tune_set(const char *key, int value);
B200AMP_API int b200amp_tune_get(const char *key, int *value);
/* *out = what gave up a bounded wait on the current device since the last call, as a bit mask:
 * 1 a shared-memory staged pass 2 waiting for a bulk copy that never completed, 2 a ZeRO-1
 * kernel waiting for another rank; 0 = nothing. Reading clears it. Synchronises the device.
 * After a nonzero answer the optimizer state of the step that gave up is not to be trusted. */
B200AMP_API int b200amp_device_error(int *out);
/* Kernel launches enqueued by this library on the calling process so far. */
B200AMP_API long long b200amp_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* B200AMP_H */
