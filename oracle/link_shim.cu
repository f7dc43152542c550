// link_shim.cu: lets the REFERENCE's own programs (test_fast, test_checkpoint, train_fast)
// link against libb200amp.so without a single change to their sources.
//
// TEST INFRASTRUCTURE (built by oracle/build_ref_tests.py into oracle/_ref/, never part of
// the library). The reference declares its optimizer launchers and CudaGraph in
// cuda/kernels/fast.h:136-166 and cuda/graph.h:14-30 and defines them in
// cuda/kernels/scaler.cu, cuda/kernels/adamw_multi.cu and cuda/graph.cu. This file includes
// the reference's headers (from the reference checkout, by -I) and defines those same C++
// symbols by forwarding to the C ABI, so a link line that drops the three reference objects
// and adds this one plus -lb200amp resolves every call site in cuda/gpt_fast.cu,
// cuda/checkpoint.cu and the tests. The structs are the reference's own; their layouts equal
// the C ABI's (checked below), so pointers pass straight through.
#include <cstdio>
#include <cstdlib>

#include "common.h"         // reference: CUDA_CHECK, g_capturing
#include "graph.h"          // reference: struct CudaGraph
#include "kernels/fast.h"   // reference: StepState, ScheduleConfig, TensorInfo, launcher declarations

#include "b200amp.h"

static_assert(sizeof(StepState) == sizeof(b200amp_step_state), "StepState layout");
static_assert(sizeof(ScheduleConfig) == sizeof(b200amp_schedule), "ScheduleConfig layout");
static_assert(sizeof(TensorInfo) == sizeof(b200amp_tensor_info), "TensorInfo layout");
static_assert(NORM_BLOCKS == B200AMP_NORM_BLOCKS && MAX_TENSORS == B200AMP_MAX_TENSORS, "constants");

#define SHIM_CHECK(call)                                                                          \
    do                                                                                            \
    {                                                                                             \
        if ((call) != B200AMP_OK)                                                                 \
        {                                                                                         \
            fprintf(stderr, "b200amp error at %s:%d: %s\n", __FILE__, __LINE__, b200amp_last_error()); \
            exit(1);                                                                              \
        }                                                                                         \
    } while (0)

static b200amp_step_state *abi(StepState *st)
{
    return reinterpret_cast<b200amp_step_state *>(st);
}

StepState initial_state(float scale)
{
    StepState st;
    SHIM_CHECK(b200amp_initial_state(scale, abi(&st)));
    return st;
}

void begin_step(StepState *st, cudaStream_t s)
{
    SHIM_CHECK(b200amp_begin_step(abi(st), s));
}

#ifndef B200AMP_SHIM_NATIVE

// ---- compat: the reference's arguments and results, bit for bit

void unscale_and_norm(float *grads, long long n, StepState *st, float *partial, cudaStream_t s)
{
    SHIM_CHECK(b200amp_unscale_and_norm_f32(grads, n, abi(st), partial, s));
}

void finalize_step(StepState *st, const float *partial, ScheduleConfig cfg, StepState *history, int history_len,
                   cudaStream_t s)
{
    SHIM_CHECK(b200amp_finalize_step(abi(st), partial, reinterpret_cast<const b200amp_schedule *>(&cfg), abi(history),
                                     history_len, s));
}

void adamw_multi(float *params, floatX *params_x, const float *grads, float *m, float *v, long long n,
                 const TensorInfo *tensors, int ntensors, const StepState *st, float beta1, float beta2, float eps,
                 cudaStream_t s)
{
    SHIM_CHECK(b200amp_adamw_multi_f32(params, params_x, grads, m, v, n,
                                       reinterpret_cast<const b200amp_tensor_info *>(tensors), ntensors,
                                       reinterpret_cast<const b200amp_step_state *>(st), beta1, beta2, eps, s));
}

#else

// ---- native (-DB200AMP_SHIM_NATIVE): the same three calls routed onto the fp16-arena step.
// The reference's backward pass leaves loss-scaled fp32 gradients in its arena; unscale_and_norm
// becomes the bridge (round to fp16 into an arena this shim keeps, pass 1 on the rounded values),
// finalize_step the finalize on the bridge's sums, adamw_multi the native pass 2 on the fp16
// arena. The fp32 arena is left for the reference's own grads.zero (cuda/gpt_fast.cu:455), which an
// unmodified trainer still runs every step, so the bridge does not clear it a second time:
// 6 + 28 B/param + the reference's 4 B/param memset, instead of 8 + 30 + 4. The
// gradients the optimizer sees are rounded to fp16 first, so a run agrees with the stock
// program to fp16 rounding of the gradients, not bit for bit; the fp32 arena is NOT unscaled in
// place (test_fast reads it back, so the test programs use the compat shim). For train_fast.

struct NativeArena
{
    const float *grads32 = nullptr;         // which fp32 arena this belongs to
    long long n = 0;
    void *grads16 = nullptr;
    void *workspace = nullptr;
};

static NativeArena g_arena;                 // the reference's programs hold one model

// Called inside train_fast's graph capture the first time (its first step IS the captured one), so
// the allocation asks for relaxed capture rules on this thread for its duration; the clearing of
// the workspace is stream-ordered and simply becomes part of the graph.
static NativeArena &arena_for(const float *grads32, long long n, cudaStream_t s)
{
    if (g_arena.grads32 == grads32 && g_arena.n == n)
    {
        return g_arena;
    }
    if (g_arena.grads32 != nullptr)
    {
        fprintf(stderr, "link shim (native): a second gradient arena appeared; this shim serves one model\n");
        exit(1);
    }
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    CUDA_CHECK(cudaThreadExchangeStreamCaptureMode(&mode));
    CUDA_CHECK(cudaMalloc(&g_arena.grads16, static_cast<size_t>(n) * 2));
    CUDA_CHECK(cudaMalloc(&g_arena.workspace, b200amp_workspace_bytes()));
    CUDA_CHECK(cudaThreadExchangeStreamCaptureMode(&mode));
    SHIM_CHECK(b200amp_workspace_init(g_arena.workspace, s));
    g_arena.grads32 = grads32;
    g_arena.n = n;
    return g_arena;
}

void unscale_and_norm(float *grads, long long n, StepState *st, float *, cudaStream_t s)
{
    NativeArena &a = arena_for(grads, n, s);
    SHIM_CHECK(b200amp_cast_pass1_f32(grads, a.grads16, n, /*clear_source=*/0, abi(st), a.workspace, nullptr, nullptr,
                                      0, s));
}

void finalize_step(StepState *st, const float *, ScheduleConfig cfg, StepState *history, int history_len,
                   cudaStream_t s)
{
    if (g_arena.workspace == nullptr)
    {
        fprintf(stderr, "link shim (native): finalize_step before unscale_and_norm\n");
        exit(1);
    }
    // the first 16 bytes of the workspace are {sum of squares, flag}: one "rank"
    SHIM_CHECK(b200amp_finalize_sums(abi(st), static_cast<const double *>(g_arena.workspace), 1,
                                     reinterpret_cast<const b200amp_schedule *>(&cfg), abi(history), history_len, s));
}

void adamw_multi(float *params, floatX *params_x, const float *grads, float *m, float *v, long long n,
                 const TensorInfo *tensors, int ntensors, const StepState *st, float beta1, float beta2, float eps,
                 cudaStream_t s)
{
    NativeArena &a = arena_for(grads, n, s);
    SHIM_CHECK(b200amp_pass2_f16(params, m, v, a.grads16, params_x, n, 0,
                                 reinterpret_cast<const b200amp_tensor_info *>(tensors), ntensors,
                                 reinterpret_cast<const b200amp_step_state *>(st), beta1, beta2, eps, s));
}

#endif

double lr_on_gpu(int step, ScheduleConfig cfg)
{
    double lr = 0.0;
    SHIM_CHECK(b200amp_lr_on_gpu(step, reinterpret_cast<const b200amp_schedule *>(&cfg), &lr));
    return lr;
}

// CudaGraph keeps a cudaGraphExec_t member; the shim parks the library's graph handle in it
// (ready() only compares it with nullptr).
static b200amp_graph *handle_of(cudaGraphExec_t exec)
{
    return reinterpret_cast<b200amp_graph *>(exec);
}

CudaGraph::~CudaGraph()
{
    if (exec != nullptr)
    {
        b200amp_graph_destroy(handle_of(exec));
    }
}

void CudaGraph::capture(cudaStream_t s, const std::function<void()> &body)
{
    if (exec != nullptr)
    {
        SHIM_CHECK(b200amp_graph_destroy(handle_of(exec)));
        exec = nullptr;
    }
    SHIM_CHECK(b200amp_graph_begin_capture(s));
    g_capturing = true;                     // debug builds of the reference: no device syncs while capturing
    body();
    g_capturing = false;
    b200amp_graph *graph = nullptr;
    SHIM_CHECK(b200amp_graph_end_capture(s, &graph));
    exec = reinterpret_cast<cudaGraphExec_t>(graph);
}

void CudaGraph::launch(cudaStream_t s)
{
    SHIM_CHECK(b200amp_graph_launch(handle_of(exec), s));
}
