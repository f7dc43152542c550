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
