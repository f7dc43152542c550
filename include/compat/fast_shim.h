// fast_shim.h: the reference's C++ operator surface for the optimizer step, over the C ABI.
//
// A translation unit of cuda-transformer that includes this header instead of the
// optimizer part of cuda/kernels/fast.h (lines 101-166) and cuda/graph.h, and links
// libb200amp.so instead of scaler.o / adamw_multi.o / graph.o, keeps compiling:
// same type names, same free functions, same argument order and meaning. Errors keep
// the reference's behaviour too: print file:line and the text, then exit(1)
// (cuda/common.h:10-20) -- the C ABI itself only returns a status.
//
// floatX is __half here (the reference's -DFP16 build, cuda/precision.h:14-17).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <functional>

#include "b200amp.h"

using floatX = __half;
using StepState = b200amp_step_state;          // cuda/kernels/fast.h:104-121
using ScheduleConfig = b200amp_schedule;       // cuda/kernels/fast.h:123-133
using TensorInfo = b200amp_tensor_info;        // cuda/kernels/fast.h:153-158
constexpr int NORM_BLOCKS = B200AMP_NORM_BLOCKS;
constexpr int MAX_TENSORS = B200AMP_MAX_TENSORS;

#define B200AMP_SHIM_CHECK(call)                                                              \
    do                                                                                        \
    {                                                                                         \
        int status_ = (call);                                                                 \
        if (status_ != B200AMP_OK)                                                            \
        {                                                                                     \
            fprintf(stderr, "b200amp error at %s:%d: %s\n    %s\n", __FILE__, __LINE__,       \
                    b200amp_last_error(), #call);                                             \
            exit(1);                                                                          \
        }                                                                                     \
    } while (0)

inline StepState initial_state(float scale)                                     // scaler.cu:21-29
{
    StepState st;
    B200AMP_SHIM_CHECK(b200amp_initial_state(scale, &st));
    return st;
}

inline void begin_step(StepState *st, cudaStream_t s)                           // scaler.cu:173-177
{
    B200AMP_SHIM_CHECK(b200amp_begin_step(st, s));
}

inline void unscale_and_norm(float *grads, long long n, StepState *st, float *partial, cudaStream_t s)
{
    B200AMP_SHIM_CHECK(b200amp_unscale_and_norm_f32(grads, n, st, partial, s));  // scaler.cu:179-184
}

inline void finalize_step(StepState *st, const float *partial, ScheduleConfig cfg, StepState *history,
                          int history_len, cudaStream_t s)                      // scaler.cu:186-192
{
    B200AMP_SHIM_CHECK(b200amp_finalize_step(st, partial, &cfg, history, history_len, s));
}

inline void adamw_multi(float *params, floatX *params_x, const float *grads, float *m, float *v, long long n,
                        const TensorInfo *tensors, int ntensors, const StepState *st, float beta1, float beta2,
                        float eps, cudaStream_t s)                              // adamw_multi.cu:93-108
{
    B200AMP_SHIM_CHECK(b200amp_adamw_multi_f32(params, params_x, grads, m, v, n, tensors, ntensors, st, beta1, beta2,
                                               eps, s));
}

inline double lr_on_gpu(int step, ScheduleConfig cfg)                           // scaler.cu:100-110
{
    double lr = 0.0;
    B200AMP_SHIM_CHECK(b200amp_lr_on_gpu(step, &cfg, &lr));
    return lr;
}

inline void cast_to_x(floatX *out, const float *in, long long n, cudaStream_t s)    // fused.cu:319-323
{
    B200AMP_SHIM_CHECK(b200amp_cast_to_x(out, in, n, s));
}

// cuda/graph.h:14-30
struct CudaGraph
{
    b200amp_graph *graph = nullptr;

    CudaGraph() = default;
    ~CudaGraph()
    {
        b200amp_graph_destroy(graph);           // never exit from a destructor
    }
    CudaGraph(const CudaGraph &) = delete;
    CudaGraph &operator=(const CudaGraph &) = delete;

    // runs body with s in capture mode (nothing executes), then instantiates
    void capture(cudaStream_t s, const std::function<void()> &body)
    {
        if (graph != nullptr)
        {
            B200AMP_SHIM_CHECK(b200amp_graph_destroy(graph));
            graph = nullptr;
        }
        B200AMP_SHIM_CHECK(b200amp_graph_begin_capture(s));
        body();
        B200AMP_SHIM_CHECK(b200amp_graph_end_capture(s, &graph));
    }
    void launch(cudaStream_t s)
    {
        B200AMP_SHIM_CHECK(b200amp_graph_launch(graph, s));
    }
    bool ready() const
    {
        return graph != nullptr;
    }
};
