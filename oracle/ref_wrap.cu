// ref_wrap.cu: extern "C" doors into the REFERENCE's own optimizer kernels, so the
// tests and the benchmark can run them on the same arenas as the library.
//
// TEST INFRASTRUCTURE ONLY. This file holds no arithmetic: it includes the reference's
// header from the reference checkout (-I paths given by oracle/build_ref.py) and
// forwards to its launchers (cuda/kernels/fast.h:136-166), which are compiled from
// cuda/kernels/scaler.cu and cuda/kernels/adamw_multi.cu where they lie. The reference
// launchers call exit(1) on a CUDA error (cuda/common.h:10-20); nothing here changes that.
#include <cuda_runtime.h>

#include "fast.h"

extern "C" __attribute__((visibility("default"))) int refamp_sizeof_state(void)
{
    return static_cast<int>(sizeof(StepState));
}

extern "C" __attribute__((visibility("default"))) void refamp_initial_state(float scale, StepState *out)
{
    *out = initial_state(scale);
}

extern "C" __attribute__((visibility("default"))) void refamp_begin_step(StepState *st, void *stream)
{
    begin_step(st, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) void refamp_unscale_and_norm(float *grads, long long n,
                                                                                StepState *st, float *partial,
                                                                                void *stream)
{
    unscale_and_norm(grads, n, st, partial, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) void refamp_finalize_step(StepState *st, const float *partial,
                                                                             const ScheduleConfig *cfg,
                                                                             StepState *history, int history_len,
                                                                             void *stream)
{
    finalize_step(st, partial, *cfg, history, history_len, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) void refamp_adamw_multi(float *params, void *params_x,
                                                                           const float *grads, float *m, float *v,
                                                                           long long n, const TensorInfo *tensors,
                                                                           int ntensors, const StepState *st,
                                                                           float beta1, float beta2, float eps,
                                                                           void *stream)
{
    adamw_multi(params, static_cast<floatX *>(params_x), grads, m, v, n, tensors, ntensors, st, beta1, beta2, eps,
                static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) double refamp_lr_on_gpu(int step, const ScheduleConfig *cfg)
{
    return lr_on_gpu(step, *cfg);
}
