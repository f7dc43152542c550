// b200amp_host.hpp: C++ owner of the optimizer state of one GPU, over the C ABI.
//
// The optimizer part of the reference's FastGPT (cuda/gpt_fast.h:63-114,
// cuda/gpt_fast.cu:96-149,245-253,438-467): the flat arenas, the tensor table, the
// device-resident step state + history ring, reset / set_params / optimizer_step /
// read_state. The gradient arena is fp16 (loss-scaled, written by the caller); the step
// is the library's two native launches. Errors print and exit(1) like the reference's
// CUDA_CHECK (cuda/common.h:10-20).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "b200amp.h"

namespace b200amp_host
{

#define B200AMP_HOST_CUDA(call)                                                               \
    do                                                                                        \
    {                                                                                         \
        cudaError_t err_ = (call);                                                            \
        if (err_ != cudaSuccess)                                                              \
        {                                                                                     \
            fprintf(stderr, "CUDA error at %s:%d: %s\n    %s\n", __FILE__, __LINE__,          \
                    cudaGetErrorString(err_), #call);                                         \
            exit(1);                                                                          \
        }                                                                                     \
    } while (0)

#define B200AMP_HOST_CHECK(call)                                                              \
    do                                                                                        \
    {                                                                                         \
        if ((call) != B200AMP_OK)                                                             \
        {                                                                                     \
            fprintf(stderr, "b200amp error at %s:%d: %s\n", __FILE__, __LINE__, b200amp_last_error()); \
            exit(1);                                                                          \
        }                                                                                     \
    } while (0)

template <typename T>
struct DeviceArray                      // one cudaMalloc, freed in the destructor, move only
{
    T *ptr = nullptr;
    size_t count = 0;

    DeviceArray() = default;
    explicit DeviceArray(size_t n) : count(n)
    {
        if (n > 0)
        {
            B200AMP_HOST_CUDA(cudaMalloc(&ptr, n * sizeof(T)));
        }
    }
    ~DeviceArray()
    {
        cudaFree(ptr);
    }
    DeviceArray(DeviceArray &&o) noexcept : ptr(o.ptr), count(o.count)
    {
        o.ptr = nullptr;
        o.count = 0;
    }
    DeviceArray &operator=(DeviceArray &&o) noexcept
    {
        if (this != &o)
        {
            cudaFree(ptr);
            ptr = o.ptr;
            count = o.count;
            o.ptr = nullptr;
            o.count = 0;
        }
        return *this;
    }
    DeviceArray(const DeviceArray &) = delete;
    DeviceArray &operator=(const DeviceArray &) = delete;

    void zero(cudaStream_t s)
    {
        if (count > 0)
        {
            B200AMP_HOST_CUDA(cudaMemsetAsync(ptr, 0, count * sizeof(T), s));
        }
    }
    std::vector<T> download() const
    {
        std::vector<T> host(count);
        if (count > 0)
        {
            B200AMP_HOST_CUDA(cudaMemcpy(host.data(), ptr, count * sizeof(T), cudaMemcpyDeviceToHost));
        }
        return host;
    }
};

struct AmpOptimizer
{
    long long n = 0;                    // elements in the arena, a multiple of 8
    int device = 0;                     // the device that was current at construction; methods switch to it
    cudaStream_t stream = nullptr;
    DeviceArray<float> master, m, v;
    DeviceArray<__half> weights16, grads16;
    DeviceArray<b200amp_tensor_info> tensors;
    DeviceArray<b200amp_step_state> state, history;
    DeviceArray<unsigned char> workspace;
    int history_len;
    b200amp_schedule sched;
    float beta1, beta2, eps;

    AmpOptimizer(long long n_, const std::vector<b200amp_tensor_info> &table, b200amp_schedule cfg, float eps_,
                 float loss_scale, int history_len_ = 256)
        : n(n_), master(n_), m(n_), v(n_), weights16(n_), grads16(n_), tensors(table.size()), state(1),
          history(history_len_), workspace(b200amp_workspace_bytes()), history_len(history_len_), sched(cfg),
          beta1(cfg.beta1), beta2(cfg.beta2), eps(eps_)
    {
        B200AMP_HOST_CUDA(cudaGetDevice(&device));
        B200AMP_HOST_CHECK(b200amp_device_check());
        B200AMP_HOST_CHECK(b200amp_check_tensor_table(table.data(), static_cast<int>(table.size()), n));
        B200AMP_HOST_CUDA(cudaStreamCreate(&stream));       // blocking, as cuda/gpt_fast.cu:94
        B200AMP_HOST_CUDA(cudaMemcpy(tensors.ptr, table.data(), table.size() * sizeof(b200amp_tensor_info),
                                     cudaMemcpyHostToDevice));
        master.zero(stream);
        weights16.zero(stream);
        reset(loss_scale);
    }
    ~AmpOptimizer()
    {
        if (stream != nullptr)
        {
            cudaStreamDestroy(stream);
        }
    }
    AmpOptimizer(const AmpOptimizer &) = delete;
    AmpOptimizer &operator=(const AmpOptimizer &) = delete;

    void reset(float loss_scale)                            // cuda/gpt_fast.cu:245-253
    {
        B200AMP_HOST_CUDA(cudaSetDevice(device));
        m.zero(stream);
        v.zero(stream);
        grads16.zero(stream);
        history.zero(stream);
        B200AMP_HOST_CHECK(b200amp_workspace_init(workspace.ptr, stream));
        b200amp_step_state st;
        B200AMP_HOST_CHECK(b200amp_initial_state(loss_scale, &st));
        B200AMP_HOST_CUDA(cudaMemcpyAsync(state.ptr, &st, sizeof(st), cudaMemcpyHostToDevice, stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));   // st lives on this stack frame
    }
    void set_params(const std::vector<float> &host)         // cuda/gpt_fast.cu:274-286
    {
        if (static_cast<long long>(host.size()) != n)
        {
            fprintf(stderr, "error: %zu parameters given, the arena has %lld\n", host.size(), n);
            exit(1);
        }
        B200AMP_HOST_CUDA(cudaSetDevice(device));
        B200AMP_HOST_CUDA(cudaMemcpy(master.ptr, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
        B200AMP_HOST_CHECK(b200amp_cast_to_x(weights16.ptr, master.ptr, n, stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));
    }
    void set_grads(const std::vector<__half> &host)         // what the backward pass would leave
    {
        B200AMP_HOST_CUDA(cudaSetDevice(device));
        B200AMP_HOST_CUDA(cudaMemcpyAsync(grads16.ptr, host.data(), host.size() * sizeof(__half),
                                          cudaMemcpyHostToDevice, stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));
    }
    void optimizer_step()                                   // the place of cuda/gpt_fast.cu:438-450
    {
        B200AMP_HOST_CUDA(cudaSetDevice(device));
        B200AMP_HOST_CHECK(b200amp_step_f16(master.ptr, m.ptr, v.ptr, grads16.ptr, weights16.ptr, n, tensors.ptr,
                                            static_cast<int>(tensors.count), state.ptr, workspace.ptr, &sched,
                                            history.ptr, history_len, beta1, beta2, eps, stream));
    }
    b200amp_step_state read_state()                         // cuda/gpt_fast.cu:461-467
    {
        b200amp_step_state st;
        B200AMP_HOST_CUDA(cudaSetDevice(device));
        B200AMP_HOST_CUDA(cudaMemcpyAsync(&st, state.ptr, sizeof(st), cudaMemcpyDeviceToHost, stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));
        return st;
    }
};

// Steps fed from pinned host memory, for a host whose loss-scaled fp16 gradients arrive there (an
// offloaded backward pass, a parameter server). Two device gradient arenas take turns: while pass 2
// of step k reads one, a copy engine fills the other with step k + 1's gradients on its own stream,
// so a step costs the longer of its host-to-device copy and its kernels instead of their sum. Each
// step's 60-byte state is copied into pinned memory behind its pass 2. At most two steps are in
// flight: submitting a third waits for the first. The reference keeps its gradients on the device
// (cuda/gpt_fast.cu:452-459) and has no counterpart.
struct HostGradientFeed
{
    AmpOptimizer &opt;
    DeviceArray<__half> second;                 // the arena that alternates with opt.grads16
    cudaStream_t copy = nullptr;
    cudaEvent_t copied[2] = {nullptr, nullptr}, done[2] = {nullptr, nullptr};
    b200amp_step_state *pinned_state = nullptr; // two of them
    long long next = 0;

    explicit HostGradientFeed(AmpOptimizer &o) : opt(o), second(static_cast<size_t>(o.n))
    {
        B200AMP_HOST_CUDA(cudaSetDevice(opt.device));
        B200AMP_HOST_CUDA(cudaStreamCreateWithFlags(&copy, cudaStreamNonBlocking));
        for (int k = 0; k < 2; k++)
        {
            B200AMP_HOST_CUDA(cudaEventCreateWithFlags(&copied[k], cudaEventDisableTiming));
            B200AMP_HOST_CUDA(cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming));
        }
        B200AMP_HOST_CUDA(cudaMallocHost(&pinned_state, 2 * sizeof(b200amp_step_state)));
    }
    ~HostGradientFeed()
    {
        cudaSetDevice(opt.device);
        cudaStreamSynchronize(opt.stream);
        cudaStreamSynchronize(copy);
        cudaFreeHost(pinned_state);
        for (int k = 0; k < 2; k++)
        {
            cudaEventDestroy(copied[k]);
            cudaEventDestroy(done[k]);
        }
        cudaStreamDestroy(copy);
    }
    HostGradientFeed(const HostGradientFeed &) = delete;
    HostGradientFeed &operator=(const HostGradientFeed &) = delete;

    // pinned: opt.n loss-scaled fp16 gradients in page-locked host memory. Returns the step's ticket.
    long long submit(const __half *pinned)
    {
        const long long ticket = next++;
        const int slot = static_cast<int>(ticket % 2);
        __half *arena = slot == 0 ? opt.grads16.ptr : second.ptr;
        B200AMP_HOST_CUDA(cudaSetDevice(opt.device));
        if (ticket >= 2)
        {
            // the step that last read this arena, and the read-back that used this pinned slot, are done
            B200AMP_HOST_CUDA(cudaEventSynchronize(done[slot]));
        }
        B200AMP_HOST_CUDA(cudaMemcpyAsync(arena, pinned, static_cast<size_t>(opt.n) * sizeof(__half),
                                          cudaMemcpyHostToDevice, copy));
        B200AMP_HOST_CUDA(cudaEventRecord(copied[slot], copy));
        B200AMP_HOST_CUDA(cudaStreamWaitEvent(opt.stream, copied[slot], 0));
        B200AMP_HOST_CHECK(b200amp_step_f16(opt.master.ptr, opt.m.ptr, opt.v.ptr, arena, opt.weights16.ptr, opt.n,
                                            opt.tensors.ptr, static_cast<int>(opt.tensors.count), opt.state.ptr,
                                            opt.workspace.ptr, &opt.sched, opt.history.ptr, opt.history_len,
                                            opt.beta1, opt.beta2, opt.eps, opt.stream));
        B200AMP_HOST_CUDA(cudaMemcpyAsync(&pinned_state[slot], opt.state.ptr, sizeof(b200amp_step_state),
                                          cudaMemcpyDeviceToHost, opt.stream));
        B200AMP_HOST_CUDA(cudaEventRecord(done[slot], opt.stream));
        return ticket;
    }
    // The state after the step of `ticket`; valid for the last two tickets submitted. Blocks until it is there.
    b200amp_step_state collect(long long ticket)
    {
        if (ticket < 0 || ticket >= next || ticket < next - 2)
        {
            fprintf(stderr, "error: ticket %lld is not one of the last two of %lld submitted\n", ticket, next);
            exit(1);
        }
        const int slot = static_cast<int>(ticket % 2);
        B200AMP_HOST_CUDA(cudaSetDevice(opt.device));
        B200AMP_HOST_CUDA(cudaEventSynchronize(done[slot]));
        return pinned_state[slot];
    }
};

} // namespace b200amp_host
