// b200amp_zero1_host.hpp: one host process driving the ZeRO-1 form of the step on R GPUs of an
// NVLink box, in C++ over the C ABI, with no other library: no NCCL, no MPI, no Python.
//
// The reference has no multi-GPU code; this is the host side of b200amp_rs_pass1_f16 /
// b200amp_pass2_ag_f16 for a trainer built like the reference's (one process, one host thread,
// everything enqueued on streams, cuda/gpt_fast.cu:94). Inside one process every device pointer
// is valid on every device once peer access is on, so the kernels of rank r read rank q's
// gradient arena and write rank q's weight arena directly, and the ordering between ranks that
// the kernels leave to the caller is done with events: each rank's stream records an event at
// the end of a phase and waits for the events of all the others before the next one. Nothing
// spins on the device and the host never blocks inside a step.
//
//     phase            on every rank's stream                              then
//     gradients ready  (the caller's backward pass has written grads16)    event exchange
//     rs_pass1         pull + average my slice, norm partials, pairs out   event exchange
//     finalize_sums    replicated: identical state bits on every rank
//     pass2_ag         AdamW on my slice, fp16 weights into every arena    event exchange
//
// `devices` may name the same GPU more than once (all ranks on device 0 is how a one-GPU
// machine runs the tests): the ranks' launches then simply serialise.
#pragma once

#include <memory>

#include "b200amp_host.hpp"

namespace b200amp_host
{

struct Zero1Rank
{
    int device;
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;             // end of this rank's part of the current phase
    DeviceArray<float> master, m, v;        // the rank's slice only
    DeviceArray<__half> grads16, weights16; // whole arena: this rank's gradients, everyone's weights
    DeviceArray<__half> reduced16;          // the averaged slice
    DeviceArray<b200amp_tensor_info> tensors;
    DeviceArray<b200amp_step_state> state, history;
    DeviceArray<unsigned char> workspace;
    DeviceArray<double> pairs;              // {sum of squares, flag} of every rank

    // the caller has made `device_` current: every array is allocated there
    Zero1Rank(int device_, long long n, long long per, size_t ntensors, int nranks, int history_len)
        : device(device_), master(per), m(per), v(per), grads16(n), weights16(n), reduced16(per), tensors(ntensors),
          state(1), history(history_len), workspace(b200amp_workspace_bytes()), pairs(2 * nranks)
    {
        B200AMP_HOST_CUDA(cudaStreamCreate(&stream));
        B200AMP_HOST_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    }
    ~Zero1Rank()
    {
        cudaSetDevice(device);
        if (done != nullptr)
        {
            cudaEventDestroy(done);
        }
        if (stream != nullptr)
        {
            cudaStreamDestroy(stream);
        }
    }
    Zero1Rank(const Zero1Rank &) = delete;
    Zero1Rank &operator=(const Zero1Rank &) = delete;
};

struct Zero1Group
{
    int nranks;
    long long n, per;                       // arena elements, elements per rank
    int history_len;
    b200amp_schedule sched;
    float beta1, beta2, eps;
    std::vector<std::unique_ptr<Zero1Rank>> ranks;

    // n must be a multiple of 8 * nranks; nranks 1, 2, 4 or 8; devices.size() == nranks.
    Zero1Group(const std::vector<int> &devices, long long n_, const std::vector<b200amp_tensor_info> &table,
               b200amp_schedule cfg, float eps_, float loss_scale, int history_len_ = 256)
        : nranks(static_cast<int>(devices.size())), n(n_), per(n_ / static_cast<long long>(devices.size())),
          history_len(history_len_), sched(cfg), beta1(cfg.beta1), beta2(cfg.beta2), eps(eps_)
    {
        if (nranks < 1 || n % (8LL * nranks) != 0)
        {
            fprintf(stderr, "error: %lld elements do not split into %d slices of whole 8-element groups\n", n, nranks);
            exit(1);
        }
        B200AMP_HOST_CHECK(b200amp_check_tensor_table(table.data(), static_cast<int>(table.size()), n));
        for (int a : devices)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(a));
            B200AMP_HOST_CHECK(b200amp_device_check());
            for (int b : devices)
            {
                if (a == b)
                {
                    continue;
                }
                int can = 0;
                B200AMP_HOST_CUDA(cudaDeviceCanAccessPeer(&can, a, b));
                if (!can)
                {
                    fprintf(stderr, "error: device %d cannot map the memory of device %d\n", a, b);
                    exit(1);
                }
                cudaError_t err = cudaDeviceEnablePeerAccess(b, 0);
                if (err == cudaErrorPeerAccessAlreadyEnabled)
                {
                    cudaGetLastError();     // clear it: asking twice is fine
                }
                else
                {
                    B200AMP_HOST_CUDA(err);
                }
            }
        }
        for (int r = 0; r < nranks; r++)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(devices[r]));
            ranks.emplace_back(new Zero1Rank(devices[r], n, per, table.size(), nranks, history_len));
            Zero1Rank &k = *ranks.back();
            B200AMP_HOST_CUDA(cudaMemcpy(k.tensors.ptr, table.data(), table.size() * sizeof(b200amp_tensor_info),
                                         cudaMemcpyHostToDevice));
            k.master.zero(k.stream);
            k.weights16.zero(k.stream);
            k.pairs.zero(k.stream);
        }
        reset(loss_scale);
    }

    void reset(float loss_scale)                            // cuda/gpt_fast.cu:245-253, on every rank
    {
        b200amp_step_state st;
        B200AMP_HOST_CHECK(b200amp_initial_state(loss_scale, &st));
        for (auto &k : ranks)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(k->device));
            k->m.zero(k->stream);
            k->v.zero(k->stream);
            k->grads16.zero(k->stream);
            k->history.zero(k->stream);
            B200AMP_HOST_CHECK(b200amp_workspace_init(k->workspace.ptr, k->stream));
            B200AMP_HOST_CUDA(cudaMemcpyAsync(k->state.ptr, &st, sizeof(st), cudaMemcpyHostToDevice, k->stream));
        }
        synchronize();                                      // st lives on this stack frame
    }

    void set_params(const std::vector<float> &host)         // whole arena in, a slice per rank kept
    {
        if (static_cast<long long>(host.size()) != n)
        {
            fprintf(stderr, "error: %zu parameters given, the arena has %lld\n", host.size(), n);
            exit(1);
        }
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            B200AMP_HOST_CUDA(cudaSetDevice(k.device));
            B200AMP_HOST_CUDA(cudaMemcpy(k.master.ptr, host.data() + r * per, per * sizeof(float),
                                         cudaMemcpyHostToDevice));
            // every rank's weight arena gets every slice: rank r casts its own and stores it everywhere
            for (auto &q : ranks)
            {
                B200AMP_HOST_CHECK(b200amp_cast_to_x(q->weights16.ptr + r * per, k.master.ptr, per, k.stream));
            }
        }
        synchronize();
    }

    void set_grads(int rank, const std::vector<__half> &host)   // what rank's backward pass would leave
    {
        Zero1Rank &k = *ranks[rank];
        B200AMP_HOST_CUDA(cudaSetDevice(k.device));
        B200AMP_HOST_CUDA(cudaMemcpyAsync(k.grads16.ptr, host.data(), host.size() * sizeof(__half),
                                          cudaMemcpyHostToDevice, k.stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(k.stream));
    }

    // Every stream waits until every other stream has reached this point.
    void exchange()
    {
        for (auto &k : ranks)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(k->device));
            B200AMP_HOST_CUDA(cudaEventRecord(k->done, k->stream));
        }
        for (auto &k : ranks)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(k->device));
            for (auto &q : ranks)
            {
                if (q.get() != k.get())
                {
                    B200AMP_HOST_CUDA(cudaStreamWaitEvent(k->stream, q->done, 0));
                }
            }
        }
    }

    void optimizer_step()
    {
        std::vector<const void *> grad_slices(nranks);
        std::vector<void *> weight_slices(nranks);
        std::vector<double *> tables(nranks);
        exchange();                                         // every rank's gradients are in its arena
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            for (int q = 0; q < nranks; q++)
            {
                grad_slices[q] = ranks[q]->grads16.ptr + r * per;
                tables[q] = ranks[q]->pairs.ptr;
            }
            B200AMP_HOST_CUDA(cudaSetDevice(k.device));
            B200AMP_HOST_CHECK(b200amp_rs_pass1_f16(grad_slices.data(), nranks, r, k.reduced16.ptr, per, k.state.ptr,
                                                    k.workspace.ptr, tables.data(), k.stream));
        }
        exchange();                                         // every pair has landed in every table
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            for (int q = 0; q < nranks; q++)
            {
                weight_slices[q] = ranks[q]->weights16.ptr + r * per;
            }
            B200AMP_HOST_CUDA(cudaSetDevice(k.device));
            B200AMP_HOST_CHECK(b200amp_finalize_sums(k.state.ptr, k.pairs.ptr, nranks, &sched, k.history.ptr,
                                                     history_len, k.stream));
            B200AMP_HOST_CHECK(b200amp_pass2_ag_f16(k.master.ptr, k.m.ptr, k.v.ptr, k.reduced16.ptr,
                                                    weight_slices.data(), nranks, per, r * per, k.tensors.ptr,
                                                    static_cast<int>(k.tensors.count), k.state.ptr, beta1, beta2, eps,
                                                    k.stream));
        }
        exchange();                                         // every slice has landed in every weight arena
    }

    void synchronize()
    {
        for (auto &k : ranks)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(k->device));
            B200AMP_HOST_CUDA(cudaStreamSynchronize(k->stream));
        }
    }

    b200amp_step_state read_state(int rank)
    {
        Zero1Rank &k = *ranks[rank];
        b200amp_step_state st;
        B200AMP_HOST_CUDA(cudaSetDevice(k.device));
        B200AMP_HOST_CUDA(cudaMemcpyAsync(&st, k.state.ptr, sizeof(st), cudaMemcpyDeviceToHost, k.stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(k.stream));
        return st;
    }

    // master, m or v of the whole arena, slices in rank order (what a checkpoint holds)
    std::vector<float> gather(DeviceArray<float> Zero1Rank::*which)
    {
        std::vector<float> whole(n);
        synchronize();
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            B200AMP_HOST_CUDA(cudaSetDevice(k.device));
            B200AMP_HOST_CUDA(cudaMemcpy(whole.data() + r * per, (k.*which).ptr, per * sizeof(float),
                                         cudaMemcpyDeviceToHost));
        }
        return whole;
    }
};

} // namespace b200amp_host
