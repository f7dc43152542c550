// b200amp_zero1_nccl_host.hpp: the ZeRO-1 form of the step with NCCL collectives AROUND the two
// passes, driven from one host process over R GPUs (ncclCommInitAll), in C++ over the C ABI.
//
// This is the plain sharding of the step: reduce-scatter of the fp16 gradients (ncclAvg), pass 1
// on the rank's slice, an all-reduce of the two doubles {sum of squares, flag}, the finalize on
// every rank (replicated state, identical bits: every rank adds the same reduced pair), pass 2 on
// the slice with the slice's offset in the arena, and an in-place all-gather of the fp16 weights.
// The reference has no multi-GPU code; the sequence per rank is FastGPT::optimizer_step
// (cuda/gpt_fast.cu:438-450) with the collectives put where the data crosses ranks.
// Zero1Group (b200amp_zero1_host.hpp) is the faster form of the same step, with the collectives
// folded into the kernels; this one needs nothing mapped between the GPUs beyond what NCCL sets up,
// and is the baseline the fused form is measured against.
//
// The inf/NaN flag and the norm are taken on the averaged gradients that the reduce-scatter
// leaves (NCCL's fp16 average), as a data-parallel trainer with a gradient scaler would see them.
// Every device must be distinct (NCCL refuses two ranks on one GPU).
#pragma once

#include <nccl.h>

#include "b200amp_zero1_host.hpp"

#define B200AMP_HOST_NCCL(call)                                                                         \
    do                                                                                                  \
    {                                                                                                   \
        ncclResult_t res_ = (call);                                                                     \
        if (res_ != ncclSuccess)                                                                        \
        {                                                                                               \
            fprintf(stderr, "NCCL error at %s:%d: %s (%s)\n", __FILE__, __LINE__, ncclGetErrorString(res_), #call); \
            exit(1);                                                                                    \
        }                                                                                               \
    } while (0)

namespace b200amp_host
{

struct Zero1NcclGroup : Zero1Group
{
    std::vector<ncclComm_t> comms;

    Zero1NcclGroup(const std::vector<int> &devices, long long n_, const std::vector<b200amp_tensor_info> &table,
                   b200amp_schedule cfg, float eps_, float loss_scale, int history_len_ = 256)
        : Zero1Group(devices, n_, table, cfg, eps_, loss_scale, history_len_), comms(devices.size())
    {
        B200AMP_HOST_NCCL(ncclCommInitAll(comms.data(), nranks, devices.data()));
    }
    ~Zero1NcclGroup()
    {
        for (ncclComm_t c : comms)
        {
            if (c != nullptr)
            {
                ncclCommDestroy(c);
            }
        }
    }

    void optimizer_step()
    {
        // reduce-scatter: slice r of every rank's arena, averaged, into rank r's reduced16
        B200AMP_HOST_NCCL(ncclGroupStart());
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            B200AMP_HOST_NCCL(ncclReduceScatter(k.grads16.ptr, k.reduced16.ptr, static_cast<size_t>(per), ncclHalf,
                                                ncclAvg, comms[r], k.stream));
        }
        B200AMP_HOST_NCCL(ncclGroupEnd());
        for (auto &k : ranks)
        {
            B200AMP_HOST_CUDA(cudaSetDevice(k->device));
            B200AMP_HOST_CHECK(b200amp_pass1_f16(k->reduced16.ptr, per, k->state.ptr, k->workspace.ptr, k->stream));
        }
        // the scalar exchange: {sum of squares, flag} are the first two doubles of the workspace
        B200AMP_HOST_NCCL(ncclGroupStart());
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            B200AMP_HOST_NCCL(ncclAllReduce(k.workspace.ptr, k.pairs.ptr, 2, ncclDouble, ncclSum, comms[r], k.stream));
        }
        B200AMP_HOST_NCCL(ncclGroupEnd());
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            B200AMP_HOST_CUDA(cudaSetDevice(k.device));
            // one pair: the sums of all ranks (any flag > 0 means some rank saw an inf or NaN)
            B200AMP_HOST_CHECK(b200amp_finalize_sums(k.state.ptr, k.pairs.ptr, 1, &sched, k.history.ptr, history_len,
                                                     k.stream));
            B200AMP_HOST_CHECK(b200amp_pass2_f16(k.master.ptr, k.m.ptr, k.v.ptr, k.reduced16.ptr,
                                                 k.weights16.ptr + r * per, per, r * per, k.tensors.ptr,
                                                 static_cast<int>(k.tensors.count), k.state.ptr, beta1, beta2, eps,
                                                 k.stream));
        }
        B200AMP_HOST_NCCL(ncclGroupStart());
        for (int r = 0; r < nranks; r++)
        {
            Zero1Rank &k = *ranks[r];
            B200AMP_HOST_NCCL(ncclAllGather(k.weights16.ptr + r * per, k.weights16.ptr, static_cast<size_t>(per),
                                            ncclHalf, comms[r], k.stream));
        }
        B200AMP_HOST_NCCL(ncclGroupEnd());
    }
};

} // namespace b200amp_host
