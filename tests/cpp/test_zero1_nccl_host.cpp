// test_zero1_nccl_host.cpp: the one-process ZeRO-1 host with NCCL around the passes
// (include/b200amp_zero1_nccl_host.hpp), tested the reference's way (a table of checks, non-zero
// exit on a failure, cuda/tests/test_fast.cu:44-52). For R = 2, 4 and 8 ranks on R distinct GPUs
// (as many as the machine has): five steps, one with an inf in one rank's gradients, against
// b200amp_host::AmpOptimizer on one GPU stepped with the averaged gradients that NCCL's
// reduce-scatter actually left (gathered from the ranks), and against the fused group
// (Zero1Group) on the same inputs within fp16 rounding of the average.
// With fewer than two GPUs it says so and exits 0. With --time it times the step at the 1.3 B
// arena over all GPUs present. Built by tests/cpp/build_host_test.py, run by tests/test_gpu_host_cpp.py.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "b200amp_zero1_nccl_host.hpp"

using namespace std;
using b200amp_host::AmpOptimizer;
using b200amp_host::Zero1Group;
using b200amp_host::Zero1NcclGroup;
using b200amp_host::Zero1Rank;

static int g_failed = 0;

static void check(bool ok, const string &what)
{
    printf("  %-76s %s\n", what.c_str(), ok ? "ok" : "FAILED");
    if (!ok)
    {
        g_failed++;
    }
}

static b200amp_schedule flat_schedule(int growth_interval)
{
    b200amp_schedule c = {};
    c.lr = 6e-4f;
    c.min_lr = 6e-4f;
    c.warmup_steps = 0;
    c.max_steps = 1 << 30;
    c.beta1 = 0.9f;
    c.beta2 = 0.95f;
    c.weight_decay = 0.1f;
    c.grad_clip = 1.0f;
    c.growth_interval = growth_interval;
    c.dynamic_scale = 1;
    c.decay_steps = 0;
    return c;
}

static vector<float> randn(size_t n, float std, unsigned seed)
{
    mt19937 gen(seed);
    normal_distribution<float> dist(0.0f, std);
    vector<float> out(n);
    for (float &x : out)
    {
        x = dist(gen);
    }
    return out;
}

static double rel_err(const vector<float> &a, const vector<float> &b)
{
    double worst = 0.0, scale = 0.0;
    for (size_t i = 0; i < b.size(); i++)
    {
        worst = fmax(worst, fabs(static_cast<double>(a[i]) - b[i]));
        scale = fmax(scale, fabs(static_cast<double>(b[i])));
    }
    return scale > 0.0 ? worst / scale : worst;
}

static void group_checks(int nranks)
{
    printf("\n%d ranks on %d GPUs, one process, NCCL around the passes\n", nranks, nranks);
    const long long n = 8LL * nranks * 1543 * (8 / nranks + 1);
    const long long per = n / nranks;
    const long long a = n / 3 / 4 * 4, b = n / 2 / 4 * 4;
    vector<b200amp_tensor_info> table = {{0, a, 1}, {a, b - a, 0}, {b, n - b, 1}};
    vector<int> devices(nranks);
    for (int r = 0; r < nranks; r++)
    {
        devices[r] = r;
    }
    const float SCALE = 65536.0f;
    Zero1NcclGroup group(devices, n, table, flat_schedule(2), 1e-8f, SCALE, 16);
    Zero1Group fused(devices, n, table, flat_schedule(2), 1e-8f, SCALE, 16);
    B200AMP_HOST_CUDA(cudaSetDevice(0));
    AmpOptimizer single(n, table, flat_schedule(2), 1e-8f, SCALE, 16);
    vector<float> init = randn(n, 0.02f, 7);
    group.set_params(init);
    fused.set_params(init);
    single.set_params(init);

    bool states_agree = true, decisions_agree = true, fused_agrees = true, norms_agree = true, arenas_agree = true;
    bool average_close = true, skipped_once = false;
    for (int step = 0; step < 5; step++)
    {
        const float scale = group.read_state(0).loss_scale;
        vector<float> sum(n, 0.0f);
        for (int r = 0; r < nranks; r++)
        {
            vector<float> g = randn(n, 1e-3f, 100 + 10 * step + r);
            vector<__half> h(n);
            for (long long i = 0; i < n; i++)
            {
                h[i] = __float2half(g[i] * scale);
            }
            if (step == 2 && r == nranks - 1)
            {
                h[per * (nranks / 2) + 11] = __float2half(INFINITY);
            }
            for (long long i = 0; i < n; i++)
            {
                sum[i] += __half2float(h[i]);
            }
            group.set_grads(r, h);
            fused.set_grads(r, h);
        }
        group.optimizer_step();
        fused.optimizer_step();
        group.synchronize();
        fused.synchronize();
        // what NCCL's reduce-scatter left, gathered: the one-GPU run steps on exactly these values
        vector<__half> avg(n);
        for (int r = 0; r < nranks; r++)
        {
            vector<__half> part = group.ranks[r]->reduced16.download();
            memcpy(avg.data() + r * per, part.data(), per * sizeof(__half));
        }
        if (step != 2)
        {
            for (long long i = 0; i < n; i++)
            {
                const float exact = sum[i] / static_cast<float>(nranks);
                // an fp16 reduction may round after every addition: a few fp16 ulps of the largest addend
                average_close = average_close && fabs(__half2float(avg[i]) - exact) <= 4e-3f * (fabs(exact) + 64.0f);
            }
        }
        B200AMP_HOST_CUDA(cudaSetDevice(0));
        single.set_grads(avg);
        single.optimizer_step();

        const b200amp_step_state want = single.read_state();
        const b200amp_step_state first = group.read_state(0);
        const b200amp_step_state other = fused.read_state(0);
        for (int r = 1; r < nranks; r++)
        {
            const b200amp_step_state st = group.read_state(r);
            states_agree = states_agree && memcmp(&st, &first, sizeof(st)) == 0;
        }
        decisions_agree = decisions_agree && first.loss_scale == want.loss_scale && first.good_steps == want.good_steps &&
                          first.found_inf == want.found_inf && first.skipped == want.skipped && first.step == want.step &&
                          first.adam_t == want.adam_t;
        fused_agrees = fused_agrees && first.loss_scale == other.loss_scale && first.found_inf == other.found_inf &&
                       first.skipped == other.skipped && first.adam_t == other.adam_t;
        if (first.found_inf)
        {
            skipped_once = true;
        }
        else
        {
            norms_agree = norms_agree && fabs(first.grad_norm - want.grad_norm) <= 1e-6 * want.grad_norm &&
                          fabs(first.clip_coef - want.clip_coef) <= 1e-6 * want.clip_coef;
            fused_agrees = fused_agrees && fabs(first.grad_norm - other.grad_norm) <= 2e-3 * other.grad_norm;
        }
        vector<__half> w0 = group.ranks[0]->weights16.download();
        for (int r = 1; r < nranks; r++)
        {
            vector<__half> w = group.ranks[r]->weights16.download();
            arenas_agree = arenas_agree && memcmp(w.data(), w0.data(), n * sizeof(__half)) == 0;
        }
    }
    check(states_agree, "every rank holds the same 60 state bytes after every step");
    check(decisions_agree, "skip decision, loss scale, good_steps, step and adam_t equal the one-GPU run");
    check(skipped_once && group.read_state(0).skipped == 1, "the step with an inf in one rank's gradients was skipped");
    check(norms_agree, "grad_norm and clip_coef within 1e-6 of the one-GPU run on the same averaged gradients");
    check(average_close, "NCCL's fp16 average within fp16 rounding of the fp32 mean");
    check(fused_agrees, "same decisions as the fused group; norms agree to fp16 rounding of the average");
    check(arenas_agree, "every rank's fp16 weight arena holds the same bits after every step");
    const vector<float> master = group.gather(&Zero1Rank::master);
    check(rel_err(master, single.master.download()) <= 1e-6, "master within 1e-6 of the one-GPU run");
    check(rel_err(group.gather(&Zero1Rank::m), single.m.download()) <= 1e-6, "m within 1e-6");
    check(rel_err(group.gather(&Zero1Rank::v), single.v.download()) <= 1e-6, "v within 1e-6");
    const vector<__half> w = group.ranks[nranks - 1]->weights16.download();
    bool cast_exact = true;
    for (long long i = 0; i < n; i++)
    {
        const __half want = __float2half(master[i]);
        cast_exact = cast_exact && memcmp(&want, &w[i], sizeof(__half)) == 0;
    }
    check(cast_exact, "the gathered fp16 arena is fp16(master) everywhere");
}

// --time: the 1.3 B arena over all GPUs present, CUDA events on rank 0's stream around 10 steps
// after 3 warm-up steps. Arenas are filled by tiling one random block.
static void time_large(int nranks)
{
    const long long n = 1315819520LL;
    vector<b200amp_tensor_info> table = {{0, n, 1}};
    vector<int> devices(nranks);
    for (int r = 0; r < nranks; r++)
    {
        devices[r] = r;
    }
    Zero1NcclGroup group(devices, n, table, flat_schedule(2000), 1e-8f, 32768.0f, 16);
    const long long block = 1 << 22;
    vector<float> g = randn(block, 1e-3f * 32768.0f, 3);
    vector<__half> h(block);
    for (long long i = 0; i < block; i++)
    {
        h[i] = __float2half(g[i]);
    }
    for (auto &k : group.ranks)
    {
        B200AMP_HOST_CUDA(cudaSetDevice(k->device));
        for (long long at = 0; at < n; at += block)
        {
            const long long count = at + block <= n ? block : n - at;
            B200AMP_HOST_CUDA(cudaMemcpyAsync(k->grads16.ptr + at, h.data(), count * sizeof(__half),
                                              cudaMemcpyHostToDevice, k->stream));
        }
    }
    group.synchronize();
    for (int i = 0; i < 3; i++)
    {
        group.optimizer_step();
    }
    group.synchronize();
    Zero1Rank &k0 = *group.ranks[0];
    cudaEvent_t e0, e1;
    B200AMP_HOST_CUDA(cudaSetDevice(k0.device));
    B200AMP_HOST_CUDA(cudaEventCreate(&e0));
    B200AMP_HOST_CUDA(cudaEventCreate(&e1));
    const int steps = 10;
    B200AMP_HOST_CUDA(cudaEventRecord(e0, k0.stream));
    for (int i = 0; i < steps; i++)
    {
        group.optimizer_step();
    }
    B200AMP_HOST_CUDA(cudaSetDevice(k0.device));
    B200AMP_HOST_CUDA(cudaEventRecord(e1, k0.stream));
    group.synchronize();
    float ms = 0.0f;
    B200AMP_HOST_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    const b200amp_step_state st = group.read_state(0);
    printf("%d ranks, NCCL around the passes, 1.3 B arena: %.3f ms/step, %.1f Gparams/s (skipped %d of %d)\n", nranks,
           ms / steps, n / (ms / steps * 1e-3) / 1e9, st.skipped, st.step);
}

int main(int argc, char **argv)
{
    int count = 0;
    B200AMP_HOST_CUDA(cudaGetDeviceCount(&count));
    printf("ZeRO-1 NCCL host layer over libb200amp %s, %d GPU%s visible\n", b200amp_version(), count,
           count == 1 ? "" : "s");
    if (count < 2)
    {
        printf("NCCL wants one GPU per rank and this machine shows %d: nothing to check\n", count);
        return 0;
    }
    if (argc > 1 && string(argv[1]) == "--time")
    {
        int nranks = 2;
        while (nranks * 2 <= count && nranks * 2 <= 8)
        {
            nranks *= 2;
        }
        time_large(nranks);
        return 0;
    }
    for (int nranks = 2; nranks <= 8 && nranks <= count; nranks *= 2)
    {
        group_checks(nranks);
    }
    printf("\n%s\n", g_failed == 0 ? "all checks passed" : "SOME CHECKS FAILED");
    return g_failed == 0 ? 0 : 1;
}
