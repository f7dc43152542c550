// test_zero1_host.cpp: the one-process ZeRO-1 host layer (include/b200amp_zero1_host.hpp), tested
// the reference's way (a program that prints a table of checks and exits non-zero on a failure,
// cuda/tests/test_fast.cu:44-52). For R = 1, 2, 4 and 8 ranks, spread over the GPUs the machine
// has (rank r on device r mod count, so one GPU runs every rank):
//   * five steps, one with an inf in one rank's gradients, against b200amp_host::AmpOptimizer on
//     one GPU stepped with the averaged gradients fp16(fp32 sum in rank order / R);
//   * every rank holds the same 60 state bytes and the same fp16 weight arena after every step.
// With --time it times the step at the 1.3 B arena over all GPUs present instead.
// Needs a GPU. Built by tests/cpp/build_host_test.py, run by tests/test_gpu_host_cpp.py.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "b200amp_zero1_host.hpp"

using namespace std;
using b200amp_host::AmpOptimizer;
using b200amp_host::Zero1Group;
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

// max |a - b| / max |b|, the reference's own measure (cuda/dump.cu:244-268)
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

static int half_order(__half h)          // fp16 bit pattern as an integer in value order
{
    unsigned short bits;
    memcpy(&bits, &h, sizeof(bits));
    return (bits & 0x8000u) ? -static_cast<int>(bits & 0x7FFFu) : static_cast<int>(bits);
}

static void group_checks(int nranks, int device_count)
{
    printf("\n%d rank%s on %d GPU%s, one process, events between the phases\n", nranks, nranks > 1 ? "s" : "",
           device_count < nranks ? device_count : nranks, device_count > 1 && nranks > 1 ? "s" : "");
    const long long n = 8LL * nranks * 1543 * (8 / nranks + 1);
    const long long per = n / nranks;
    const long long a = n / 3 / 4 * 4, b = n / 2 / 4 * 4;         // tensor edges inside slices and inside groups
    vector<b200amp_tensor_info> table = {{0, a, 1}, {a, b - a, 0}, {b, n - b, 1}};
    vector<int> devices(nranks);
    for (int r = 0; r < nranks; r++)
    {
        devices[r] = r % device_count;
    }
    const float SCALE = 65536.0f;
    Zero1Group group(devices, n, table, flat_schedule(2), 1e-8f, SCALE, 16);
    B200AMP_HOST_CUDA(cudaSetDevice(0));
    AmpOptimizer single(n, table, flat_schedule(2), 1e-8f, SCALE, 16);
    vector<float> init = randn(n, 0.02f, 7);
    group.set_params(init);
    single.set_params(init);

    bool states_agree = true, decisions_agree = true, norms_agree = true, arenas_agree = true, skipped_once = false;
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
                sum[i] += __half2float(h[i]);                   // fp32, in rank order, as rs_pass1 adds
            }
            group.set_grads(r, h);
        }
        vector<__half> avg(n);
        const float inv_ranks = 1.0f / static_cast<float>(nranks);
        for (long long i = 0; i < n; i++)
        {
            avg[i] = __float2half(sum[i] * inv_ranks);
        }
        B200AMP_HOST_CUDA(cudaSetDevice(0));
        single.set_grads(avg);
        group.optimizer_step();
        single.optimizer_step();
        group.synchronize();

        const b200amp_step_state want = single.read_state();
        const b200amp_step_state first = group.read_state(0);
        for (int r = 1; r < nranks; r++)
        {
            const b200amp_step_state st = group.read_state(r);
            states_agree = states_agree && memcmp(&st, &first, sizeof(st)) == 0;
        }
        decisions_agree = decisions_agree && first.loss_scale == want.loss_scale && first.good_steps == want.good_steps &&
                          first.found_inf == want.found_inf && first.skipped == want.skipped && first.step == want.step &&
                          first.adam_t == want.adam_t;
        if (first.found_inf)
        {
            skipped_once = true;
        }
        else
        {
            norms_agree = norms_agree && fabs(first.grad_norm - want.grad_norm) <= 1e-6 * want.grad_norm &&
                          fabs(first.clip_coef - want.clip_coef) <= 1e-6 * want.clip_coef;
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
    check(norms_agree, "grad_norm and clip_coef within 1e-6 of the one-GPU run");
    check(arenas_agree, "every rank's fp16 weight arena holds the same bits after every step");

    const vector<float> master = group.gather(&Zero1Rank::master);
    check(rel_err(master, single.master.download()) <= 1e-6, "master within 1e-6 of the one-GPU run");
    check(rel_err(group.gather(&Zero1Rank::m), single.m.download()) <= 1e-6, "m within 1e-6");
    check(rel_err(group.gather(&Zero1Rank::v), single.v.download()) <= 1e-6, "v within 1e-6");
    const vector<__half> w = group.ranks[nranks - 1]->weights16.download();
    const vector<__half> ws = single.weights16.download();
    bool cast_exact = true;
    int far = 0;
    for (long long i = 0; i < n; i++)
    {
        const __half want = __float2half(master[i]);
        cast_exact = cast_exact && memcmp(&want, &w[i], sizeof(__half)) == 0;
        const int d = half_order(w[i]) - half_order(ws[i]);
        far = d > far ? d : (-d > far ? -d : far);
    }
    check(cast_exact, "the gathered fp16 arena is fp16(master) everywhere");
    check(far <= 1, "fp16 weights within 1 ulp of the one-GPU run");
}

// --time: the 1.3 B arena (config 4) over all the GPUs present, CUDA events on rank 0's stream
// around 10 steps after 3 warm-up steps. Arenas are filled by tiling one random block.
static void time_full_arena(int device_count)
{
    const int nranks = device_count >= 8 ? 8 : device_count >= 4 ? 4 : device_count >= 2 ? 2 : 1;
    const long long n = 1315819520LL;
    vector<b200amp_tensor_info> table = {{0, 103022592LL, 1}, {103022592LL, n - 103022592LL - 4096, 1},
                                         {n - 4096, 4096, 0}};
    vector<int> devices(nranks);
    for (int r = 0; r < nranks; r++)
    {
        devices[r] = r;
    }
    Zero1Group group(devices, n, table, flat_schedule(2000), 1e-8f, 32768.0f, 16);
    const long long block = 1 << 20;
    vector<float> p = randn(block, 0.02f, 1);
    for (int r = 0; r < nranks; r++)
    {
        Zero1Rank &k = *group.ranks[r];
        B200AMP_HOST_CUDA(cudaSetDevice(k.device));
        vector<float> g = randn(block, 1e-3f * 32768.0f, 10 + r);
        vector<__half> h(block);
        for (long long i = 0; i < block; i++)
        {
            h[i] = __float2half(g[i]);
        }
        for (long long at = 0; at < n; at += block)
        {
            const long long count = at + block <= n ? block : n - at;
            B200AMP_HOST_CUDA(cudaMemcpyAsync(k.grads16.ptr + at, h.data(), count * sizeof(__half),
                                              cudaMemcpyHostToDevice, k.stream));
        }
        for (long long at = 0; at < group.per; at += block)
        {
            const long long count = at + block <= group.per ? block : group.per - at;
            B200AMP_HOST_CUDA(cudaMemcpyAsync(k.master.ptr + at, p.data(), count * sizeof(float),
                                              cudaMemcpyHostToDevice, k.stream));
        }
        B200AMP_HOST_CUDA(cudaStreamSynchronize(k.stream));
    }
    for (int i = 0; i < 3; i++)
    {
        group.optimizer_step();
    }
    group.synchronize();
    Zero1Rank &first = *group.ranks[0];
    cudaEvent_t t0, t1;
    B200AMP_HOST_CUDA(cudaSetDevice(first.device));
    B200AMP_HOST_CUDA(cudaEventCreate(&t0));
    B200AMP_HOST_CUDA(cudaEventCreate(&t1));
    const int steps = 10;
    B200AMP_HOST_CUDA(cudaEventRecord(t0, first.stream));
    for (int i = 0; i < steps; i++)
    {
        group.optimizer_step();            // ends with an exchange: rank 0's stream has waited for all
    }
    B200AMP_HOST_CUDA(cudaSetDevice(first.device));
    B200AMP_HOST_CUDA(cudaEventRecord(t1, first.stream));
    group.synchronize();
    float ms = 0.0f;
    B200AMP_HOST_CUDA(cudaEventElapsedTime(&ms, t0, t1));
    const b200amp_step_state st = group.read_state(0);
    printf("timing: %d ranks, %lld params, %.3f ms/step, %.1f Gparams/s (step %d, skipped %d, grad_norm %.4f)\n",
           nranks, n, ms / steps, n / (ms / steps * 1e-3) / 1e9, st.step, st.skipped, st.grad_norm);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
}

int main(int argc, char *argv[])
{
    int device_count = 0;
    B200AMP_HOST_CUDA(cudaGetDeviceCount(&device_count));
    if (device_count < 1)
    {
        fprintf(stderr, "no CUDA device\n");
        return 2;
    }
    if (argc > 1 && strcmp(argv[1], "--time") == 0)
    {
        time_full_arena(device_count);
        return 0;
    }
    printf("ZeRO-1 host layer over libb200amp %s, %d GPU%s visible\n", b200amp_version(), device_count,
           device_count > 1 ? "s" : "");
    for (int nranks : {1, 2, 4, 8})
    {
        group_checks(nranks, device_count);
    }
    if (g_failed == 0)
    {
        printf("\nall checks passed\n");
        return 0;
    }
    printf("\n%d checks FAILED\n", g_failed);
    return 1;
}
