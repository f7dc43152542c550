// test_amp_host.cpp: the reference's way of testing (a program that prints a table of checks and
// exits non-zero on a failure, cuda/tests/test_fast.cu:44-52) applied to the C++ host layer:
//   * the reference-signature shim (include/compat/fast_shim.h) driven exactly as
//     FastGPT::optimizer_step does (cuda/gpt_fast.cu:438-450), with the expectations of
//     scaler_checks (cuda/tests/test_fast.cu:272-326);
//   * b200amp_host::AmpOptimizer (fp16 gradient arena) against the shim path on the same values;
//   * graph_checks (cuda/tests/test_fast.cu:330-371): capture runs nothing, replays equal eager.
// Needs a GPU. Built by tests/cpp/build_host_test.py, run by tests/test_gpu_host_cpp.py.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "b200amp_host.hpp"
#include "compat/fast_shim.h"

using namespace std;
using b200amp_host::AmpOptimizer;
using b200amp_host::DeviceArray;

static int g_failed = 0;

static void check(bool ok, const string &what)
{
    printf("  %-72s %s\n", what.c_str(), ok ? "ok" : "FAILED");
    if (!ok)
    {
        g_failed++;
    }
}

static ScheduleConfig flat_schedule(int growth_interval)
{
    ScheduleConfig c = {};
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

// The optimizer part of FastGPT with the reference's own arena types (fp32 gradients), driven
// through the shim's reference signatures.
struct CompatModel
{
    long long n;
    cudaStream_t stream;
    DeviceArray<float> params, grads, m, v, partial;
    DeviceArray<floatX> params_x;
    DeviceArray<TensorInfo> tensors;
    DeviceArray<StepState> state, history;
    ScheduleConfig sched;
    int history_len = 64;

    CompatModel(long long n_, const vector<TensorInfo> &table, ScheduleConfig cfg, float scale)
        : n(n_), params(n_), grads(n_), m(n_), v(n_), partial(NORM_BLOCKS), params_x(n_), tensors(table.size()),
          state(1), history(64), sched(cfg)
    {
        B200AMP_HOST_CUDA(cudaStreamCreate(&stream));
        B200AMP_HOST_CUDA(cudaMemcpy(tensors.ptr, table.data(), table.size() * sizeof(TensorInfo),
                                     cudaMemcpyHostToDevice));
        reset(scale);
    }
    void reset(float scale)
    {
        m.zero(stream);
        v.zero(stream);
        grads.zero(stream);
        StepState st = initial_state(scale);
        B200AMP_HOST_CUDA(cudaMemcpyAsync(state.ptr, &st, sizeof(st), cudaMemcpyHostToDevice, stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));
    }
    void set_params(const vector<float> &host)
    {
        B200AMP_HOST_CUDA(cudaMemcpy(params.ptr, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
        cast_to_x(params_x.ptr, params.ptr, n, stream);
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));
    }
    void set_grads(const vector<float> &host)
    {
        B200AMP_HOST_CUDA(cudaMemcpy(grads.ptr, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    void optimizer_step()
    {
        unscale_and_norm(grads.ptr, n, state.ptr, partial.ptr, stream);
        finalize_step(state.ptr, partial.ptr, sched, history.ptr, history_len, stream);
        adamw_multi(params.ptr, params_x.ptr, grads.ptr, m.ptr, v.ptr, n, tensors.ptr, static_cast<int>(tensors.count),
                    state.ptr, sched.beta1, sched.beta2, 1e-8f, stream);
    }
    void train_step_on(const vector<float> &scaled_grads)
    {
        begin_step(state.ptr, stream);
        set_grads(scaled_grads);
        optimizer_step();
    }
    StepState read_state()
    {
        StepState st;
        B200AMP_HOST_CUDA(cudaMemcpyAsync(&st, state.ptr, sizeof(st), cudaMemcpyDeviceToHost, stream));
        B200AMP_HOST_CUDA(cudaStreamSynchronize(stream));
        return st;
    }
};

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

static vector<float> scaled_fp16_values(const vector<float> &g, float scale, vector<__half> *as_half)
{
    vector<float> out(g.size());
    as_half->resize(g.size());
    for (size_t i = 0; i < g.size(); i++)
    {
        __half h = __float2half(g[i] * scale);
        (*as_half)[i] = h;
        out[i] = __half2float(h);               // what a backward pass into fp32 gradients would hold
    }
    return out;
}

static bool same_bits(const vector<float> &a, const vector<float> &b)
{
    return a.size() == b.size() && memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0;
}

static void scaler_checks()
{
    printf("\nloss scaler through the reference-signature shim: skipped steps and growth\n");
    const long long n = 1 << 18;
    const float SCALE = 65536.0f;
    vector<TensorInfo> table = {{0, n / 2, 1}, {n / 2, n / 2, 0}};
    CompatModel model(n, table, flat_schedule(2000), SCALE);
    vector<float> init = randn(n, 0.02f, 1);
    model.set_params(init);
    vector<float> before = model.params.download();
    vector<__half> unused;

    vector<float> g = scaled_fp16_values(randn(n, 1e-3f, 2), SCALE, &unused);
    g[12345 % n] = INFINITY;
    model.train_step_on(g);
    StepState st = model.read_state();
    check(st.found_inf == 1 && st.skipped == 1, "an inf gradient is found and the step is skipped");
    check(st.adam_t == 0 && st.step == 1, "AdamW t stays 0, the schedule step moves on");
    check(same_bits(model.params.download(), before), "the parameters did not move");
    bool m_zero = true;
    for (float x : model.m.download())
    {
        m_zero = m_zero && x == 0.0f;
    }
    check(m_zero, "AdamW m did not move");
    check(st.loss_scale == SCALE / 2 && st.good_steps == 0, "S halved");

    model.train_step_on(scaled_fp16_values(randn(n, 1e-3f, 3), SCALE / 2, &unused));
    st = model.read_state();
    check(st.found_inf == 0 && st.adam_t == 1 && st.step == 2 && st.skipped == 1, "the next step runs (t 1, step 2)");
    check(!same_bits(model.params.download(), before), "and moves the parameters");

    model.sched.growth_interval = 2;
    model.train_step_on(scaled_fp16_values(randn(n, 1e-3f, 4), SCALE / 2, &unused));
    st = model.read_state();
    check(st.loss_scale == SCALE && st.good_steps == 0, "2 finite steps in a row: S doubles back to 65,536");

    model.reset(1073741824.0f);
    vector<float> overflow = scaled_fp16_values(randn(n, 1e-3f, 5), 1073741824.0f, &unused);   // fp16 saturates to inf
    model.train_step_on(overflow);
    st = model.read_state();
    check(st.found_inf == 1 && st.skipped == 1, "S = 2^30 overflows fp16: found and skipped");
    check(st.loss_scale == 536870912.0f, "S halved to 2^29");

    ScheduleConfig wsd = flat_schedule(2000);
    wsd.lr = 6e-4f;
    wsd.min_lr = 6e-5f;
    wsd.warmup_steps = 10;
    wsd.max_steps = 100;
    wsd.decay_steps = 20;
    bool lr_ok = fabs(lr_on_gpu(0, wsd) - static_cast<double>(wsd.lr) / 10) < 1e-15 &&
                 fabs(lr_on_gpu(50, wsd) - static_cast<double>(wsd.lr)) < 1e-15 &&
                 fabs(lr_on_gpu(100, wsd) - static_cast<double>(wsd.min_lr)) < 1e-15;
    check(lr_ok, "lr_on_gpu: warmup, flat and floor of the WSD schedule");
}

static void native_against_compat()
{
    printf("\nfp16 gradient arena (AmpOptimizer) against the reference-signature path, same values\n");
    const long long n = 1 << 20;
    const float SCALE = 65536.0f;
    vector<TensorInfo> table = {{0, 4096, 0}, {4096, n - 4096, 1}};
    CompatModel compat(n, table, flat_schedule(3), SCALE);
    AmpOptimizer native(n, table, flat_schedule(3), 1e-8f, SCALE);
    vector<float> init = randn(n, 0.02f, 7);
    compat.set_params(init);
    native.set_params(init);
    bool control_same = true, close = true;
    for (int k = 0; k < 6; k++)
    {
        float S = native.read_state().loss_scale;
        vector<__half> g16;
        vector<float> g32 = scaled_fp16_values(randn(n, 1e-3f, 100 + k), S, &g16);
        if (k == 3)
        {
            g16[777] = __float2half(INFINITY);
            g32[777] = INFINITY;
        }
        native.set_grads(g16);
        native.optimizer_step();
        compat.train_step_on(g32);
        StepState a = native.read_state(), b = compat.read_state();
        control_same = control_same && a.loss_scale == b.loss_scale && a.inv_scale == b.inv_scale &&
                       a.good_steps == b.good_steps && a.found_inf == b.found_inf && a.skipped == b.skipped &&
                       a.step == b.step && a.adam_t == b.adam_t && a.lr == b.lr && a.step_size == b.step_size &&
                       a.bc2_sqrt == b.bc2_sqrt && a.decay == b.decay;
        if (k != 3)
        {
            close = close && fabsf(a.grad_norm - b.grad_norm) <= 1e-6f * b.grad_norm;
        }
    }
    check(control_same, "skip decisions, loss scale, counters and step scalars identical on every step");
    check(close, "gradient norms agree to 1e-6");
    vector<float> pa = native.master.download(), pb = compat.params.download();
    float worst = 0.0f, scale = 0.0f;
    for (size_t i = 0; i < pa.size(); i++)
    {
        worst = fmaxf(worst, fabsf(pa[i] - pb[i]));
        scale = fmaxf(scale, fabsf(pb[i]));
    }
    check(worst <= 1e-6f * scale, "master weights agree to 1e-6 of the largest value");
    vector<__half> wa = native.weights16.download();
    size_t off = 0;
    for (size_t i = 0; i < pa.size(); i++)
    {
        if (__half2float(wa[i]) != __half2float(__float2half(pa[i])))
        {
            off++;
        }
    }
    check(off == 0, "the fp16 weight copy is exactly fp16(params) after the steps");
    StepState st = native.read_state();
    check(st.skipped == 1 && st.adam_t == 5 && st.step == 6, "one skipped step of six");
}

static void graph_checks()
{
    printf("\nCUDA Graph: 4 captured steps against 4 eager steps\n");
    const int STEPS = 4;
    const long long n = 1 << 18;
    vector<TensorInfo> table = {{0, n, 1}};
    AmpOptimizer eager(n, table, flat_schedule(2000), 1e-8f, 65536.0f);
    AmpOptimizer graphed(n, table, flat_schedule(2000), 1e-8f, 65536.0f);
    vector<float> init = randn(n, 0.02f, 11);
    vector<__half> g16;
    scaled_fp16_values(randn(n, 1e-3f, 12), 65536.0f, &g16);
    for (AmpOptimizer *o : {&eager, &graphed})
    {
        o->set_params(init);
        o->set_grads(g16);
    }
    for (int k = 0; k < STEPS; k++)
    {
        eager.optimizer_step();
    }
    CudaGraph graph;
    graph.capture(graphed.stream, [&]() { graphed.optimizer_step(); });
    check(graph.ready() && graphed.read_state().step == 0, "capturing ran nothing");
    for (int k = 0; k < STEPS; k++)
    {
        graph.launch(graphed.stream);
    }
    StepState a = eager.read_state(), b = graphed.read_state();
    check(a.step == STEPS && b.step == STEPS && b.adam_t == STEPS, "both took 4 steps");
    check(memcmp(&a, &b, sizeof(a)) == 0, "the 60 state bytes are identical");
    check(same_bits(eager.master.download(), graphed.master.download()), "parameters after 4 steps: same bits");
    check(same_bits(eager.v.download(), graphed.v.download()), "AdamW v after 4 steps: same bits");
}

static void host_feed_checks()
{
    printf("\nsteps fed from pinned host memory (two arenas taking turns) against serial steps\n");
    const int STEPS = 5;
    const long long n = 1 << 18;
    vector<TensorInfo> table = {{0, n / 2, 1}, {n / 2, n / 2, 0}};
    AmpOptimizer serial(n, table, flat_schedule(2), 1e-8f, 4096.0f);
    AmpOptimizer fed(n, table, flat_schedule(2), 1e-8f, 4096.0f);
    vector<float> init = randn(n, 0.02f, 21);
    serial.set_params(init);
    fed.set_params(init);
    __half *pinned = nullptr;
    B200AMP_HOST_CUDA(cudaMallocHost(&pinned, STEPS * n * sizeof(__half)));
    vector<StepState> want;
    for (int k = 0; k < STEPS; k++)
    {
        vector<__half> g16;
        scaled_fp16_values(randn(n, 1e-3f, 30 + k), 4096.0f, &g16);
        if (k == 2)
        {
            g16[777] = __float2half(INFINITY);
        }
        memcpy(pinned + k * n, g16.data(), n * sizeof(__half));
        serial.set_grads(g16);
        serial.optimizer_step();
        want.push_back(serial.read_state());
    }
    bool states_same = true;
    {
        b200amp_host::HostGradientFeed feed(fed);
        long long last = -1;
        for (int k = 0; k < STEPS; k++)
        {
            const long long ticket = feed.submit(pinned + k * n);
            if (last >= 0)
            {
                const StepState got = feed.collect(last);
                states_same = states_same && memcmp(&got, &want[last], sizeof(got)) == 0;
            }
            last = ticket;
        }
        const StepState got = feed.collect(last);
        states_same = states_same && memcmp(&got, &want[last], sizeof(got)) == 0;
    }
    B200AMP_HOST_CUDA(cudaFreeHost(pinned));
    check(states_same, "every step's 60 state bytes equal the serial run's (one skipped step of five)");
    check(same_bits(serial.master.download(), fed.master.download()), "parameters after 5 steps: same bits");
    check(same_bits(serial.m.download(), fed.m.download()) && same_bits(serial.v.download(), fed.v.download()),
          "AdamW m and v after 5 steps: same bits");
    const StepState st = fed.read_state();
    check(st.skipped == 1 && st.adam_t == 4 && st.step == 5, "one skipped step, four applied");
}

int main()
{
    static_assert(sizeof(StepState) == 60, "StepState is the reference's 60-byte checkpoint ABI");
    static_assert(sizeof(ScheduleConfig) == 44 && sizeof(TensorInfo) == 24, "struct layouts");
    if (b200amp_device_check() != B200AMP_OK)
    {
        fprintf(stderr, "%s\n", b200amp_last_error());
        return 2;
    }
    scaler_checks();
    native_against_compat();
    graph_checks();
    host_feed_checks();
    printf("\n%s\n", g_failed == 0 ? "all checks passed" : "SOME CHECKS FAILED");
    return g_failed == 0 ? 0 : 1;
}
