// api.cu: the parts of the C ABI that are not kernels: error text, version, device
// check, tuning knobs, the launch counter, the all-in-one step and the CUDA-graph
// helpers (capture / launch, cuda/graph.cu:17-41 of the reference).

#include <atomic>
#include <cstring>
#include <new>

#include "internal.cuh"

namespace b200amp
{

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t err, const char *what, const char *file, int line)
{
    set_error("CUDA error at %s:%d: %s (%s)", file, line, cudaGetErrorString(err), what);
    return B200AMP_ERR_CUDA;
}

void count_launch()
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
}

int sm_count()
{
    constexpr int MAX_DEVICES = 64;
    static std::atomic<int> cache[MAX_DEVICES];
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
    {
        cuda_fail(err, "cudaGetDevice", __FILE__, __LINE__);
        return -1;
    }
    if (dev < 0 || dev >= MAX_DEVICES)
    {
        set_error("device index %d is outside the %d devices this library keeps state for", dev, MAX_DEVICES);
        return -1;
    }
    int have = cache[dev].load(std::memory_order_relaxed);
    if (have > 0)
    {
        return have;
    }
    int sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess || sms <= 0)
    {
        cuda_fail(err, "cudaDeviceGetAttribute(MultiProcessorCount)", __FILE__, __LINE__);
        return -1;
    }
    cache[dev].store(sms, std::memory_order_relaxed);
    return sms;
}

Tunables &tunables()
{
    static Tunables t = {4, 2, 1, 256, 0, 6, 0, 8, 0, 16, 2};   // measured best on B200 at the 1.3 B arena
    return t;
}

struct Knob
{
    const char *key;
    int Tunables::*field;
    int lo, hi;
};

static const Knob KNOBS[] = {
    {"pass1_blocks_per_sm", &Tunables::pass1_blocks_per_sm, 1, 32},
    {"pass2_blocks_per_sm", &Tunables::pass2_blocks_per_sm, 1, 32},
    {"pass2_store_hint", &Tunables::pass2_store_hint, 0, 1},
    {"pass2_threads", &Tunables::pass2_threads, 256, 1024},
    {"pass2_variant", &Tunables::pass2_variant, 0, 1},
    {"pass2_stages", &Tunables::pass2_stages, 3, 7},
    {"pass2_test_starve", &Tunables::pass2_test_starve, 0, 1},
    {"rs_blocks_per_sm", &Tunables::rs_blocks_per_sm, 1, 32},
    {"ag_blocks_per_sm", &Tunables::ag_blocks_per_sm, 0, 32},
    {"bridge_blocks_per_sm", &Tunables::bridge_blocks_per_sm, 1, 32},
    {"ce_lanes", &Tunables::ce_lanes, 1, 7},
};

} // namespace b200amp

using namespace b200amp;

struct b200amp_graph
{
    cudaGraphExec_t exec;
};

extern "C" B200AMP_API const char *b200amp_last_error(void)
{
    return g_error;
}

extern "C" B200AMP_API const char *b200amp_version(void)
{
    return "0.2.0";
}

extern "C" B200AMP_API int b200amp_device_check(void)
{
    int dev = 0;
    B200AMP_CUDA(cudaGetDevice(&dev));
    int major = 0;
    B200AMP_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10)
    {
        set_error("device %d has compute capability %d.x; this library holds sm_100a code only", dev, major);
        return B200AMP_ERR_DEVICE;
    }
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_check_tensor_table(const b200amp_tensor_info *host_table, int ntensors,
                                                      long long n)
{
    B200AMP_REQUIRE(host_table != nullptr, "tensor table: null pointer");
    B200AMP_REQUIRE(ntensors > 0 && ntensors <= B200AMP_MAX_TENSORS, "tensor table: %d entries, must be 1..%d",
                    ntensors, B200AMP_MAX_TENSORS);
    for (int k = 0; k < ntensors; k++)
    {
        const b200amp_tensor_info &t = host_table[k];
        B200AMP_REQUIRE(t.offset >= 0 && t.offset % 4 == 0, "tensor table: entry %d starts at %lld, not a multiple "
                                                            "of 4", k, t.offset);
        B200AMP_REQUIRE(t.count > 0, "tensor table: entry %d has %lld elements", k, t.count);
        B200AMP_REQUIRE(t.decay == 0 || t.decay == 1, "tensor table: entry %d has decay flag %d", k, t.decay);
        if (k + 1 < ntensors)
        {
            B200AMP_REQUIRE(t.offset + t.count <= host_table[k + 1].offset,
                            "tensor table: entry %d (%lld + %lld) reaches into entry %d (%lld)", k, t.offset, t.count,
                            k + 1, host_table[k + 1].offset);
        }
        else if (n > 0)
        {
            B200AMP_REQUIRE(t.offset + t.count <= n, "tensor table: entry %d ends at %lld, the arena has %lld "
                                                     "elements", k, t.offset + t.count, n);
        }
    }
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_tune_set(const char *key, int value)
{
    B200AMP_REQUIRE(key != nullptr, "tune_set: key is null");
    for (const Knob &k : KNOBS)
    {
        if (strcmp(k.key, key) == 0)
        {
            B200AMP_REQUIRE(value >= k.lo && value <= k.hi, "tune_set: %s = %d outside %d..%d", key, value, k.lo,
                            k.hi);
            tunables().*(k.field) = value;
            return B200AMP_OK;
        }
    }
    set_error("tune_set: no knob named %s", key);
    return B200AMP_ERR_ARG;
}

extern "C" B200AMP_API int b200amp_tune_get(const char *key, int *value)
{
    B200AMP_REQUIRE(key != nullptr && value != nullptr, "tune_get: null pointer");
    for (const Knob &k : KNOBS)
    {
        if (strcmp(k.key, key) == 0)
        {
            *value = tunables().*(k.field);
            return B200AMP_OK;
        }
    }
    set_error("tune_get: no knob named %s", key);
    return B200AMP_ERR_ARG;
}

extern "C" B200AMP_API long long b200amp_launch_count(void)
{
    return g_launches.load(std::memory_order_relaxed);
}

extern "C" B200AMP_API int b200amp_step_f16(float *master, float *m, float *v, const void *grads16, void *weights16, long long n,
                                const b200amp_tensor_info *tensors, int ntensors, b200amp_step_state *st,
                                void *workspace, const b200amp_schedule *cfg, b200amp_step_state *history,
                                int history_len, float beta1, float beta2, float eps, b200amp_stream s)
{
    int rc = b200amp_pass1_finalize_f16(grads16, n, st, workspace, cfg, history, history_len, s);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    return b200amp_pass2_f16(master, m, v, grads16, weights16, n, 0, tensors, ntensors, st, beta1, beta2, eps, s);
}

// ---------------------------------------------------------------- graphs

extern "C" B200AMP_API int b200amp_graph_begin_capture(b200amp_stream s)
{
    // thread-local mode: other host threads may keep calling the CUDA API while this one captures
    B200AMP_CUDA(cudaStreamBeginCapture(as_stream(s), cudaStreamCaptureModeThreadLocal));
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_graph_end_capture(b200amp_stream s, b200amp_graph **out)
{
    B200AMP_REQUIRE(out != nullptr, "graph_end_capture: out is null");
    *out = nullptr;
    cudaGraph_t graph = nullptr;
    B200AMP_CUDA(cudaStreamEndCapture(as_stream(s), &graph));
    cudaGraphExec_t exec = nullptr;
    cudaError_t err = cudaGraphInstantiateWithFlags(&exec, graph, 0);
    cudaGraphDestroy(graph);                    // the instantiated copy is all a replay needs
    if (err != cudaSuccess)
    {
        return cuda_fail(err, "cudaGraphInstantiateWithFlags", __FILE__, __LINE__);
    }
    b200amp_graph *g = new (std::nothrow) b200amp_graph;
    if (g == nullptr)
    {
        cudaGraphExecDestroy(exec);
        set_error("graph_end_capture: out of host memory");
        return B200AMP_ERR_CUDA;
    }
    g->exec = exec;
    *out = g;
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_graph_launch(b200amp_graph *g, b200amp_stream s)
{
    B200AMP_REQUIRE(g != nullptr && g->exec != nullptr, "graph_launch: no captured graph");
    B200AMP_CUDA(cudaGraphLaunch(g->exec, as_stream(s)));
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_graph_destroy(b200amp_graph *g)
{
    if (g == nullptr)
    {
        return B200AMP_OK;
    }
    cudaError_t err = g->exec != nullptr ? cudaGraphExecDestroy(g->exec) : cudaSuccess;
    delete g;
    if (err != cudaSuccess)
    {
        return cuda_fail(err, "cudaGraphExecDestroy", __FILE__, __LINE__);
    }
    return B200AMP_OK;
}
