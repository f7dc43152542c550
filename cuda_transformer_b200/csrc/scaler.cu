// scaler.cu: everything of the step that comes before AdamW: the unscale, the
// inf/NaN flag, the global gradient norm, and the finalize that turns them into
// this step's clip coefficient, learning rate, skip decision and next loss scale,
// all on the device with no host sync.
//
// Semantics follow cuda/kernels/scaler.cu of the reference (file:line cited at each
// piece). What is different is the shape of the work:
//   * native pass 1 reads an fp16 gradient arena (2 B/param), never writes it, and
//     runs a persistent grid over a FIXED virtual partition of the arena, so the
//     sum comes out bit-identical whatever the launch shape;
//   * the last block to finish runs the finalize, so no separate 1-block launch
//     sits between the two passes;
//   * the compat entry points keep the reference's arguments (fp32 gradients
//     unscaled in place, partial[512]) and its summation order.

#include <climits>
#include <cmath>
#include <mutex>

#include "finalize.cuh"
#include "pass1_common.cuh"

namespace b200amp
{

// ---------------------------------------------------------------- compat kernels

__global__ void begin_step_kernel(b200amp_step_state *st)
{
    st->found_inf = 0;
    st->inv_scale = 1.0f / st->loss_scale;
}

constexpr int COMPAT_THREADS = 256;
constexpr int COMPAT_UNROLL = 4;

// Same partition and the same order of additions as cuda/kernels/scaler.cu:39-66
// (512 x 256 threads, quad i belongs to thread i mod 131072, squares added quad after
// quad in fp32, butterfly over the warp, 8 warp sums through shared memory, butterfly
// again), so partial[] carries the reference's bits. The loads of COMPAT_UNROLL quads are
// issued together; the additions stay in order.
__global__ void __launch_bounds__(COMPAT_THREADS)
    unscale_norm_f32_kernel(float4 *g4, long long n4, b200amp_step_state *st, float *partial)
{
    __shared__ float warp_part[32];
    const float inv = st->inv_scale;
    const long long stride = static_cast<long long>(gridDim.x) * COMPAT_THREADS;
    float sum = 0.0f;
    bool bad = false;
    long long i = static_cast<long long>(blockIdx.x) * COMPAT_THREADS + threadIdx.x;
    for (; i + (COMPAT_UNROLL - 1) * stride < n4; i += COMPAT_UNROLL * stride)
    {
        float4 q[COMPAT_UNROLL];
#pragma unroll
        for (int u = 0; u < COMPAT_UNROLL; u++)
        {
            q[u] = g4[i + u * stride];
        }
#pragma unroll
        for (int u = 0; u < COMPAT_UNROLL; u++)
        {
            float4 g = q[u];
            g.x *= inv;
            g.y *= inv;
            g.z *= inv;
            g.w *= inv;
            g4[i + u * stride] = g;
            bad = bad || !isfinite(g.x) || !isfinite(g.y) || !isfinite(g.z) || !isfinite(g.w);
            sum += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
        }
    }
    for (; i < n4; i += stride)
    {
        float4 g = g4[i];
        g.x *= inv;
        g.y *= inv;
        g.z *= inv;
        g.w *= inv;
        g4[i] = g;
        bad = bad || !isfinite(g.x) || !isfinite(g.y) || !isfinite(g.z) || !isfinite(g.w);
        sum += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
    }
    if (bad)
    {
        st->found_inf = 1;                  // every writer stores the same value
    }
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    sum = warp_sum_f32(sum);
    if (lane == 0)
    {
        warp_part[warp] = sum;
    }
    __syncthreads();
    float total = lane < COMPAT_THREADS / 32 ? warp_part[lane] : 0.0f;
    total = warp_sum_f32(total);
    if (threadIdx.x == 0)
    {
        partial[blockIdx.x] = total;
    }
}

// 512 partials -> double, halving tree in shared memory (the fixed order of
// cuda/kernels/scaler.cu:118-129), then the finalize on thread 0.
__global__ void __launch_bounds__(B200AMP_NORM_BLOCKS)
    finalize_partials_kernel(b200amp_step_state *st, const float *partial, b200amp_schedule cfg,
                             b200amp_step_state *history, int history_len)
{
    __shared__ double tree[B200AMP_NORM_BLOCKS];
    const int tid = threadIdx.x;
    tree[tid] = static_cast<double>(partial[tid]);
    __syncthreads();
    for (int half = B200AMP_NORM_BLOCKS / 2; half > 0; half >>= 1)
    {
        if (tid < half)
        {
            tree[tid] += tree[tid + half];
        }
        __syncthreads();
    }
    if (tid == 0)
    {
        finalize_state(st, tree[0], 0, cfg, history, history_len, false);
    }
}

__global__ void lr_probe_kernel(double *out, int step, b200amp_schedule cfg)
{
    *out = schedule_lr(step, cfg);
}

// ---------------------------------------------------------------- native pass 1

// (partition, workspace layout and the 8-value accumulation: pass1_common.cuh)
#ifndef B200AMP_P1_LOAD_HINT
#define B200AMP_P1_LOAD_HINT 1
#endif

// FINALIZE: the last block also runs finalize_state (one GPU holds the whole arena).
// Otherwise it only publishes {sum, flag} in the workspace (a shard of a larger arena).
template <bool FINALIZE>
__global__ void __launch_bounds__(P1_THREADS)
    pass1_f16_kernel(const uint4 *__restrict__ g8, long long n8, b200amp_step_state *st, Workspace *ws,
                     b200amp_schedule cfg, b200amp_step_state *history, int history_len)
{
    __shared__ double warp_part[P1_WARPS];
    __shared__ int last_block;

    const float inv = 1.0f / st->loss_scale;
    const P1Partition part = p1_partition(n8);
    uint32_t bad = 0;

    for (int vb = blockIdx.x; vb < part.vblocks; vb += gridDim.x)
    {
        const long long begin = static_cast<long long>(vb) * part.vec_per_vblock;
        long long end = begin + part.vec_per_vblock;
        if (end > n8)
        {
            end = n8;
        }
        float acc[P1_UNROLL];
#pragma unroll
        for (int u = 0; u < P1_UNROLL; u++)
        {
            acc[u] = 0.0f;
        }
        long long i = begin + threadIdx.x;
        // full trips: P1_UNROLL loads in flight per thread
        for (; i + (P1_UNROLL - 1) * P1_THREADS < end; i += P1_UNROLL * P1_THREADS)
        {
            uint4 w[P1_UNROLL];
#pragma unroll
            for (int u = 0; u < P1_UNROLL; u++)
            {
                w[u] = load_h8<B200AMP_P1_LOAD_HINT>(g8 + i + u * P1_THREADS);
            }
#pragma unroll
            for (int u = 0; u < P1_UNROLL; u++)
            {
                accumulate_h8(w[u], inv, acc[u], bad);
            }
        }
        // the arena's ragged end: same slot -> same accumulator as a full trip would use
#pragma unroll
        for (int u = 0; u < P1_UNROLL; u++)
        {
            if (i + u * P1_THREADS < end)
            {
                uint4 w = load_h8<B200AMP_P1_LOAD_HINT>(g8 + i + u * P1_THREADS);
                accumulate_h8(w, inv, acc[u], bad);
            }
        }
        const float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        vblock_store_partial(mine, warp_part, ws, vb);
    }

    if (!pass1_take_ticket(bad, ws, &last_block))
    {
        return;
    }
    __shared__ double tree[P1_THREADS];
    int any_bad = 0;
    const double total = pass1_final_sum(part, ws, tree, &any_bad);
    if (FINALIZE && threadIdx.x == 0)
    {
        finalize_state(st, total, any_bad, cfg, history, history_len, true);
    }
}

// Pairs {sum, flag} of every rank, added in rank order.
__global__ void finalize_sums_kernel(b200amp_step_state *st, const double *sums, int nranks, b200amp_schedule cfg,
                                     b200amp_step_state *history, int history_len)
{
    double total = 0.0;
    int bad = 0;
    for (int r = 0; r < nranks; r++)
    {
        total += sums[2 * r];
        bad |= (sums[2 * r + 1] != 0.0) ? 1 : 0;
    }
    finalize_state(st, total, bad, cfg, history, history_len, true);
}

static int check_schedule(const b200amp_schedule *cfg, const b200amp_step_state *history, int history_len)
{
    B200AMP_REQUIRE(cfg != nullptr, "schedule is null");
    B200AMP_REQUIRE(history == nullptr || history_len > 0, "history given with history_len %d", history_len);
    return B200AMP_OK;
}

int launch_pass1(const void *grads16, long long n, b200amp_step_state *st, void *workspace, bool finalize,
                 const b200amp_schedule *cfg, b200amp_step_state *history, int history_len, cudaStream_t s)
{
    B200AMP_REQUIRE(grads16 != nullptr && st != nullptr && workspace != nullptr, "pass 1: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass 1: n = %lld must be a positive multiple of 8", n);
    B200AMP_REQUIRE(aligned(grads16, 16), "pass 1: the fp16 gradient pointer must be 16-byte aligned");
    B200AMP_REQUIRE(aligned(workspace, 16), "pass 1: the workspace must be 16-byte aligned");
    const long long n8 = n / 8;
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const P1Partition part = p1_partition(n8);
    int grid = sms * tunables().pass1_blocks_per_sm;
    if (grid > part.vblocks)
    {
        grid = part.vblocks;
    }
    b200amp_schedule c = {};
    if (finalize)
    {
        int rc = check_schedule(cfg, history, history_len);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
        c = *cfg;
        pass1_f16_kernel<true><<<grid, P1_THREADS, 0, s>>>(static_cast<const uint4 *>(grads16), n8, st,
                                                           static_cast<Workspace *>(workspace), c, history,
                                                           history_len);
    }
    else
    {
        pass1_f16_kernel<false><<<grid, P1_THREADS, 0, s>>>(static_cast<const uint4 *>(grads16), n8, st,
                                                            static_cast<Workspace *>(workspace), c, nullptr, 0);
    }
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

} // namespace b200amp

using namespace b200amp;

// ---------------------------------------------------------------- C ABI

extern "C" B200AMP_API int b200amp_initial_state(float scale, b200amp_step_state *out)
{
    B200AMP_REQUIRE(out != nullptr, "initial_state: out is null");
    b200amp_step_state st = {};
    st.loss_scale = scale;
    st.inv_scale = 1.0f / scale;
    st.clip_coef = 1.0f;
    st.decay = 1.0f;
    *out = st;
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_begin_step(b200amp_step_state *st, b200amp_stream s)
{
    B200AMP_REQUIRE(st != nullptr, "begin_step: state is null");
    begin_step_kernel<<<1, 1, 0, as_stream(s)>>>(st);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_unscale_and_norm_f32(float *grads, long long n, b200amp_step_state *st, float *partial,
                                            b200amp_stream s)
{
    B200AMP_REQUIRE(grads != nullptr && st != nullptr && partial != nullptr, "unscale_and_norm: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 4 == 0, "unscale_and_norm: n = %lld must be a positive multiple of 4", n);
    B200AMP_REQUIRE(aligned(grads, 16), "unscale_and_norm: grads must be 16-byte aligned");
    unscale_norm_f32_kernel<<<B200AMP_NORM_BLOCKS, COMPAT_THREADS, 0, as_stream(s)>>>(
        reinterpret_cast<float4 *>(grads), n / 4, st, partial);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_finalize_step(b200amp_step_state *st, const float *partial, const b200amp_schedule *cfg,
                                     b200amp_step_state *history, int history_len, b200amp_stream s)
{
    B200AMP_REQUIRE(st != nullptr && partial != nullptr, "finalize_step: null pointer");
    int rc = check_schedule(cfg, history, history_len);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    finalize_partials_kernel<<<1, B200AMP_NORM_BLOCKS, 0, as_stream(s)>>>(st, partial, *cfg, history, history_len);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_lr_on_gpu(int step, const b200amp_schedule *cfg, double *out)
{
    B200AMP_REQUIRE(cfg != nullptr && out != nullptr, "lr_on_gpu: null pointer");
    double *d = nullptr;
    B200AMP_CUDA(cudaMalloc(&d, sizeof(double)));
    lr_probe_kernel<<<1, 1>>>(d, step, *cfg);
    count_launch();
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess)
    {
        err = cudaMemcpy(out, d, sizeof(double), cudaMemcpyDeviceToHost);
    }
    cudaFree(d);
    if (err != cudaSuccess)
    {
        return cuda_fail(err, "lr_on_gpu", __FILE__, __LINE__);
    }
    return B200AMP_OK;
}

extern "C" B200AMP_API size_t b200amp_workspace_bytes(void)
{
    return sizeof(Workspace);
}

extern "C" B200AMP_API int b200amp_workspace_init(void *workspace, b200amp_stream s)
{
    B200AMP_REQUIRE(workspace != nullptr, "workspace_init: null pointer");
    B200AMP_CUDA(cudaMemsetAsync(workspace, 0, sizeof(Workspace), as_stream(s)));
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_pass1_f16(const void *grads16, long long n, const b200amp_step_state *st, void *workspace,
                                 b200amp_stream s)
{
    return launch_pass1(grads16, n, const_cast<b200amp_step_state *>(st), workspace, false, nullptr, nullptr, 0,
                        as_stream(s));
}

extern "C" B200AMP_API int b200amp_pass1_finalize_f16(const void *grads16, long long n, b200amp_step_state *st, void *workspace,
                                          const b200amp_schedule *cfg, b200amp_step_state *history, int history_len,
                                          b200amp_stream s)
{
    return launch_pass1(grads16, n, st, workspace, true, cfg, history, history_len, as_stream(s));
}

extern "C" B200AMP_API int b200amp_finalize_sums(b200amp_step_state *st, const double *sums, int nranks,
                                     const b200amp_schedule *cfg, b200amp_step_state *history, int history_len,
                                     b200amp_stream s)
{
    B200AMP_REQUIRE(st != nullptr && sums != nullptr, "finalize_sums: null pointer");
    B200AMP_REQUIRE(nranks > 0, "finalize_sums: nranks = %d", nranks);
    int rc = check_schedule(cfg, history, history_len);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    finalize_sums_kernel<<<1, 1, 0, as_stream(s)>>>(st, sums, nranks, *cfg, history, history_len);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

// ---------------------------------------------------------------- pass 1 without a caller-supplied workspace
//
// For callers that cannot hand the library any device memory beyond the arrays the step itself
// reads and writes, and cannot allocate more: a trainer that gave all of the device's memory to
// its own arenas when it started (the reference's FastGPT allocates everything in its
// constructor and nothing afterwards), a plugin running inside another framework's memory
// pool, or a step loop where cudaMalloc's implicit device-wide synchronisation is not
// acceptable. The scratch that pass 1 needs (one fp64 partial per virtual block, the ticket, the
// flag word) lives in the library image instead: every GPU that loads the library holds these
// 37,920 bytes until the process exits.

namespace b200amp
{

// A limit of this entry point by policy, not one the array imposes: the 4,736 partial sums cover
// any n (the virtual blocks just grow), but a stated maximum is part of this entry point's contract.
constexpr long long STATIC_PASS1_MAX_ELEMENTS = 1LL << 32;     // 4,294,967,296 fp16 gradients (8 GiB)

static __device__ __align__(256) unsigned char g_pass1_scratch[sizeof(Workspace)];

// The device address of g_pass1_scratch on the current device. In host code the array's name
// is only a handle for the runtime, not a pointer a kernel could use, so the address is asked
// for once per device (with that device current) and kept.
static int pass1_scratch_address(Workspace **out)
{
    constexpr int MAX_DEVICES = 64;
    static Workspace *known[MAX_DEVICES] = {};
    static std::mutex guard;
    int dev = -1;
    B200AMP_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES)
    {
        set_error("pass1_f16_static: device index %d out of range", dev);
        return B200AMP_ERR_ARG;
    }
    std::lock_guard<std::mutex> hold(guard);
    if (known[dev] == nullptr)
    {
        void *address = nullptr;
        B200AMP_CUDA(cudaGetSymbolAddress(&address, g_pass1_scratch));
        known[dev] = static_cast<Workspace *>(address);
    }
    *out = known[dev];
    return B200AMP_OK;
}

} // namespace b200amp

extern "C" B200AMP_API int b200amp_pass1_f16_static(const void *grads16, long long n, const b200amp_step_state *st,
                                                    double *sums_out, b200amp_stream s)
{
    // every argument is checked before anything is enqueued: a refused call leaves the shared
    // array and the stream untouched
    B200AMP_REQUIRE(sums_out != nullptr, "pass1_f16_static: sums_out is null");
    B200AMP_REQUIRE(aligned(sums_out, 8), "pass1_f16_static: sums_out must be 8-byte aligned");
    B200AMP_REQUIRE(grads16 != nullptr && st != nullptr, "pass1_f16_static: null pointer");
    B200AMP_REQUIRE(aligned(grads16, 16), "pass1_f16_static: the fp16 gradient pointer must be 16-byte aligned");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass1_f16_static: n = %lld must be a positive multiple of 8", n);
    if (n > STATIC_PASS1_MAX_ELEMENTS)
    {
        set_error("pass1_f16_static: n = %lld is beyond the %lld elements this entry point accepts; "
                  "use b200amp_pass1_f16 with a workspace of your own",
                  n, STATIC_PASS1_MAX_ELEMENTS);
        return B200AMP_ERR_LIMIT;
    }
    Workspace *scratch = nullptr;
    int rc = pass1_scratch_address(&scratch);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    cudaStream_t stream = as_stream(s);
    // The array keeps whatever the last call left. The kernel resets its ticket and flag itself
    // when it finishes; clearing them here too makes a call independent of how the last one ended.
    B200AMP_CUDA(cudaMemsetAsync(&scratch->ticket, 0, sizeof(scratch->ticket) + sizeof(scratch->bad), stream));
    rc = launch_pass1(grads16, n, const_cast<b200amp_step_state *>(st), scratch, false, nullptr, nullptr, 0, stream);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_CUDA(cudaMemcpyAsync(sums_out, scratch->sums, 2 * sizeof(double), cudaMemcpyDeviceToDevice, stream));
    return B200AMP_OK;
}

// ---------------------------------------------------------------- gradient producer + pass 1
//
// The step before the path. The reference's backward pass accumulates loss-scaled parameter
// gradients into an fp32 arena and clears it with a memset every step
// (cuda/gpt_fast.cu:455, cuda/kernels/gemm_common.cuh:11). This kernel is the bridge from that
// arena to the fp16 arena the native step reads: one sweep rounds the fp32 gradients to fp16
// (round to nearest even; a value beyond the fp16 range becomes inf and skips the step, which
// is what loss scaling is for), takes pass 1's squared norm and inf/NaN flag on exactly the
// rounded values, and, if asked, leaves zeros behind in the fp32 arena so the memset goes away.
// 4 B read + 2 B written (+ 4 B written when clearing) per parameter; the step that follows is
// b200amp_finalize_sums + b200amp_pass2_f16 (28 B): 34-38 B/param against the reference's 42.

namespace b200amp
{

template <bool FINALIZE, bool CLEAR>
__global__ void __launch_bounds__(P1_THREADS)
    cast_pass1_f32_kernel(float *__restrict__ g32, uint4 *__restrict__ g16, long long n8, b200amp_step_state *st,
                          Workspace *ws, b200amp_schedule cfg, b200amp_step_state *history, int history_len)
{
    __shared__ double warp_part[P1_WARPS];
    __shared__ int last_block;

    const float inv = 1.0f / st->loss_scale;
    const P1Partition part = p1_partition(n8);
    uint32_t bad = 0;
    const Float8 zeros = {{0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f}};

    for (int vb = blockIdx.x; vb < part.vblocks; vb += gridDim.x)
    {
        const long long begin = static_cast<long long>(vb) * part.vec_per_vblock;
        long long end = begin + part.vec_per_vblock;
        if (end > n8)
        {
            end = n8;
        }
        float acc[P1_UNROLL];
#pragma unroll
        for (int u = 0; u < P1_UNROLL; u++)
        {
            acc[u] = 0.0f;
        }
        // the same slots and accumulators as pass1_f16_kernel, so the sum has the bits pass 1 alone
        // would give on the fp16 arena this kernel writes
        for (long long base = begin + threadIdx.x; base < end; base += P1_UNROLL * P1_THREADS)
        {
            Float8 w[P1_UNROLL];
#pragma unroll
            for (int u = 0; u < P1_UNROLL; u++)
            {
                const long long i = base + u * P1_THREADS;
                if (i < end)
                {
                    w[u] = load8<0>(g32 + i * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < P1_UNROLL; u++)
            {
                const long long i = base + u * P1_THREADS;
                if (i < end)
                {
                    uint4 h;
                    h.x = float2_to_half2_bits(w[u].v[0], w[u].v[1]);
                    h.y = float2_to_half2_bits(w[u].v[2], w[u].v[3]);
                    h.z = float2_to_half2_bits(w[u].v[4], w[u].v[5]);
                    h.w = float2_to_half2_bits(w[u].v[6], w[u].v[7]);
                    store_h8<0>(g16 + i, h);
                    if (CLEAR)
                    {
                        store8<1>(g32 + i * 8, zeros);
                    }
                    accumulate_h8(h, inv, acc[u], bad);
                }
            }
        }
        const float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        vblock_store_partial(mine, warp_part, ws, vb);
    }

    if (!pass1_take_ticket(bad, ws, &last_block))
    {
        return;
    }
    __shared__ double tree[P1_THREADS];
    int any_bad = 0;
    const double total = pass1_final_sum(part, ws, tree, &any_bad);
    if (FINALIZE && threadIdx.x == 0)
    {
        finalize_state(st, total, any_bad, cfg, history, history_len, true);
    }
}

} // namespace b200amp

extern "C" B200AMP_API int b200amp_cast_pass1_f32(float *grads32, void *grads16, long long n, int clear_source,
                                                  b200amp_step_state *st, void *workspace,
                                                  const b200amp_schedule *cfg, b200amp_step_state *history,
                                                  int history_len, b200amp_stream s)
{
    B200AMP_REQUIRE(grads32 != nullptr && grads16 != nullptr && st != nullptr && workspace != nullptr,
                    "cast_pass1: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "cast_pass1: n = %lld must be a positive multiple of 8", n);
    B200AMP_REQUIRE(aligned(grads32, 32) && aligned(grads16, 16) && aligned(workspace, 16),
                    "cast_pass1: grads32 must be 32-byte, grads16 and the workspace 16-byte aligned");
    const bool finalize = cfg != nullptr;
    b200amp_schedule c = {};
    if (finalize)
    {
        int rc = check_schedule(cfg, history, history_len);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
        c = *cfg;
    }
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const long long n8 = n / 8;
    const P1Partition part = p1_partition(n8);
    // measured at the 1.3 B arena: 16 CTAs per SM move 6.16 TB/s (clearing) / 6.55 TB/s, 4 (pass 1's
    // best) 5.86 / 6.37: with writes in the mix a finer spread of the virtual blocks pays
    int grid = sms * tunables().bridge_blocks_per_sm;
    if (grid > part.vblocks)
    {
        grid = part.vblocks;
    }
    uint4 *out = static_cast<uint4 *>(grads16);
    Workspace *ws = static_cast<Workspace *>(workspace);
    cudaStream_t stream = as_stream(s);
#define B200AMP_CAST(FIN, CLR)                                                                               \
    cast_pass1_f32_kernel<FIN, CLR><<<grid, P1_THREADS, 0, stream>>>(grads32, out, n8, st, ws, c, history, \
                                                                     history_len)
    if (finalize && clear_source)
    {
        B200AMP_CAST(true, true);
    }
    else if (finalize)
    {
        B200AMP_CAST(true, false);
    }
    else if (clear_source)
    {
        B200AMP_CAST(false, true);
    }
    else
    {
        B200AMP_CAST(false, false);
    }
#undef B200AMP_CAST
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}
