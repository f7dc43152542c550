// pass2.cu: pass 2 of the step on an fp16 gradient arena: unscale, clip, AdamW on the fp32
// master / m / v with decoupled weight decay and bias correction, and the fp16 weight
// cast, in one launch over the flat arena (or over one shard of it).
//
// Per element this is cuda/kernels/adamw_multi.cu:20-29,75-89 of the reference. The work
// is laid out for HBM3e: 28 bytes move per element and nothing else matters. Two kernels
// do the same arithmetic (same bits):
//
//   pass2_f16_kernel   registers only. A persistent grid strides over 8-element groups;
//                      every access is one 256-bit (fp32 arrays) or 128-bit (fp16 arrays)
//                      request, so a warp moves 1 KB / 512 B of contiguous memory per
//                      instruction. Measured on B200 at 1.3 B elements: 2 CTAs x 256 threads
//                      per SM and one group per thread per trip beat every other shape
//                      (more threads, 2 or 4 groups per trip, a contiguous range per CTA,
//                      register prefetch of the next trip: all 1-15 % slower).
//   pass2_bulk_kernel  shared-memory staging. One CTA per SM runs a ring of stages; one
//                      thread moves whole tiles (2048 elements: 4 KB of gradients, 8 KB each
//                      of master, m, v) with bulk asynchronous copies (cp.async.bulk, no
//                      multicast) completing on an mbarrier; all threads update the tile in
//                      place in shared memory; the tile leaves with bulk stores (the fp16
//                      weights overwrite the gradient slot, which has the same size). Many
//                      KB in flight per SM without many threads, and every request to DRAM
//                      is a long contiguous run.
//
// The decay flag comes from a cursor into the tensor table that advances as positions
// grow, instead of a binary search per vector (the search runs once per thread).

#include <mutex>

#include "adamw_math.cuh"

namespace b200amp
{

// ---------------------------------------------------------------- registers-only kernel

// The whole grid sweeps the arena together: group i of a sweep belongs to thread i mod
// (grid * THREADS). A thread's positions only grow, so it walks the tensor table once, and
// between two run boundaries its warp runs trips with no decay lookup at all (sweep_groups).
template <int THREADS, int ST>
__global__ void __launch_bounds__(THREADS)
    pass2_f16_kernel(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                     const uint4 *__restrict__ g16, uint4 *__restrict__ w16, long long n8, long long arena_offset,
                     const b200amp_tensor_info *__restrict__ tensors, int ntensors,
                     const b200amp_step_state *__restrict__ st, float b1, float b2, float eps)
{
    __shared__ TensorTable tab;
    const int nruns = table_load(tab, tensors, ntensors);
    if (st->found_inf)
    {
        return;                                 // skipped step: nothing moves
    }
    const float wd_decay = st->decay;
    const StepFactors f = step_factors(st, b1, b2, eps);

    // group indices fit 32 bits (the launcher refuses ranges beyond 2^31 - 2^23 groups): one
    // multiply-add makes each address, and the loop counter is a single register
    const int groups = static_cast<int>(n8);
    const int stride = static_cast<int>(gridDim.x) * THREADS;
    const int first = static_cast<int>(blockIdx.x) * THREADS + static_cast<int>(threadIdx.x);
    sweep_groups<ST>(master, m, v, g16, tab, nruns, arena_offset, groups, first, stride, wd_decay, f,
                     [&](int j, const uint4 &half8) {
                         if (w16 != nullptr)
                         {
                             store_h8<ST>(w16 + j, half8);
                         }
                     });
}

// The same sweep with the decay runs as a kernel parameter (b200amp_decay_runs, at most
// B200AMP_MAX_RUNS of them: a GPT layout has 8 per layer + 3). No static shared memory, no table
// prologue, no CTA barrier: a CTA starts loading with its first instruction.
template <int THREADS, int ST>
__global__ void __launch_bounds__(THREADS)
    pass2_f16_runs_kernel(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                          const uint4 *__restrict__ g16, uint4 *__restrict__ w16, long long n8,
                          long long arena_offset, const __grid_constant__ DecayRuns runs,
                          const b200amp_step_state *__restrict__ st, float b1, float b2, float eps)
{
    if (st->found_inf)
    {
        return;
    }
    const float wd_decay = st->decay;
    const StepFactors f = step_factors(st, b1, b2, eps);
    const int nruns = runs.nruns;
    const int groups = static_cast<int>(n8);
    const int stride = static_cast<int>(gridDim.x) * THREADS;
    const int first = static_cast<int>(blockIdx.x) * THREADS + static_cast<int>(threadIdx.x);
    sweep_groups<ST>(master, m, v, g16, runs, nruns, arena_offset, groups, first, stride, wd_decay, f,
                     [&](int j, const uint4 &half8) {
                         if (w16 != nullptr)
                         {
                             store_h8<ST>(w16 + j, half8);
                         }
                     });
}

// ---------------------------------------------------------------- shared-memory staged kernel

constexpr int BULK_TILE = 2048;                 // elements per tile
constexpr int BULK_THREADS = 512;               // one quad (4 elements) per thread per tile
constexpr int BULK_MAX_STAGES = 7;
constexpr unsigned BULK_WAIT_LIMIT = 1u << 20;  // polls of one barrier before the kernel gives up (a fraction of a second)

struct __align__(128) BulkStage
{
    float p[BULK_TILE];
    float m[BULK_TILE];
    float v[BULK_TILE];
    __half g[BULK_TILE];                        // gradients in, fp16 weights out
};
static_assert(sizeof(BulkStage) == 14 * BULK_TILE, "a stage holds 14 bytes per element (updated in place)");

// Set when a barrier wait ran out (a copy that never completed). Read by b200amp_device_error().
__device__ int g_bulk_timeout = 0;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" : : "r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" : : "r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity)
{
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}

// Bounded wait: true when the phase completed, false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity)
{
    for (unsigned tries = 0; tries < BULK_WAIT_LIMIT; tries++)
    {
        if (mbar_try_wait(bar, parity))
        {
            return true;
        }
        if (tries > 64)
        {
            __nanosleep(64);
        }
    }
    return false;
}

// global -> shared, completes `bytes` on the barrier. No multicast: the destination is this CTA's
// own shared memory (a CTA launched without a cluster is a cluster of one).
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :
                 : "r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// shared -> global, tracked by the thread's bulk async-group
__device__ __forceinline__ void bulk_store(void *dst_gmem, const void *src_smem, unsigned bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :
                 : "l"(dst_gmem), "r"(smem_u32(src_smem)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit()
{
    asm volatile("cp.async.bulk.commit_group;" : : : "memory");
}

template <int PENDING>
__device__ __forceinline__ void bulk_wait_read()        // at most PENDING store groups still reading shared memory
{
    asm volatile("cp.async.bulk.wait_group.read %0;" : : "n"(PENDING) : "memory");
}

__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" : : : "memory");
}

__device__ __forceinline__ void fence_async_proxy()     // generic-proxy writes to shared memory -> async proxy
{
    asm volatile("fence.proxy.async.shared::cta;" : : : "memory");
}

// Tile t of the range holds elements [t * BULK_TILE, min(n, (t + 1) * BULK_TILE)). CTA b owns tiles
// b, b + grid, b + 2 grid, ... Stage of the k-th owned tile: k mod stages.
__global__ void __launch_bounds__(BULK_THREADS, 1)
    pass2_bulk_kernel(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                      const __half *__restrict__ g16, __half *__restrict__ w16, long long n, long long arena_offset,
                      const b200amp_tensor_info *__restrict__ tensors, int ntensors,
                      const b200amp_step_state *__restrict__ st, float b1, float b2, float eps, int stages,
                      int starve)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    BulkStage *stage = reinterpret_cast<BulkStage *>(smem_raw);
    __shared__ TensorTable tab;
    __shared__ uint64_t full[BULK_MAX_STAGES];
    __shared__ int gave_up;

    const int nruns = table_load(tab, tensors, ntensors);
    if (st->found_inf)
    {
        return;                                 // skipped step: nothing moves
    }
    const float coef = st->clip_coef;
    const float step_size = st->step_size;
    const float bc2_sqrt = st->bc2_sqrt;
    const float wd_decay = st->decay;
    const float inv = st->inv_scale;
    const float w1 = 1.0f - b1;
    const float w2 = 1.0f - b2;

    const long long ntiles = (n + BULK_TILE - 1) / BULK_TILE;
    const long long first_tile = blockIdx.x;
    if (first_tile >= ntiles)
    {
        return;
    }
    const long long my_tiles = (ntiles - first_tile + gridDim.x - 1) / gridDim.x;
    const int lookahead = stages - 2;           // loads in flight; one stage computes, one drains its stores

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < stages; s++)
        {
            mbar_init(&full[s], 1);
        }
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" : : : "memory");
    }
    __syncthreads();

    auto tile_elems = [&](long long k) -> unsigned
    {
        const long long begin = (first_tile + k * gridDim.x) * BULK_TILE;
        const long long left = n - begin;
        return static_cast<unsigned>(left < BULK_TILE ? left : BULK_TILE);
    };
    auto issue_load = [&](long long k)
    {
        const long long begin = (first_tile + k * gridDim.x) * BULK_TILE;
        const unsigned cnt = tile_elems(k);
        BulkStage &sg = stage[k % stages];
        uint64_t *bar = &full[k % stages];
        // starve (test hook): CTA 0 announces 16 bytes that never come for its second tile, so that
        // barrier's wait runs into its limit and the give-up path below is exercised
        const unsigned never = (starve != 0 && blockIdx.x == 0 && k == 1) ? 16u : 0u;
        mbar_expect_tx(bar, cnt * 14u + never);
        bulk_load(sg.g, g16 + begin, cnt * 2u, bar);
        bulk_load(sg.p, master + begin, cnt * 4u, bar);
        bulk_load(sg.m, m + begin, cnt * 4u, bar);
        bulk_load(sg.v, v + begin, cnt * 4u, bar);
    };

    if (threadIdx.x == 0)
    {
        for (long long k = 0; k < lookahead && k < my_tiles; k++)
        {
            issue_load(k);
        }
    }

    Cursor cur = cursor_seek(tab, nruns, arena_offset + first_tile * BULK_TILE, wd_decay);
    long long done = 0;                         // tiles whose barrier this thread has passed
    for (long long k = 0; k < my_tiles; k++)
    {
        if (threadIdx.x == 0 && k + lookahead < my_tiles)
        {
            // the stage about to be refilled held tile k + lookahead - stages = k - 2: its stores
            // were committed two trips ago; all but the latest store group must be done reading
            bulk_wait_read<1>();
            issue_load(k + lookahead);
        }
        BulkStage &sg = stage[k % stages];
        const unsigned parity = static_cast<unsigned>((k / stages) & 1);
        if (!mbar_wait(&full[k % stages], parity))
        {
            gave_up = 1;                        // every thread that timed out stores the same value
        }
        __syncthreads();
        if (gave_up)
        {
            break;
        }
        done = k + 1;

        const long long tile_begin = (first_tile + k * gridDim.x) * BULK_TILE;
        const unsigned cnt = tile_elems(k);
        const long long at0 = arena_offset + tile_begin;
        cursor_advance(cur, tab, nruns, at0, wd_decay);
        const bool uniform = at0 + cnt <= cur.next;
        const float d_tile = cur.factor;

        const unsigned q = threadIdx.x;         // quad of this thread: BULK_TILE / 4 == BULK_THREADS
        if (q * 4 < cnt)
        {
            float d = d_tile;
            if (!uniform)
            {
                Cursor c2 = cur;
                cursor_advance(c2, tab, nruns, at0 + q * 4, wd_decay);
                d = c2.factor;
            }
            float4 p4 = reinterpret_cast<float4 *>(sg.p)[q];
            float4 m4 = reinterpret_cast<float4 *>(sg.m)[q];
            float4 v4 = reinterpret_cast<float4 *>(sg.v)[q];
            const uint2 gq = reinterpret_cast<const uint2 *>(sg.g)[q];
            const float2 g01 = half2_bits_to_float2(gq.x);
            const float2 g23 = half2_bits_to_float2(gq.y);
            adamw_element(p4.x, m4.x, v4.x, (g01.x * inv) * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
            adamw_element(p4.y, m4.y, v4.y, (g01.y * inv) * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
            adamw_element(p4.z, m4.z, v4.z, (g23.x * inv) * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
            adamw_element(p4.w, m4.w, v4.w, (g23.y * inv) * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
            reinterpret_cast<float4 *>(sg.p)[q] = p4;
            reinterpret_cast<float4 *>(sg.m)[q] = m4;
            reinterpret_cast<float4 *>(sg.v)[q] = v4;
            uint2 wq;
            wq.x = float2_to_half2_bits(p4.x, p4.y);
            wq.y = float2_to_half2_bits(p4.z, p4.w);
            reinterpret_cast<uint2 *>(sg.g)[q] = wq;
        }
        fence_async_proxy();
        __syncthreads();
        if (threadIdx.x == 0)
        {
            bulk_store(master + tile_begin, sg.p, cnt * 4u);
            bulk_store(m + tile_begin, sg.m, cnt * 4u);
            bulk_store(v + tile_begin, sg.v, cnt * 4u);
            if (w16 != nullptr)
            {
                bulk_store(w16 + tile_begin, sg.g, cnt * 2u);
            }
            bulk_commit();
        }
    }

    if (threadIdx.x == 0)
    {
        bulk_wait_all();                        // stores of this thread: complete before the CTA leaves
        if (gave_up)
        {
            g_bulk_timeout = 1;
            // loads already issued still target this CTA's shared memory: give each one more bounded
            // wait before the memory is handed back
            // tiles 0 .. done + lookahead have been requested (the trip that gave up had already
            // asked for its look-ahead tile)
            long long issued = done + lookahead + 1 < my_tiles ? done + lookahead + 1 : my_tiles;
            for (long long k = done; k < issued; k++)
            {
                mbar_wait(&full[k % stages], static_cast<unsigned>((k / stages) & 1));
            }
        }
    }
}

// ---------------------------------------------------------------- launch

template <int THREADS>
static void launch_registers(int st_hint, int grid, cudaStream_t s, float *master, float *m, float *v,
                             const uint4 *g16, uint4 *w16, long long n8, long long arena_offset,
                             const b200amp_tensor_info *tensors, int ntensors, const b200amp_step_state *st, float b1,
                             float b2, float eps)
{
    if (st_hint == 1)
    {
        pass2_f16_kernel<THREADS, 1><<<grid, THREADS, 0, s>>>(master, m, v, g16, w16, n8, arena_offset, tensors,
                                                              ntensors, st, b1, b2, eps);
    }
    else
    {
        pass2_f16_kernel<THREADS, 0><<<grid, THREADS, 0, s>>>(master, m, v, g16, w16, n8, arena_offset, tensors,
                                                              ntensors, st, b1, b2, eps);
    }
}

static int bulk_smem_bytes(int stages)
{
    return stages * static_cast<int>(sizeof(BulkStage));
}

static int prepare_bulk(int stages)
{
    // opt in to more than 48 KB of dynamic shared memory, once per device and stage count
    constexpr int MAX_DEVICES = 64;
    static int prepared[MAX_DEVICES] = {};
    static std::mutex guard;
    std::lock_guard<std::mutex> hold(guard);
    int dev = 0;
    B200AMP_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES)
    {
        set_error("device index %d out of range", dev);
        return B200AMP_ERR_ARG;
    }
    if (prepared[dev] != stages)
    {
        B200AMP_CUDA(cudaFuncSetAttribute(pass2_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          bulk_smem_bytes(stages)));
        prepared[dev] = stages;
    }
    return B200AMP_OK;
}

} // namespace b200amp

using namespace b200amp;

extern "C" B200AMP_API int b200amp_pass2_f16(float *master, float *m, float *v, const void *grads16, void *weights16,
                                             long long n, long long arena_offset, const b200amp_tensor_info *tensors,
                                             int ntensors, const b200amp_step_state *st, float beta1, float beta2,
                                             float eps, b200amp_stream s)
{
    B200AMP_REQUIRE(master != nullptr && m != nullptr && v != nullptr && grads16 != nullptr && st != nullptr,
                    "pass 2: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass 2: n = %lld must be a positive multiple of 8", n);
    if (n / 8 > (1LL << 31) - (1LL << 23))      // the largest grid strides by 148 * 32 * 1024 < 2^23 groups
    {
        set_error("pass 2: n = %lld is beyond the 17,112,760,320 elements one launch addresses; split the range", n);
        return B200AMP_ERR_LIMIT;
    }
    B200AMP_REQUIRE(arena_offset >= 0 && arena_offset % 4 == 0, "pass 2: arena_offset = %lld must be a multiple of 4",
                    arena_offset);
    B200AMP_REQUIRE(aligned(master, 32) && aligned(m, 32) && aligned(v, 32),
                    "pass 2: master, m and v must be 32-byte aligned");
    B200AMP_REQUIRE(aligned(grads16, 16) && aligned(weights16, 16),
                    "pass 2: the fp16 arenas must be 16-byte aligned");
    B200AMP_REQUIRE(tensors != nullptr, "pass 2: tensor table is null");
    B200AMP_REQUIRE(ntensors > 0 && ntensors <= B200AMP_MAX_TENSORS, "pass 2: ntensors = %d, must be in 1..%d",
                    ntensors, B200AMP_MAX_TENSORS);
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const Tunables &t = tunables();
    cudaStream_t stream = as_stream(s);

    if (t.pass2_variant == 1)
    {
        const int stages = t.pass2_stages;
        int rc = prepare_bulk(stages);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
        const long long ntiles = (n + BULK_TILE - 1) / BULK_TILE;
        int grid = sms;
        if (grid > ntiles)
        {
            grid = static_cast<int>(ntiles);
        }
        pass2_bulk_kernel<<<grid, BULK_THREADS, bulk_smem_bytes(stages), stream>>>(
            master, m, v, static_cast<const __half *>(grads16), static_cast<__half *>(weights16), n, arena_offset,
            tensors, ntensors, st, beta1, beta2, eps, stages, t.pass2_test_starve);
        B200AMP_LAUNCHED();
        return B200AMP_OK;
    }

    const long long n8 = n / 8;
    const int threads = t.pass2_threads >= 1024 ? 1024 : (t.pass2_threads >= 512 ? 512 : 256);
    long long want = (n8 + threads - 1) / threads;
    int grid = sms * t.pass2_blocks_per_sm;
    if (grid > want)
    {
        grid = static_cast<int>(want);
    }
    const uint4 *g16 = static_cast<const uint4 *>(grads16);
    uint4 *w16 = static_cast<uint4 *>(weights16);
    if (threads >= 1024)
    {
        launch_registers<1024>(t.pass2_store_hint, grid, stream, master, m, v, g16, w16, n8, arena_offset, tensors,
                               ntensors, st, beta1, beta2, eps);
    }
    else if (threads >= 512)
    {
        launch_registers<512>(t.pass2_store_hint, grid, stream, master, m, v, g16, w16, n8, arena_offset, tensors,
                              ntensors, st, beta1, beta2, eps);
    }
    else
    {
        launch_registers<256>(t.pass2_store_hint, grid, stream, master, m, v, g16, w16, n8, arena_offset, tensors,
                              ntensors, st, beta1, beta2, eps);
    }
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

// The tensor table as runs of equal decay flag, for b200amp_pass2_f16_runs. Host only.
extern "C" B200AMP_API int b200amp_decay_runs_build(const b200amp_tensor_info *host_table, int ntensors,
                                                    b200amp_decay_runs *out)
{
    B200AMP_REQUIRE(out != nullptr, "decay_runs_build: out is null");
    int rc = b200amp_check_tensor_table(host_table, ntensors, 0);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    b200amp_decay_runs runs = {};
    for (int k = 0; k < ntensors; k++)
    {
        const int flag = host_table[k].decay ? 1 : 0;
        if (k > 0 && (host_table[k - 1].decay ? 1 : 0) == flag)
        {
            continue;
        }
        if (runs.nruns == B200AMP_MAX_RUNS)
        {
            set_error("decay_runs_build: more than %d runs of equal decay flag; use b200amp_pass2_f16 with the "
                      "table in device memory",
                      B200AMP_MAX_RUNS);
            return B200AMP_ERR_LIMIT;
        }
        if (host_table[k].offset / 4 > 0xFFFFFFFFLL)
        {
            set_error("decay_runs_build: entry %d starts at %lld, beyond the 17,179,869,180 elements a run can "
                      "start at",
                      k, host_table[k].offset);
            return B200AMP_ERR_LIMIT;
        }
        if (runs.nruns == 0)
        {
            runs.flag0 = flag;
        }
        runs.first4[runs.nruns++] = static_cast<unsigned int>(host_table[k].offset / 4);
    }
    *out = runs;
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_pass2_f16_runs(float *master, float *m, float *v, const void *grads16,
                                                  void *weights16, long long n, long long arena_offset,
                                                  const b200amp_decay_runs *runs, const b200amp_step_state *st,
                                                  float beta1, float beta2, float eps, b200amp_stream s)
{
    B200AMP_REQUIRE(master != nullptr && m != nullptr && v != nullptr && grads16 != nullptr && st != nullptr &&
                        runs != nullptr,
                    "pass 2 (runs): null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass 2 (runs): n = %lld must be a positive multiple of 8", n);
    if (n / 8 > (1LL << 31) - (1LL << 23))
    {
        set_error("pass 2 (runs): n = %lld is beyond the 17,112,760,320 elements one launch addresses; split the "
                  "range",
                  n);
        return B200AMP_ERR_LIMIT;
    }
    B200AMP_REQUIRE(arena_offset >= 0 && arena_offset % 4 == 0,
                    "pass 2 (runs): arena_offset = %lld must be a multiple of 4", arena_offset);
    B200AMP_REQUIRE(aligned(master, 32) && aligned(m, 32) && aligned(v, 32),
                    "pass 2 (runs): master, m and v must be 32-byte aligned");
    B200AMP_REQUIRE(aligned(grads16, 16) && aligned(weights16, 16),
                    "pass 2 (runs): the fp16 arenas must be 16-byte aligned");
    B200AMP_REQUIRE(runs->nruns > 0 && runs->nruns <= B200AMP_MAX_RUNS, "pass 2 (runs): nruns = %d, must be in 1..%d",
                    runs->nruns, B200AMP_MAX_RUNS);
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const Tunables &t = tunables();
    const long long n8 = n / 8;
    long long want = (n8 + 255) / 256;
    int grid = sms * t.pass2_blocks_per_sm;
    if (grid > want)
    {
        grid = static_cast<int>(want);
    }
    const uint4 *g16 = static_cast<const uint4 *>(grads16);
    uint4 *w16 = static_cast<uint4 *>(weights16);
    if (t.pass2_store_hint == 1)
    {
        pass2_f16_runs_kernel<256, 1><<<grid, 256, 0, as_stream(s)>>>(master, m, v, g16, w16, n8, arena_offset, *runs,
                                                                      st, beta1, beta2, eps);
    }
    else
    {
        pass2_f16_runs_kernel<256, 0><<<grid, 256, 0, as_stream(s)>>>(master, m, v, g16, w16, n8, arena_offset, *runs,
                                                                      st, beta1, beta2, eps);
    }
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

// What gave up a bounded wait on the current device since the last call, as a bit mask (the flags
// are cleared by reading them): 1 = a shared-memory staged launch waiting for a bulk copy,
// 2 = a ZeRO-1 kernel waiting for another rank. Synchronises the device.
extern "C" B200AMP_API int b200amp_device_error(int *out)
{
    B200AMP_REQUIRE(out != nullptr, "device_error: out is null");
    int flag = 0;
    B200AMP_CUDA(cudaMemcpyFromSymbol(&flag, g_bulk_timeout, sizeof(int)));
    if (flag != 0)
    {
        const int zero = 0;
        B200AMP_CUDA(cudaMemcpyToSymbol(g_bulk_timeout, &zero, sizeof(int)));
    }
    int rank_wait = 0;
    int rc = zero1_sync_timeout_take(&rank_wait);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    *out = (flag != 0 ? 1 : 0) | (rank_wait != 0 ? 2 : 0);
    return B200AMP_OK;
}
