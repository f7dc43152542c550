// peer_bandwidth.cu: what bounds a kernel that reads or writes another GPU's memory over NVLink.
// It prints the bandwidth per direction of a 1 GiB copy between
// GPU 0 and GPU 1 for each way of moving the bytes, first with one direction busy, then with both
// GPUs copying against each other at once (the situation of the ZeRO-1 step, where every rank
// pulls from and pushes to its peers at the same time):
//
//   copy engine    cudaMemcpyAsync
//   SM ld / st     256-bit ld.global / st.global from a persistent grid (what rs_pass1 and
//                  pass2_ag of the library issue)
//   bulk           cp.async.bulk global -> shared -> global through a ring of stages, one thread
//                  per CTA driving it (no multicast; every barrier wait bounded)
//
// With four or eight GPUs a second table follows: the all-to-all pattern of the ZeRO-1 step at that
// rank count (every GPU exchanges one slice with each of its R - 1 peers at the same time, 256 MiB
// per pair), inbound GB/s per GPU, for the copy engines (one stream per peer) and for one kernel
// per GPU that issues the loads or the stores itself.
//
// One process, peer access on. Needs two GPUs; prints a note and exits 0 with fewer.
// Built by tests/cpp/build_host_test.py; run and checked by tests/test_gpu_host_cpp.py.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define CK(call)                                                                                     \
    do                                                                                               \
    {                                                                                                \
        cudaError_t err_ = (call);                                                                   \
        if (err_ != cudaSuccess)                                                                     \
        {                                                                                            \
            fprintf(stderr, "CUDA error at line %d: %s (%s)\n", __LINE__, cudaGetErrorString(err_), #call); \
            exit(1);                                                                                 \
        }                                                                                            \
    } while (0)

constexpr long long BYTES = 1LL << 30;
constexpr int SM_GRID = 148 * 4;            // CTAs of the ld/st kernel
constexpr int BULK_GRID = 148 * 2;
constexpr int BULK_TILE = 16384;
constexpr int BULK_STAGES = 6;
constexpr unsigned WAIT_LIMIT = 1u << 20;   // polls of one barrier before the kernel gives up

__device__ int g_gave_up = 0;

// ---------------------------------------------------------------- SM loads and stores

struct Float8
{
    float v[8];
};

__device__ __forceinline__ Float8 load8(const float *p)
{
    Float8 r;
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]),
                   "=f"(r.v[7])
                 : "l"(p));
    return r;
}

__device__ __forceinline__ void store8(float *p, const Float8 &r)
{
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :
                 : "l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]),
                   "f"(r.v[7])
                 : "memory");
}

// two 32-byte groups per thread per trip, loads first
__global__ void __launch_bounds__(256) sm_copy(const float *__restrict__ src, float *__restrict__ dst, long long n8)
{
    const long long stride = static_cast<long long>(gridDim.x) * 256;
    long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    for (; i + stride < n8; i += 2 * stride)
    {
        const Float8 a = load8(src + i * 8);
        const Float8 b = load8(src + (i + stride) * 8);
        store8(dst + i * 8, a);
        store8(dst + (i + stride) * 8, b);
    }
    if (i < n8)
    {
        store8(dst + i * 8, load8(src + i * 8));
    }
}

// ---------------------------------------------------------------- bulk copies through shared memory

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool barrier_wait(uint64_t *bar, unsigned parity)
{
    for (unsigned tries = 0; tries < WAIT_LIMIT; tries++)
    {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(smem_u32(bar)), "r"(parity)
                     : "memory");
        if (ok)
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

__device__ __forceinline__ void request_tile(char *slot, const char *src, uint64_t *bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" : : "r"(smem_u32(bar)), "r"(BULK_TILE)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :
                 : "r"(smem_u32(slot)), "l"(src), "r"(BULK_TILE), "r"(smem_u32(bar))
                 : "memory");
}

// Tile t of the buffer goes through slot (k mod stages) of CTA (t mod grid), k its index among the
// CTA's tiles. The slot refilled at trip d was stored from at trip d - 2, so at most the newest
// store group may still be reading shared memory when the refill is requested.
__global__ void __launch_bounds__(32) bulk_copy(const char *__restrict__ src, char *__restrict__ dst, long long tiles)
{
    extern __shared__ __align__(128) char ring[];
    __shared__ uint64_t full[BULK_STAGES];
    if (threadIdx.x != 0)
    {
        return;                                 // one thread drives the whole pipeline
    }
    for (int s = 0; s < BULK_STAGES; s++)
    {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" : : "r"(smem_u32(&full[s])) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" : : : "memory");
    long long mine = 0;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x)
    {
        mine++;
    }
    constexpr int AHEAD = BULK_STAGES - 2;
    for (long long k = 0; k < AHEAD && k < mine; k++)
    {
        request_tile(ring + (k % BULK_STAGES) * BULK_TILE, src + (blockIdx.x + k * gridDim.x) * BULK_TILE,
                     &full[k % BULK_STAGES]);
    }
    long long done = 0;
    bool ok = true;
    for (; done < mine; done++)
    {
        const long long next = done + AHEAD;
        if (next < mine)
        {
            asm volatile("cp.async.bulk.wait_group.read 1;" : : : "memory");
            request_tile(ring + (next % BULK_STAGES) * BULK_TILE, src + (blockIdx.x + next * gridDim.x) * BULK_TILE,
                         &full[next % BULK_STAGES]);
        }
        if (!barrier_wait(&full[done % BULK_STAGES], static_cast<unsigned>((done / BULK_STAGES) & 1)))
        {
            ok = false;
            break;
        }
        asm volatile("fence.proxy.async.shared::cta;" : : : "memory");
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                     :
                     : "l"(dst + (blockIdx.x + done * gridDim.x) * BULK_TILE),
                       "r"(smem_u32(ring + (done % BULK_STAGES) * BULK_TILE)), "r"(BULK_TILE)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" : : : "memory");
    }
    if (!ok)
    {
        g_gave_up = 1;
        // loads already requested still target this CTA's shared memory: one more bounded wait each
        const long long requested = done + AHEAD + 1 < mine ? done + AHEAD + 1 : mine;
        for (long long k = done; k < requested; k++)
        {
            barrier_wait(&full[k % BULK_STAGES], static_cast<unsigned>((k / BULK_STAGES) & 1));
        }
    }
    asm volatile("cp.async.bulk.wait_group 0;" : : : "memory");
}

// ---------------------------------------------------------------- host

enum Mover
{
    COPY_ENGINE,
    SM_LD_ST,
    BULK
};

static const char *MOVER_NAMES[3] = {"copy engine", "SM ld / st (256-bit)", "bulk through shared memory"};

static void enqueue(Mover how, const char *src, char *dst, cudaStream_t s)
{
    if (how == COPY_ENGINE)
    {
        CK(cudaMemcpyAsync(dst, src, BYTES, cudaMemcpyDefault, s));
    }
    else if (how == SM_LD_ST)
    {
        sm_copy<<<SM_GRID, 256, 0, s>>>(reinterpret_cast<const float *>(src), reinterpret_cast<float *>(dst), BYTES / 32);
        CK(cudaGetLastError());
    }
    else
    {
        bulk_copy<<<BULK_GRID, 32, BULK_STAGES * BULK_TILE, s>>>(src, dst, BYTES / BULK_TILE);
        CK(cudaGetLastError());
    }
}

struct Side                                     // one GPU: a stream, two events, three buffers
{
    int device;
    cudaStream_t stream;
    cudaEvent_t begin, end;
    char *a, *b;                                // local source and local destination
};

static Side make_side(int device, int peer)
{
    Side s;
    s.device = device;
    CK(cudaSetDevice(device));
    CK(cudaDeviceEnablePeerAccess(peer, 0));
    CK(cudaStreamCreate(&s.stream));
    CK(cudaEventCreate(&s.begin));
    CK(cudaEventCreate(&s.end));
    CK(cudaMalloc(&s.a, BYTES));
    CK(cudaMalloc(&s.b, BYTES));
    CK(cudaMemset(s.a, device + 1, BYTES));
    CK(cudaMemset(s.b, 0, BYTES));
    CK(cudaFuncSetAttribute(bulk_copy, cudaFuncAttributeMaxDynamicSharedMemorySize, BULK_STAGES * BULK_TILE));
    CK(cudaDeviceSynchronize());
    return s;
}

static bool gave_up(const Side &s)
{
    int flag = 0;
    CK(cudaSetDevice(s.device));
    CK(cudaMemcpyFromSymbol(&flag, g_gave_up, sizeof(int)));
    return flag != 0;
}

// read: each active side copies the OTHER side's `a` into its own `b`; write: its own `a` into the
// other side's `b`. Returns GB/s per direction as seen by each side (0 for an idle side).
static void run(Mover how, bool read, Side &x, Side &y, bool both, double out[2])
{
    Side *sides[2] = {&x, &y};
    const int reps = 5;
    for (int pass = 0; pass < 2; pass++)        // pass 0 warms up
    {
        for (int k = 0; k < (both ? 2 : 1); k++)
        {
            CK(cudaSetDevice(sides[k]->device));
            CK(cudaEventRecord(sides[k]->begin, sides[k]->stream));
        }
        for (int i = 0; i < reps; i++)
        {
            for (int k = 0; k < (both ? 2 : 1); k++)
            {
                Side &me = *sides[k], &other = *sides[1 - k];
                CK(cudaSetDevice(me.device));
                enqueue(how, read ? other.a : me.a, read ? me.b : other.b, me.stream);
            }
        }
        for (int k = 0; k < (both ? 2 : 1); k++)
        {
            CK(cudaSetDevice(sides[k]->device));
            CK(cudaEventRecord(sides[k]->end, sides[k]->stream));
        }
        for (int k = 0; k < (both ? 2 : 1); k++)
        {
            CK(cudaSetDevice(sides[k]->device));
            CK(cudaStreamSynchronize(sides[k]->stream));
        }
    }
    out[0] = out[1] = 0.0;
    for (int k = 0; k < (both ? 2 : 1); k++)
    {
        float ms = 0.0f;
        CK(cudaEventElapsedTime(&ms, sides[k]->begin, sides[k]->end));
        out[k] = static_cast<double>(BYTES) * reps / (ms * 1e-3) / 1e9;
    }
}

// ---------------------------------------------------------------- SM accesses and a copy engine at once
//
// Do kernel-issued peer accesses and a copy engine add up on one link? Both GPUs do the same
// thing against each other: a kernel moves `sm_bytes` (loads from the peer, or stores to the
// peer) while a copy engine pushes `ce_bytes` to the peer on a second stream. Reported: the bytes
// that ARRIVE at a GPU per second (for loads: its own kernel's bytes + the peer's push; for
// stores: the peer kernel's bytes + the peer's push), slower GPU.
static double hybrid(Side &x, Side &y, bool sm_reads, long long sm_bytes, long long ce_bytes)
{
    Side *sides[2] = {&x, &y};
    static cudaStream_t copy_stream[2] = {nullptr, nullptr};
    static cudaEvent_t copy_done[2] = {nullptr, nullptr};
    for (int k = 0; k < 2; k++)
    {
        CK(cudaSetDevice(sides[k]->device));
        if (copy_stream[k] == nullptr)
        {
            CK(cudaStreamCreateWithFlags(&copy_stream[k], cudaStreamNonBlocking));
            CK(cudaEventCreateWithFlags(&copy_done[k], cudaEventDisableTiming));
        }
    }
    const int reps = 4;
    for (int pass = 0; pass < 2; pass++)
    {
        for (int k = 0; k < 2; k++)
        {
            CK(cudaSetDevice(sides[k]->device));
            CK(cudaEventRecord(sides[k]->begin, sides[k]->stream));
            CK(cudaStreamWaitEvent(copy_stream[k], sides[k]->begin, 0));
        }
        for (int i = 0; i < reps; i++)
        {
            for (int k = 0; k < 2; k++)
            {
                Side &me = *sides[k], &other = *sides[1 - k];
                CK(cudaSetDevice(me.device));
                if (sm_bytes > 0)
                {
                    // the kernel uses the lower part of the buffers, the copy engine the upper part
                    sm_copy<<<SM_GRID, 256, 0, me.stream>>>(reinterpret_cast<const float *>(sm_reads ? other.a : me.a),
                                                            reinterpret_cast<float *>(sm_reads ? me.b : other.b),
                                                            sm_bytes / 32);
                    CK(cudaGetLastError());
                }
                if (ce_bytes > 0)
                {
                    CK(cudaMemcpyAsync(other.b + BYTES - ce_bytes, me.a + BYTES - ce_bytes, ce_bytes, cudaMemcpyDefault,
                                       copy_stream[k]));
                }
            }
        }
        for (int k = 0; k < 2; k++)
        {
            CK(cudaSetDevice(sides[k]->device));
            CK(cudaEventRecord(copy_done[k], copy_stream[k]));
            CK(cudaStreamWaitEvent(sides[k]->stream, copy_done[k], 0));
            CK(cudaEventRecord(sides[k]->end, sides[k]->stream));
        }
        for (int k = 0; k < 2; k++)
        {
            CK(cudaSetDevice(sides[k]->device));
            CK(cudaStreamSynchronize(sides[k]->stream));
        }
    }
    double slowest = 1e30;
    for (int k = 0; k < 2; k++)
    {
        float ms = 0.0f;
        CK(cudaEventElapsedTime(&ms, sides[k]->begin, sides[k]->end));
        const double gbs = static_cast<double>(sm_bytes + ce_bytes) * reps / (ms * 1e-3) / 1e9;
        slowest = gbs < slowest ? gbs : slowest;
    }
    return slowest;
}

static void hybrid_table(Side &x, Side &y)
{
    printf("\nSM accesses and a copy-engine push at once, both GPUs against each other, 1 GiB in total per direction,\n"
           "GB/s arriving per GPU (SM share of the bytes -> loads | stores)\n");
    const int shares[] = {100, 85, 75, 65, 50, 0};
    for (int share : shares)
    {
        const long long sm_bytes = BYTES / 100 * share / 4096 * 4096;
        const long long ce_bytes = (BYTES - sm_bytes) / 4096 * 4096;
        const double loads = hybrid(x, y, true, sm_bytes, share == 100 ? 0 : ce_bytes);
        const double stores = hybrid(x, y, false, sm_bytes, share == 100 ? 0 : ce_bytes);
        printf("hybrid SM %3d %% + copy engine %3d %%  %8.1f | %8.1f\n", share, 100 - share, loads, stores);
    }
}

// ---------------------------------------------------------------- all-to-all among R GPUs

constexpr long long SLICE = 256LL << 20;        // bytes each pair of GPUs exchanges per direction
constexpr int MAX_R = 8;

struct PeerList
{
    const float *src[MAX_R - 1];
    float *dst[MAX_R - 1];
    int count;
};

// One kernel moves all R - 1 slices: the loads of a trip are issued together, then the stores.
// Pull: src on the peers, dst local. Push: src local, dst on the peers.
__global__ void __launch_bounds__(256) a2a_copy(PeerList p, long long n8)
{
    const long long stride = static_cast<long long>(gridDim.x) * 256;
    for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < n8; i += stride)
    {
        Float8 v[MAX_R - 1];
#pragma unroll
        for (int k = 0; k < MAX_R - 1; k++)
        {
            if (k < p.count)
            {
                v[k] = load8(p.src[k] + i * 8);
            }
        }
#pragma unroll
        for (int k = 0; k < MAX_R - 1; k++)
        {
            if (k < p.count)
            {
                store8(p.dst[k] + i * 8, v[k]);
            }
        }
    }
}

// The same with 128-bit accesses (what a kernel issues when a thread owns 8 fp16 values).
__global__ void __launch_bounds__(256) a2a_copy_128(PeerList p, long long n4)
{
    const long long stride = static_cast<long long>(gridDim.x) * 256;
    for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < n4; i += stride)
    {
        float4 v[MAX_R - 1];
#pragma unroll
        for (int k = 0; k < MAX_R - 1; k++)
        {
            if (k < p.count)
            {
                v[k] = reinterpret_cast<const float4 *>(p.src[k])[i];
            }
        }
#pragma unroll
        for (int k = 0; k < MAX_R - 1; k++)
        {
            if (k < p.count)
            {
                reinterpret_cast<float4 *>(p.dst[k])[i] = v[k];
            }
        }
    }
}

struct Node
{
    char *src = nullptr, *dst = nullptr;        // R slices each: slice q is what goes to / came from GPU q
    cudaStream_t main = nullptr, lane[MAX_R - 1] = {};
    cudaEvent_t begin = nullptr, end = nullptr, done[MAX_R - 1] = {};
};

// mode 0: copy engine pull, 1: copy engine push, 2: SM loads (pull), 3: SM stores (push), 4 and 5: the
// last two with 128-bit instead of 256-bit accesses.
// Prints the slowest and the fastest GPU's inbound GB/s.
static void all_to_all(Node *nodes, int R, int mode, const char *label)
{
    const int reps = 3;
    for (int pass = 0; pass < 2; pass++)        // pass 0 warms up
    {
        for (int g = 0; g < R; g++)
        {
            CK(cudaSetDevice(g));
            CK(cudaEventRecord(nodes[g].begin, nodes[g].main));
        }
        for (int i = 0; i < reps; i++)
        {
            for (int g = 0; g < R; g++)
            {
                CK(cudaSetDevice(g));
                Node &me = nodes[g];
                if (mode < 2)
                {
                    for (int k = 1; k < R; k++)
                    {
                        const int q = (g + k) % R;
                        if (i == 0)
                        {
                            CK(cudaStreamWaitEvent(me.lane[k - 1], me.begin, 0));
                        }
                        if (mode == 0)
                        {
                            CK(cudaMemcpyAsync(me.dst + q * SLICE, nodes[q].src + g * SLICE, SLICE, cudaMemcpyDefault,
                                               me.lane[k - 1]));
                        }
                        else
                        {
                            CK(cudaMemcpyAsync(nodes[q].dst + g * SLICE, me.src + q * SLICE, SLICE, cudaMemcpyDefault,
                                               me.lane[k - 1]));
                        }
                    }
                }
                else
                {
                    PeerList p = {};
                    p.count = R - 1;
                    const bool pull = mode == 2 || mode == 4;
                    for (int k = 1; k < R; k++)
                    {
                        const int q = (g + k) % R;
                        p.src[k - 1] = reinterpret_cast<const float *>(pull ? nodes[q].src + g * SLICE
                                                                            : me.src + q * SLICE);
                        p.dst[k - 1] = reinterpret_cast<float *>(pull ? me.dst + q * SLICE : nodes[q].dst + g * SLICE);
                    }
                    if (mode < 4)
                    {
                        a2a_copy<<<148 * 4, 256, 0, me.main>>>(p, SLICE / 32);
                    }
                    else
                    {
                        a2a_copy_128<<<148 * 8, 256, 0, me.main>>>(p, SLICE / 16);
                    }
                    CK(cudaGetLastError());
                }
            }
        }
        for (int g = 0; g < R; g++)
        {
            CK(cudaSetDevice(g));
            Node &me = nodes[g];
            if (mode < 2)
            {
                for (int k = 0; k < R - 1; k++)
                {
                    CK(cudaEventRecord(me.done[k], me.lane[k]));
                    CK(cudaStreamWaitEvent(me.main, me.done[k], 0));
                }
            }
            CK(cudaEventRecord(me.end, me.main));
        }
        for (int g = 0; g < R; g++)
        {
            CK(cudaSetDevice(g));
            CK(cudaStreamSynchronize(nodes[g].main));
        }
    }
    double lo = 1e30, hi = 0.0;
    for (int g = 0; g < R; g++)
    {
        float ms = 0.0f;
        CK(cudaEventElapsedTime(&ms, nodes[g].begin, nodes[g].end));
        const double gbs = static_cast<double>(SLICE) * (R - 1) * reps / (ms * 1e-3) / 1e9;
        lo = gbs < lo ? gbs : lo;
        hi = gbs > hi ? gbs : hi;
    }
    printf("all-to-all R=%d %-28s %8.1f .. %8.1f\n", R, label, lo, hi);
}

static int all_to_all_tables(int count)
{
    for (int R = 2; R <= MAX_R && R <= count; R *= 2)
    {
        for (int a = 0; a < R; a++)
        {
            for (int b = 0; b < R; b++)
            {
                int can = 1;
                if (a != b)
                {
                    CK(cudaDeviceCanAccessPeer(&can, a, b));
                }
                if (!can)
                {
                    printf("GPU %d cannot map GPU %d: no all-to-all table for R=%d\n", a, b, R);
                    return 0;
                }
            }
        }
        Node nodes[MAX_R];
        for (int g = 0; g < R; g++)
        {
            CK(cudaSetDevice(g));
            for (int q = 0; q < R; q++)
            {
                if (q != g)
                {
                    cudaError_t err = cudaDeviceEnablePeerAccess(q, 0);
                    if (err != cudaSuccess && err != cudaErrorPeerAccessAlreadyEnabled)
                    {
                        CK(err);
                    }
                    cudaGetLastError();
                }
            }
            Node &me = nodes[g];
            CK(cudaMalloc(&me.src, SLICE * R));
            CK(cudaMalloc(&me.dst, SLICE * R));
            CK(cudaMemset(me.src, g + 1, SLICE * R));
            CK(cudaMemset(me.dst, 0, SLICE * R));
            CK(cudaStreamCreate(&me.main));
            CK(cudaEventCreate(&me.begin));
            CK(cudaEventCreate(&me.end));
            for (int k = 0; k < R - 1; k++)
            {
                CK(cudaStreamCreateWithFlags(&me.lane[k], cudaStreamNonBlocking));
                CK(cudaEventCreateWithFlags(&me.done[k], cudaEventDisableTiming));
            }
            CK(cudaDeviceSynchronize());
        }
        printf("\nall-to-all among %d GPUs, %lld MiB per pair and direction, inbound GB/s per GPU (slowest .. fastest)\n",
               R, SLICE >> 20);
        all_to_all(nodes, R, 0, "copy engine, pull");
        all_to_all(nodes, R, 1, "copy engine, push");
        all_to_all(nodes, R, 2, "SM loads (pull)");
        all_to_all(nodes, R, 4, "SM loads, 128-bit");
        all_to_all(nodes, R, 5, "SM stores, 128-bit");
        all_to_all(nodes, R, 3, "SM stores (push)");
        // the last mode pushed: slice g of GPU q's destination holds GPU g's pattern
        unsigned char got = 0;
        CK(cudaSetDevice(1));
        CK(cudaMemcpy(&got, nodes[1].dst + 0 * SLICE + SLICE - 1, 1, cudaMemcpyDeviceToHost));
        if (got != 1)
        {
            printf("all-to-all R=%d: wrong byte %d in a destination (expected 1)\n", R, got);
            return 1;
        }
        for (int g = 0; g < R; g++)
        {
            CK(cudaSetDevice(g));
            CK(cudaFree(nodes[g].src));
            CK(cudaFree(nodes[g].dst));
        }
    }
    return 0;
}

int main()
{
    int count = 0;
    CK(cudaGetDeviceCount(&count));
    if (count < 2)
    {
        printf("peer_bandwidth needs two GPUs, this machine shows %d: nothing measured\n", count);
        return 0;
    }
    int can01 = 0, can10 = 0;
    CK(cudaDeviceCanAccessPeer(&can01, 0, 1));
    CK(cudaDeviceCanAccessPeer(&can10, 1, 0));
    if (!can01 || !can10)
    {
        printf("GPU 0 and GPU 1 cannot map each other's memory: nothing measured\n");
        return 0;
    }
    Side x = make_side(0, 1), y = make_side(1, 0);
    printf("1 GiB per copy, 5 copies per figure, GB/s per direction\n\n");
    printf("%-30s %-6s %12s %22s\n", "mover", "", "one direction", "both directions (0 | 1)");
    for (int how = 0; how < 3; how++)
    {
        for (int read = 1; read >= 0; read--)
        {
            double one[2], two[2];
            run(static_cast<Mover>(how), read != 0, x, y, false, one);
            run(static_cast<Mover>(how), read != 0, x, y, true, two);
            printf("%-30s %-6s %12.1f %12.1f | %7.1f\n", MOVER_NAMES[how], read ? "read" : "write", one[0], two[0],
                   two[1]);
            if (gave_up(x) || gave_up(y))
            {
                printf("a bulk copy never completed (bounded wait ran out): stopping\n");
                return 1;
            }
        }
    }
    // the last figure was a bulk write of side 0's pattern (1) into side 1's b, and of side 1's (2) into side 0's
    unsigned char tail0 = 0, tail1 = 0;
    CK(cudaMemcpy(&tail0, x.b + BYTES - 1, 1, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&tail1, y.b + BYTES - 1, 1, cudaMemcpyDeviceToHost));
    printf("\nlast byte of each destination: %d and %d (expected 2 and 1)\n", tail0, tail1);
    if (tail0 != 2 || tail1 != 1)
    {
        return 1;
    }
    hybrid_table(x, y);
    CK(cudaSetDevice(0));
    CK(cudaFree(x.a));
    CK(cudaFree(x.b));
    CK(cudaSetDevice(1));
    CK(cudaFree(y.a));
    CK(cudaFree(y.b));
    return all_to_all_tables(count);
}
