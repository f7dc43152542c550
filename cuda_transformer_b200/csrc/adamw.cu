// adamw.cu: pass 2 of the step: clip, AdamW on the fp32 master / m / v with
// decoupled weight decay and bias correction, and the fp16 weight cast, in one
// launch over the flat arena (or over one shard of it).
//
// Per element this is cuda/kernels/adamw_multi.cu:20-29,75-89 of the reference.
// The work is laid out for HBM3e instead of for a 46-SM part:
//   * a persistent grid (a multiple of the SM count) strides over 8-element groups;
//     every access is one 256-bit (fp32 arrays) or 128-bit (fp16 arrays) request, so
//     a warp moves 1 KB / 512 B of contiguous memory per instruction and the fp16
//     copy leaves as 16-byte stores, not 2-byte ones;
//   * the decay flag comes from a cursor into the tensor table that each thread
//     advances as its position grows (positions only increase), instead of a binary
//     search per vector; the search runs once per thread, in shared memory;
//   * the native kernel reads the loss-scaled fp16 gradients directly and unscales
//     in registers, so no unscaled copy is ever written or re-read.

#include <climits>

#include "internal.cuh"

namespace b200amp
{

constexpr int P2_THREADS = 256;

// One element, the arithmetic of the reference (cuda/kernels/adamw_multi.cu:20-29): decay the
// parameter, m += (1-b1)(g-m), v = v*b2 + ((1-b2)*g)*g, denom = sqrt(v)/bc2_sqrt + eps,
// p = decayed - step_size*(m/denom). Written as plain expressions and built with nvcc's
// defaults (fused multiply-add contraction on, IEEE sqrt and division: no fast-math, as the
// reference's Makefile:44-46), so the compiler rounds them the way it rounds the reference's.
__device__ __forceinline__ void adamw_element(float &p, float &m, float &v, float g, float w1, float w2, float b2,
                                              float eps, float decay, float step_size, float bc2_sqrt)
{
    const float decayed = p * decay;
    m = m + w1 * (g - m);
    v = v * b2 + w2 * g * g;
    const float denom = sqrtf(v) / bc2_sqrt + eps;
    p = decayed - step_size * (m / denom);
}

// Tensor table in shared memory + the cursor over it.
struct TensorTable
{
    long long first[B200AMP_MAX_TENSORS];
    unsigned char decay[B200AMP_MAX_TENSORS];
};

__device__ __forceinline__ void table_load(TensorTable &tab, const b200amp_tensor_info *tensors, int ntensors)
{
    for (int k = threadIdx.x; k < ntensors; k += blockDim.x)
    {
        tab.first[k] = tensors[k].offset;
        tab.decay[k] = tensors[k].decay ? 1 : 0;
    }
    __syncthreads();
}

struct Cursor
{
    int k;              // the last tensor whose first element is <= the position (0 if none is)
    long long next;     // first element of tensor k + 1, LLONG_MAX past the end
};

__device__ __forceinline__ long long table_next(const TensorTable &tab, int ntensors, int k)
{
    return k + 1 < ntensors ? tab.first[k + 1] : LLONG_MAX;
}

__device__ __forceinline__ Cursor cursor_seek(const TensorTable &tab, int ntensors, long long at)
{
    int lo = 0, hi = ntensors - 1;
    while (lo < hi)
    {
        const int mid = (lo + hi + 1) >> 1;
        if (tab.first[mid] <= at)
        {
            lo = mid;
        }
        else
        {
            hi = mid - 1;
        }
    }
    Cursor c;
    c.k = lo;
    c.next = table_next(tab, ntensors, lo);
    return c;
}

__device__ __forceinline__ void cursor_advance(Cursor &c, const TensorTable &tab, int ntensors, long long at)
{
    while (at >= c.next)
    {
        c.k += 1;
        c.next = table_next(tab, ntensors, c.k);
    }
}

// Decay factors of the two quads of the 8-element group that starts at `at`. Tensor
// offsets are multiples of 4, so a quad never straddles two tensors but a group can.
__device__ __forceinline__ void group_decay(Cursor &c, const TensorTable &tab, int ntensors, long long at,
                                            float wd_decay, float &lo, float &hi)
{
    cursor_advance(c, tab, ntensors, at);
    lo = tab.decay[c.k] ? wd_decay : 1.0f;
    hi = lo;
    if (at + 4 >= c.next)
    {
        Cursor c2 = c;
        cursor_advance(c2, tab, ntensors, at + 4);
        hi = tab.decay[c2.k] ? wd_decay : 1.0f;
    }
}

// ---------------------------------------------------------------- native pass 2 (fp16 gradients)

template <int UNROLL, int LD, int ST>
__global__ void __launch_bounds__(P2_THREADS)
    pass2_f16_kernel(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                     const uint4 *__restrict__ g16, uint4 *__restrict__ w16, long long n8, long long arena_offset,
                     const b200amp_tensor_info *__restrict__ tensors, int ntensors,
                     const b200amp_step_state *__restrict__ st, float b1, float b2, float eps)
{
    __shared__ TensorTable tab;
    table_load(tab, tensors, ntensors);
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

    const long long stride = static_cast<long long>(gridDim.x) * P2_THREADS;
    long long i = static_cast<long long>(blockIdx.x) * P2_THREADS + threadIdx.x;
    if (i >= n8)
    {
        return;
    }
    Cursor cur = cursor_seek(tab, ntensors, arena_offset + i * 8);

    for (; i < n8; i += UNROLL * stride)
    {
        uint4 gw[UNROLL];
        Float8 pp[UNROLL], mm[UNROLL], vv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
        {
            const long long j = i + u * stride;
            if (u == 0 || j < n8)
            {
                gw[u] = load_h8<LD>(g16 + j);
                pp[u] = load8<LD>(master + j * 8);
                mm[u] = load8<LD>(m + j * 8);
                vv[u] = load8<LD>(v + j * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
        {
            const long long j = i + u * stride;
            if (u == 0 || j < n8)
            {
                float d_lo, d_hi;
                group_decay(cur, tab, ntensors, arena_offset + j * 8, wd_decay, d_lo, d_hi);
                const uint32_t words[4] = {gw[u].x, gw[u].y, gw[u].z, gw[u].w};
#pragma unroll
                for (int k = 0; k < 4; k++)
                {
                    const float2 f = half2_bits_to_float2(words[k]);
                    const float d = k < 2 ? d_lo : d_hi;
                    // (g16 * inv) is the unscaled fp32 gradient of the reference, then * clip
                    adamw_element(pp[u].v[2 * k], mm[u].v[2 * k], vv[u].v[2 * k], (f.x * inv) * coef, w1, w2, b2,
                                  eps, d, step_size, bc2_sqrt);
                    adamw_element(pp[u].v[2 * k + 1], mm[u].v[2 * k + 1], vv[u].v[2 * k + 1], (f.y * inv) * coef,
                                  w1, w2, b2, eps, d, step_size, bc2_sqrt);
                }
                store8<ST>(master + j * 8, pp[u]);
                store8<ST>(m + j * 8, mm[u]);
                store8<ST>(v + j * 8, vv[u]);
                if (w16 != nullptr)
                {
                    uint4 out;
                    out.x = float2_to_half2_bits(pp[u].v[0], pp[u].v[1]);
                    out.y = float2_to_half2_bits(pp[u].v[2], pp[u].v[3]);
                    out.z = float2_to_half2_bits(pp[u].v[4], pp[u].v[5]);
                    out.w = float2_to_half2_bits(pp[u].v[6], pp[u].v[7]);
                    store_h8<ST>(w16 + j, out);
                }
            }
        }
    }
}

// ---------------------------------------------------------------- compat pass 2 (fp32 unscaled gradients)

constexpr int P2C_UNROLL = 2;

// 4 elements per request (the reference's granularity: n and every offset are
// multiples of 4 only), grads already unscaled by unscale_and_norm.
__global__ void __launch_bounds__(P2_THREADS)
    adamw_multi_f32_kernel(float4 *__restrict__ params, uint2 *__restrict__ params_x,
                           const float4 *__restrict__ grads, float4 *__restrict__ m, float4 *__restrict__ v,
                           long long n4, const b200amp_tensor_info *__restrict__ tensors, int ntensors,
                           const b200amp_step_state *__restrict__ st, float b1, float b2, float eps)
{
    __shared__ TensorTable tab;
    table_load(tab, tensors, ntensors);
    if (st->found_inf)
    {
        return;
    }
    const float coef = st->clip_coef;
    const float step_size = st->step_size;
    const float bc2_sqrt = st->bc2_sqrt;
    const float wd_decay = st->decay;
    const float w1 = 1.0f - b1;
    const float w2 = 1.0f - b2;

    const long long stride = static_cast<long long>(gridDim.x) * P2_THREADS;
    long long i = static_cast<long long>(blockIdx.x) * P2_THREADS + threadIdx.x;
    if (i >= n4)
    {
        return;
    }
    Cursor cur = cursor_seek(tab, ntensors, i * 4);
    for (; i < n4; i += P2C_UNROLL * stride)
    {
        float4 g[P2C_UNROLL], p[P2C_UNROLL], mm[P2C_UNROLL], vv[P2C_UNROLL];
#pragma unroll
        for (int u = 0; u < P2C_UNROLL; u++)
        {
            const long long j = i + u * stride;
            if (u == 0 || j < n4)
            {
                g[u] = __ldg(grads + j);
                p[u] = params[j];
                mm[u] = m[j];
                vv[u] = v[j];
            }
        }
#pragma unroll
        for (int u = 0; u < P2C_UNROLL; u++)
        {
            const long long j = i + u * stride;
            if (u == 0 || j < n4)
            {
                cursor_advance(cur, tab, ntensors, j * 4);
                const float d = tab.decay[cur.k] ? wd_decay : 1.0f;
                adamw_element(p[u].x, mm[u].x, vv[u].x, g[u].x * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
                adamw_element(p[u].y, mm[u].y, vv[u].y, g[u].y * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
                adamw_element(p[u].z, mm[u].z, vv[u].z, g[u].z * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
                adamw_element(p[u].w, mm[u].w, vv[u].w, g[u].w * coef, w1, w2, b2, eps, d, step_size, bc2_sqrt);
                params[j] = p[u];
                m[j] = mm[u];
                v[j] = vv[u];
                if (params_x != nullptr)
                {
                    uint2 out;
                    out.x = float2_to_half2_bits(p[u].x, p[u].y);
                    out.y = float2_to_half2_bits(p[u].z, p[u].w);
                    params_x[j] = out;
                }
            }
        }
    }
}

// ---------------------------------------------------------------- fp32 -> fp16 arena copy

__global__ void __launch_bounds__(256) cast_f16_kernel(__half *out, const float *in, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    {
        out[i] = __float2half_rn(in[i]);
    }
}

template <int UNROLL>
static void launch_pass2_variant(int ld, int st_hint, int grid, cudaStream_t s, float *master, float *m, float *v,
                                 const uint4 *g16, uint4 *w16, long long n8, long long arena_offset,
                                 const b200amp_tensor_info *tensors, int ntensors, const b200amp_step_state *st,
                                 float b1, float b2, float eps)
{
#define B200AMP_P2(LD, ST)                                                                                         \
    pass2_f16_kernel<UNROLL, LD, ST><<<grid, P2_THREADS, 0, s>>>(master, m, v, g16, w16, n8, arena_offset, tensors, \
                                                                 ntensors, st, b1, b2, eps)
    const int which = (ld < 0 || ld > 2 ? 0 : ld) * 2 + (st_hint == 1 ? 1 : 0);
    switch (which)
    {
    case 0: B200AMP_P2(0, 0); break;
    case 1: B200AMP_P2(0, 1); break;
    case 2: B200AMP_P2(1, 0); break;
    case 3: B200AMP_P2(1, 1); break;
    case 4: B200AMP_P2(2, 0); break;
    default: B200AMP_P2(2, 1); break;
    }
#undef B200AMP_P2
}

static int check_table(const b200amp_tensor_info *tensors, int ntensors)
{
    B200AMP_REQUIRE(tensors != nullptr, "tensor table is null");
    B200AMP_REQUIRE(ntensors > 0 && ntensors <= B200AMP_MAX_TENSORS, "ntensors = %d, must be in 1..%d", ntensors,
                    B200AMP_MAX_TENSORS);
    return B200AMP_OK;
}

} // namespace b200amp

using namespace b200amp;

extern "C" B200AMP_API int b200amp_pass2_f16(float *master, float *m, float *v, const void *grads16, void *weights16,
                                 long long n, long long arena_offset, const b200amp_tensor_info *tensors,
                                 int ntensors, const b200amp_step_state *st, float beta1, float beta2, float eps,
                                 b200amp_stream s)
{
    B200AMP_REQUIRE(master != nullptr && m != nullptr && v != nullptr && grads16 != nullptr && st != nullptr,
                    "pass 2: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass 2: n = %lld must be a positive multiple of 8", n);
    B200AMP_REQUIRE(arena_offset >= 0 && arena_offset % 4 == 0, "pass 2: arena_offset = %lld must be a multiple of 4",
                    arena_offset);
    B200AMP_REQUIRE(aligned(master, 32) && aligned(m, 32) && aligned(v, 32),
                    "pass 2: master, m and v must be 32-byte aligned");
    B200AMP_REQUIRE(aligned(grads16, 16) && aligned(weights16, 16),
                    "pass 2: the fp16 arenas must be 16-byte aligned");
    int rc = check_table(tensors, ntensors);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const Tunables &t = tunables();
    const long long n8 = n / 8;
    long long want = (n8 + P2_THREADS - 1) / P2_THREADS;
    int grid = sms * t.pass2_blocks_per_sm;
    if (grid > want)
    {
        grid = static_cast<int>(want);
    }
    const uint4 *g16 = static_cast<const uint4 *>(grads16);
    uint4 *w16 = static_cast<uint4 *>(weights16);
    if (t.pass2_unroll == 2)
    {
        launch_pass2_variant<2>(t.pass2_load_hint, t.pass2_store_hint, grid, as_stream(s), master, m, v, g16, w16, n8,
                                arena_offset, tensors, ntensors, st, beta1, beta2, eps);
    }
    else
    {
        launch_pass2_variant<1>(t.pass2_load_hint, t.pass2_store_hint, grid, as_stream(s), master, m, v, g16, w16, n8,
                                arena_offset, tensors, ntensors, st, beta1, beta2, eps);
    }
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_adamw_multi_f32(float *params, void *params_x, const float *grads, float *m, float *v,
                                       long long n, const b200amp_tensor_info *tensors, int ntensors,
                                       const b200amp_step_state *st, float beta1, float beta2, float eps,
                                       b200amp_stream s)
{
    B200AMP_REQUIRE(params != nullptr && grads != nullptr && m != nullptr && v != nullptr && st != nullptr,
                    "adamw_multi: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 4 == 0, "adamw_multi: n = %lld must be a positive multiple of 4", n);
    B200AMP_REQUIRE(aligned(params, 16) && aligned(grads, 16) && aligned(m, 16) && aligned(v, 16),
                    "adamw_multi: params, grads, m and v must be 16-byte aligned");
    B200AMP_REQUIRE(aligned(params_x, 8), "adamw_multi: params_x must be 8-byte aligned");
    int rc = check_table(tensors, ntensors);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const long long n4 = n / 4;
    long long want = (n4 + P2_THREADS - 1) / P2_THREADS;
    int grid = sms * tunables().pass2_blocks_per_sm;
    if (grid > want)
    {
        grid = static_cast<int>(want);
    }
    adamw_multi_f32_kernel<<<grid, P2_THREADS, 0, as_stream(s)>>>(
        reinterpret_cast<float4 *>(params), static_cast<uint2 *>(params_x), reinterpret_cast<const float4 *>(grads),
        reinterpret_cast<float4 *>(m), reinterpret_cast<float4 *>(v), n4, tensors, ntensors, st, beta1, beta2, eps);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_cast_to_x(void *out_f16, const float *in, long long n, b200amp_stream s)
{
    B200AMP_REQUIRE(n >= 0, "cast_to_x: n = %lld", n);
    if (n == 0)
    {
        return B200AMP_OK;
    }
    B200AMP_REQUIRE(out_f16 != nullptr && in != nullptr, "cast_to_x: null pointer");
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    long long want = (n + 255) / 256;
    int grid = sms * 16;
    if (grid > want)
    {
        grid = static_cast<int>(want);
    }
    cast_f16_kernel<<<grid, 256, 0, as_stream(s)>>>(static_cast<__half *>(out_f16), in, n);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}
