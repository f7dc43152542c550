// adamw.cu: the compat form of pass 2 (the reference's adamw_multi arguments: unscaled
// fp32 gradients, granularity 4) and the fp32 -> fp16 arena copy. The native pass 2 over
// an fp16 gradient arena is in pass2.cu.

#include "adamw_math.cuh"

namespace b200amp
{

constexpr int P2_THREADS = 256;

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
    const int nruns = table_load(tab, tensors, ntensors);
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
    Cursor cur = cursor_seek(tab, nruns, i * 4, wd_decay);
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
                cursor_advance(cur, tab, nruns, j * 4, wd_decay);
                const float d = cur.factor;
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

// The same update on 8 elements per request (256-bit accesses, the shape of the native pass 2),
// used when n is a multiple of 8 and every array is 32-byte aligned (params_x 16-byte). The
// per-element arithmetic is adamw_element either way, so the two forms give the same bits.
__global__ void __launch_bounds__(P2_THREADS)
    adamw_multi_f32_v8_kernel(float *__restrict__ params, uint4 *__restrict__ params_x,
                              const float *__restrict__ grads, float *__restrict__ m, float *__restrict__ v,
                              int groups, const b200amp_tensor_info *__restrict__ tensors, int ntensors,
                              const b200amp_step_state *__restrict__ st, float b1, float b2, float eps)
{
    __shared__ TensorTable tab;
    const int nruns = table_load(tab, tensors, ntensors);
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

    const int stride = static_cast<int>(gridDim.x) * P2_THREADS;
    int i = static_cast<int>(blockIdx.x) * P2_THREADS + static_cast<int>(threadIdx.x);
    if (i >= groups)
    {
        return;
    }
    Cursor cur = cursor_seek(tab, nruns, static_cast<long long>(i) * 8, wd_decay);
    for (; i < groups; i += stride)
    {
        const size_t e = static_cast<size_t>(i) * 8;
        const Float8 gg = load8<0>(grads + e);
        Float8 pp = load8<0>(params + e);
        Float8 mm = load8<0>(m + e);
        Float8 vv = load8<0>(v + e);
        float d_lo, d_hi;
        group_decay(cur, tab, nruns, static_cast<long long>(e), wd_decay, d_lo, d_hi);
#pragma unroll
        for (int k = 0; k < 8; k++)
        {
            adamw_element(pp.v[k], mm.v[k], vv.v[k], gg.v[k] * coef, w1, w2, b2, eps, k < 4 ? d_lo : d_hi, step_size,
                          bc2_sqrt);
        }
        store8<1>(params + e, pp);
        store8<1>(m + e, mm);
        store8<1>(v + e, vv);
        if (params_x != nullptr)
        {
            uint4 out;
            out.x = float2_to_half2_bits(pp.v[0], pp.v[1]);
            out.y = float2_to_half2_bits(pp.v[2], pp.v[3]);
            out.z = float2_to_half2_bits(pp.v[4], pp.v[5]);
            out.w = float2_to_half2_bits(pp.v[6], pp.v[7]);
            store_h8<1>(params_x + i, out);
        }
    }
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
    const bool wide = n % 8 == 0 && n / 8 <= (1LL << 31) - (1LL << 23) && aligned(params, 32) && aligned(grads, 32) &&
                      aligned(m, 32) && aligned(v, 32) && aligned(params_x, 16);
    if (wide)
    {
        const long long groups = n / 8;
        long long want8 = (groups + P2_THREADS - 1) / P2_THREADS;
        int grid8 = sms * 2;                    // the native pass 2's shape: 2 CTAs per SM
        if (grid8 > want8)
        {
            grid8 = static_cast<int>(want8);
        }
        adamw_multi_f32_v8_kernel<<<grid8, P2_THREADS, 0, as_stream(s)>>>(
            params, static_cast<uint4 *>(params_x), grads, m, v, static_cast<int>(groups), tensors, ntensors, st,
            beta1, beta2, eps);
        B200AMP_LAUNCHED();
        return B200AMP_OK;
    }
    const long long n4 = n / 4;
    long long want = (n4 + P2_THREADS - 1) / P2_THREADS;
    int grid = sms * 4;                         // 4 CTAs per SM measured best for the 128-bit form on B200
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
