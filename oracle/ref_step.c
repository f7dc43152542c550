/* ref_step.c: CPU restatement of cuda-transformer's AMP optimizer step.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing the library ships calls into this file; the
 * tests, the smoke check and the CPU-baseline leg of the benchmark are its only
 * users, and there only as the checker.
 *
 * Parity is pinned two ways (see tests/test_oracle_golden.py): against golden
 * vectors produced by importing the reference's own PyTorch path
 * (reference/model.py:246-260, reference/train.py:141-154, reference/dump.py:104-158),
 * and, on a GPU box, against the reference's own CUDA kernels compiled from its
 * sources (oracle/build_ref.py).
 *
 * Each function names the reference lines it restates. `contract` selects how the
 * three multiply-add expressions of the per-element update are rounded:
 *   0      every operation rounded on its own (what torch's CPU AdamW does, and what
 *          the reference's kernels would do if built with -fmad=false);
 *   bit 0  fused multiply-adds, as nvcc contracts by default (the reference's
 *          Makefile:44-46 keeps the default). m + w1*(g-m) has one possible fusion;
 *          v*b2 + (w2*g)*g and p*decay - step*(m/denom) are each a sum of two products,
 *          and a compiler may fuse either product:
 *   bit 1  v: fuse (w2*g)*g instead of v*b2;
 *   bit 2  p: fuse p*decay instead of step*(m/denom).
 * Which pair nvcc picks is found on the GPU by the test that compares against the
 * reference's compiled kernels; all variants differ by at most one rounding per operation.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define NORM_BLOCKS 512     /* cuda/kernels/fast.h:150 */
#define NORM_THREADS 256    /* cuda/kernels/scaler.cu:19 */

typedef struct
{
    float loss_scale, inv_scale;
    int good_steps, found_inf, skipped, step, adam_t;
    float lr, grad_norm, clip_coef, step_size, bc2_sqrt, decay, loss;
    int n_valid;
} step_state;               /* cuda/kernels/fast.h:104-121 */

typedef struct
{
    float lr, min_lr;
    int warmup_steps, max_steps;
    float beta1, beta2, weight_decay, grad_clip;
    int growth_interval, dynamic_scale, decay_steps;
} schedule;                 /* cuda/kernels/fast.h:123-133 */

typedef struct
{
    long long offset, count;
    int decay;
} tensor_info;              /* cuda/kernels/fast.h:153-158 */

int oracle_sizeof_state(void) { return (int)sizeof(step_state); }
int oracle_sizeof_schedule(void) { return (int)sizeof(schedule); }
int oracle_sizeof_tensor_info(void) { return (int)sizeof(tensor_info); }

/* ------------------------------------------------------------ fp16 <-> fp32, bit level
 * cuda/precision.h:39-43: __float2half is round-to-nearest-even; __half2float is exact. */
float oracle_half_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0)
    {
        if (man == 0)
        {
            bits = sign;
        }
        else
        {                                   /* subnormal: normalise */
            int e = -1;
            do
            {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    }
    else if (exp == 31)
    {
        bits = sign | 0x7F800000u | (man << 13);
    }
    else
    {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_float_to_half(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u)                  /* inf or NaN */
    {
        return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x0200u | ((ax >> 13) & 0x3FFu) : 0u));
    }
    if (ax >= 0x477FF000u)                  /* rounds to >= 65520: overflow to inf */
    {
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax < 0x33000001u)                   /* <= 2^-25: rounds to zero (2^-25 itself ties to even = 0) */
    {
        return sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift = e < -14 ? (13 + (-14 - e)) : 13;    /* bits dropped from the 24-bit significand */
    uint32_t kept = man >> shift;
    uint32_t rest = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rest > halfway || (rest == halfway && (kept & 1u)))
    {
        kept++;
    }
    uint32_t out;
    if (e < -14)
    {
        out = kept;                         /* subnormal; a carry into bit 10 lands on the smallest normal */
    }
    else
    {
        out = ((uint32_t)(e + 15) << 10) + (kept - 0x400u);    /* a carry out of the mantissa bumps the exponent */
    }
    return (uint16_t)(sign | out);
}

/* ------------------------------------------------------------ state */

/* cuda/kernels/scaler.cu:21-29 */
void oracle_initial_state(float scale, step_state *out)
{
    memset(out, 0, sizeof(*out));
    out->loss_scale = scale;
    out->inv_scale = 1.0f / scale;
    out->clip_coef = 1.0f;
    out->decay = 1.0f;
}

/* cuda/kernels/scaler.cu:31-35 */
void oracle_begin_step(step_state *st)
{
    st->found_inf = 0;
    st->inv_scale = 1.0f / st->loss_scale;
}

/* cuda/kernels/scaler.cu:69-93 (and reference/train.py:79-96) */
double oracle_lr(int step, const schedule *c)
{
    if (step < c->warmup_steps)
    {
        return (double)c->lr * (step + 1) / c->warmup_steps;
    }
    if (step >= c->max_steps)
    {
        return c->min_lr;
    }
    if (c->decay_steps > 0)
    {
        int from = c->max_steps - c->decay_steps;
        if (step < from)
        {
            return c->lr;
        }
        double p = (double)(step - from) / c->decay_steps;
        return c->min_lr + ((double)c->lr - c->min_lr) * (1.0 - sqrt(p));
    }
    int span = c->max_steps - c->warmup_steps;
    double progress = (double)(step - c->warmup_steps) / (span > 1 ? span : 1);
    return c->min_lr + 0.5 * (1.0 + cos(3.14159265358979323846 * progress)) * ((double)c->lr - c->min_lr);
}

/* cuda/kernels/scaler.cu:131-170, from an already reduced squared norm */
void oracle_finalize_sumsq(step_state *st, double sumsq, const schedule *c, step_state *history, int history_len)
{
    step_state s = *st;
    float norm = (float)sqrt(sumsq);
    s.grad_norm = norm;
    float ratio = c->grad_clip / (norm + 1e-6f);
    s.clip_coef = fminf(1.0f, ratio);       /* fminf drops a NaN: a NaN norm gives 1 */
    double lr = oracle_lr(s.step, c);
    s.lr = (float)lr;
    if (s.found_inf)
    {
        s.skipped++;
        s.good_steps = 0;
        if (c->dynamic_scale)
        {
            s.loss_scale *= 0.5f;
        }
    }
    else
    {
        s.adam_t++;
        double bc1 = 1.0 - pow((double)c->beta1, (double)s.adam_t);
        double bc2 = 1.0 - pow((double)c->beta2, (double)s.adam_t);
        s.step_size = (float)(lr / bc1);
        s.bc2_sqrt = (float)sqrt(bc2);
        s.decay = (float)(1.0 - lr * c->weight_decay);
        s.good_steps++;
        if (c->dynamic_scale && s.good_steps >= c->growth_interval)
        {
            s.loss_scale *= 2.0f;
            s.good_steps = 0;
        }
    }
    if (history != NULL)
    {
        history[s.step % history_len] = s;
    }
    s.step++;
    *st = s;
}

/* cuda/kernels/scaler.cu:115-130: the 512 partials in double, halving tree */
double oracle_tree_sum(const float *partial)
{
    double tree[NORM_BLOCKS];
    for (int i = 0; i < NORM_BLOCKS; i++)
    {
        tree[i] = partial[i];
    }
    for (int half = NORM_BLOCKS / 2; half > 0; half /= 2)
    {
        for (int i = 0; i < half; i++)
        {
            tree[i] += tree[i + half];
        }
    }
    return tree[0];
}

void oracle_finalize(step_state *st, const float *partial, const schedule *c, step_state *history, int history_len)
{
    oracle_finalize_sumsq(st, oracle_tree_sum(partial), c, history, history_len);
}

/* ------------------------------------------------------------ pass 1, fp32 gradients in place
 * cuda/kernels/scaler.cu:39-66 with the launch of :179-184 (512 blocks x 256 threads):
 * quad i belongs to virtual thread i mod 131072; each thread adds its quads' squares in
 * fp32 in order; cuda/kernels/reduce.cuh:11-47: xor butterfly over the 32 lanes, one
 * value per warp through shared memory, butterfly again. */
static float butterfly32(float *lanes)      /* lanes[32] -> the value every lane ends with */
{
    float cur[32], nxt[32];
    memcpy(cur, lanes, sizeof(cur));
    for (int offset = 16; offset > 0; offset /= 2)
    {
        for (int l = 0; l < 32; l++)
        {
            nxt[l] = cur[l] + cur[l ^ offset];
        }
        memcpy(cur, nxt, sizeof(cur));
    }
    return cur[0];
}

void oracle_unscale_and_norm_f32(float *grads, long long n, step_state *st, float *partial, int contract)
{
    const long long n4 = n / 4;
    const long long stride = (long long)NORM_BLOCKS * NORM_THREADS;
    const float inv = st->inv_scale;
    int any_bad = 0;
#pragma omp parallel for schedule(static) reduction(| : any_bad)
    for (int b = 0; b < NORM_BLOCKS; b++)
    {
        float thread_sum[NORM_THREADS];
        for (int t = 0; t < NORM_THREADS; t++)
        {
            float sum = 0.0f;
            for (long long i = (long long)b * NORM_THREADS + t; i < n4; i += stride)
            {
                float *g = grads + 4 * i;
                float x = g[0] * inv, y = g[1] * inv, z = g[2] * inv, w = g[3] * inv;
                g[0] = x;
                g[1] = y;
                g[2] = z;
                g[3] = w;
                if (!isfinite(x) || !isfinite(y) || !isfinite(z) || !isfinite(w))
                {
                    any_bad |= 1;
                }
                float q;
                if (contract)
                {
                    q = fmaf(w, w, fmaf(z, z, fmaf(y, y, x * x)));
                }
                else
                {
                    q = ((x * x + y * y) + z * z) + w * w;
                }
                sum += q;
            }
            thread_sum[t] = sum;
        }
        float warp_total[32];
        memset(warp_total, 0, sizeof(warp_total));
        for (int w = 0; w < NORM_THREADS / 32; w++)
        {
            warp_total[w] = butterfly32(thread_sum + 32 * w);
        }
        partial[b] = butterfly32(warp_total);
    }
    if (any_bad)
    {
        st->found_inf = 1;
    }
}

/* ------------------------------------------------------------ pass 2
 * cuda/kernels/adamw_multi.cu:20-29 */
static inline void adamw_one(float *p, float *m, float *v, float g, float b1, float b2, float eps, float decay,
                             float step_size, float bc2_sqrt, int contract)
{
    float w1 = 1.0f - b1, w2 = 1.0f - b2;
    float mi, vi, denom, out;
    if (contract & 1)
    {
        mi = fmaf(w1, g - *m, *m);
        if (contract & 2)
        {
            vi = fmaf(w2 * g, g, *v * b2);              /* the product v*b2 rounded, the other fused */
        }
        else
        {
            vi = fmaf(*v, b2, (w2 * g) * g);            /* the product (w2*g)*g rounded, v*b2 fused */
        }
        denom = sqrtf(vi) / bc2_sqrt + eps;
        if (contract & 4)
        {
            out = fmaf(*p, decay, -(step_size * (mi / denom)));     /* p*decay fused, the update rounded */
        }
        else
        {
            out = fmaf(-step_size, mi / denom, *p * decay);         /* p*decay rounded, the update fused */
        }
    }
    else
    {
        float param = *p * decay;
        mi = *m + w1 * (g - *m);
        vi = *v * b2 + (w2 * g) * g;
        denom = sqrtf(vi) / bc2_sqrt + eps;
        out = param - step_size * (mi / denom);
    }
    *m = mi;
    *v = vi;
    *p = out;
}

/* the last tensor whose first element is <= at (cuda/kernels/adamw_multi.cu:55-69) */
static int find_tensor(const tensor_info *tensors, int ntensors, long long at)
{
    int lo = 0, hi = ntensors - 1;
    while (lo < hi)
    {
        int mid = (lo + hi + 1) / 2;
        if (tensors[mid].offset <= at)
        {
            lo = mid;
        }
        else
        {
            hi = mid - 1;
        }
    }
    return lo;
}

/* cuda/kernels/adamw_multi.cu:31-91. grads: unscaled fp32. params_x: fp16 bits or NULL.
 * arena_offset: index of element 0 in the whole arena (the reference has no shards: 0). */
void oracle_adamw_multi(float *params, uint16_t *params_x, const float *grads, float *m, float *v, long long n,
                        long long arena_offset, const tensor_info *tensors, int ntensors, const step_state *st,
                        float b1, float b2, float eps, int contract)
{
    if (st->found_inf)
    {
        return;
    }
    const float coef = st->clip_coef, step_size = st->step_size, bc2_sqrt = st->bc2_sqrt, wd = st->decay;
#pragma omp parallel for schedule(static)
    for (long long q = 0; q < n / 4; q++)
    {
        long long at = 4 * q;
        int k = find_tensor(tensors, ntensors, arena_offset + at);
        float decay = tensors[k].decay ? wd : 1.0f;
        for (int e = 0; e < 4; e++)
        {
            long long i = at + e;
            adamw_one(&params[i], &m[i], &v[i], grads[i] * coef, b1, b2, eps, decay, step_size, bc2_sqrt, contract);
            if (params_x != NULL)
            {
                params_x[i] = oracle_float_to_half(params[i]);
            }
        }
    }
}

/* ------------------------------------------------------------ fp16 gradient arena
 * No reference function takes fp16 gradients. The reference's pass 1 applied to
 * float(fp16 gradient): the widening and the multiplication by the power-of-two 1/S are
 * exact, so element values equal the reference's unscaled fp32 gradients. The sum of
 * squares is taken in double here (the exact value up to 1e-16), which is what the
 * reference's 131072 short fp32 sums + fp64 tree approximate to about 1e-7. */
void oracle_pass1_f16(const uint16_t *g16, long long n, float loss_scale, double *sumsq, int *bad)
{
    const float inv = 1.0f / loss_scale;
    double total = 0.0;
    int any_bad = 0;
    /* fixed chunks so the double sum does not depend on the thread count */
    const long long chunk = 1 << 16;
    const long long nchunks = (n + chunk - 1) / chunk;
    double *part = (double *)calloc((size_t)nchunks, sizeof(double));
#pragma omp parallel for schedule(static) reduction(| : any_bad)
    for (long long c = 0; c < nchunks; c++)
    {
        long long end = (c + 1) * chunk < n ? (c + 1) * chunk : n;
        double s = 0.0;
        for (long long i = c * chunk; i < end; i++)
        {
            if ((g16[i] & 0x7C00u) == 0x7C00u)
            {
                any_bad |= 1;
            }
            float g = oracle_half_to_float(g16[i]) * inv;
            s += (double)g * (double)g;
        }
        part[c] = s;
    }
    for (long long c = 0; c < nchunks; c++)
    {
        total += part[c];
    }
    free(part);
    *sumsq = total;
    *bad = any_bad;
}

/* out[i] = float(g16[i]) * inv_scale: the reference's unscaled fp32 gradient arena */
void oracle_unscale_f16(const uint16_t *g16, long long n, float inv_scale, float *out)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++)
    {
        out[i] = oracle_half_to_float(g16[i]) * inv_scale;
    }
}

/* out[i] = fp16(in[i]) round to nearest even (cuda/kernels/fused.cu:285-292 in the fp16 build) */
void oracle_cast_to_half(uint16_t *out, const float *in, long long n)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++)
    {
        out[i] = oracle_float_to_half(in[i]);
    }
}
