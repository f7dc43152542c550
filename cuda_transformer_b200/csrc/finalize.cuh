// finalize.cuh: the part of the step that turns the squared norm and the inf/NaN flag into this
// step's clip coefficient, learning rate, skip decision and next loss scale, on one device
// thread. Shared by every kernel that ends a pass 1 (scaler.cu) and by the ZeRO-1 finalize that
// first waits for the other ranks' pairs (zero1.cu).
#pragma once

#include <climits>
#include <cmath>

#include "internal.cuh"

namespace b200amp
{

// ---------------------------------------------------------------- finalize (shared)

// Learning rate of a 0-based step: linear warmup, then cosine to min_lr, or (decay_steps > 0)
// flat then 1 - sqrt down over the last decay_steps. Double throughout, the numbers of
// cuda/kernels/scaler.cu:69-93 and reference/train.py:79-96.
__device__ inline double schedule_lr(int step, const b200amp_schedule &c)
{
    const double peak = static_cast<double>(c.lr);
    const double floor_lr = static_cast<double>(c.min_lr);
    if (step < c.warmup_steps)
    {
        return peak * (step + 1) / c.warmup_steps;
    }
    if (step >= c.max_steps)
    {
        return floor_lr;
    }
    if (c.decay_steps > 0)
    {
        const int knee = c.max_steps - c.decay_steps;
        if (step < knee)
        {
            return peak;
        }
        const double frac = static_cast<double>(step - knee) / c.decay_steps;
        return floor_lr + (peak - floor_lr) * (1.0 - sqrt(frac));
    }
    const int span = c.max_steps - c.warmup_steps;
    const double frac = static_cast<double>(step - c.warmup_steps) / (span > 1 ? span : 1);
    return floor_lr + 0.5 * (1.0 + cos(3.14159265358979323846 * frac)) * (peak - floor_lr);
}

// One thread. sumsq is the squared norm of the unscaled gradients, bad the inf/NaN
// flag. Field by field what cuda/kernels/scaler.cu:131-170 does: a skipped step
// halves S and leaves adam_t alone; a finite one advances adam_t, computes the bias
// corrections in double from the float betas, and doubles S after growth_interval
// finite steps in a row.
__device__ inline void finalize_state(b200amp_step_state *st, double sumsq, int bad, const b200amp_schedule &c,
                               b200amp_step_state *history, int history_len, bool set_begin_fields)
{
    b200amp_step_state s = *st;
    if (set_begin_fields)
    {
        s.inv_scale = 1.0f / s.loss_scale;      // of THIS step: S changes below, the unscale factor must not
        s.found_inf = bad;
    }
    const float norm = static_cast<float>(sqrt(sumsq));
    s.grad_norm = norm;
    s.clip_coef = fminf(1.0f, c.grad_clip / (norm + 1e-6f));
    const double lr = schedule_lr(s.step, c);
    s.lr = static_cast<float>(lr);
    if (s.found_inf)
    {
        s.skipped += 1;
        s.good_steps = 0;
        if (c.dynamic_scale)
        {
            s.loss_scale *= 0.5f;
        }
    }
    else
    {
        s.adam_t += 1;
        const double t = static_cast<double>(s.adam_t);
        const double bc1 = 1.0 - pow(static_cast<double>(c.beta1), t);
        const double bc2 = 1.0 - pow(static_cast<double>(c.beta2), t);
        s.step_size = static_cast<float>(lr / bc1);
        s.bc2_sqrt = static_cast<float>(sqrt(bc2));
        s.decay = static_cast<float>(1.0 - lr * c.weight_decay);
        s.good_steps += 1;
        if (c.dynamic_scale && s.good_steps >= c.growth_interval)
        {
            s.loss_scale *= 2.0f;
            s.good_steps = 0;
        }
    }
    if (history != nullptr)
    {
        history[s.step % history_len] = s;
    }
    s.step += 1;
    *st = s;
}

} // namespace b200amp
