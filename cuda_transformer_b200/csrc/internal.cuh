// internal.cuh: what the .cu files of the library share: error reporting, the
// launch counter, tuning knobs, 128/256-bit global memory accessors and the
// reductions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "b200amp.h"

namespace b200amp
{

// ---------------------------------------------------------------- host side
void set_error(const char *fmt, ...);           // text for b200amp_last_error() on this thread
int cuda_fail(cudaError_t err, const char *what, const char *file, int line);
void count_launch();                            // one more kernel launch enqueued
int sm_count();                                 // SMs of the current device (cached per device), <= 0 on error
int zero1_sync_timeout_take(int *out);          // zero1.cu: *out = 1 if a wait on another rank gave up (clears it)

struct Tunables
{
    int pass1_blocks_per_sm;    // resident CTAs per SM asked for in pass 1
    int pass2_blocks_per_sm;    // same, pass 2
    int pass2_store_hint;       // 0: plain stores, 1: st.global.cs (streaming)
    int pass2_threads;          // threads per CTA of the registers-only kernel: 256, 512 or 1024
    int pass2_variant;          // 0: registers-only kernel, 1: shared-memory staged kernel (bulk async copies)
    int pass2_stages;           // ring depth of the staged kernel: 3..7 (28 KB each)
    int pass2_test_starve;      // test hook of the staged kernel: 1 makes one barrier wait run out (see pass2.cu)
    int rs_blocks_per_sm;       // resident CTAs per SM of the fused reduce-scatter + pass 1
    int ag_blocks_per_sm;       // resident CTAs per SM of the fused pass 2 + all-gather, 0 = by rank count
    int bridge_blocks_per_sm;   // CTAs per SM asked for by the fp32 -> fp16 bridge (cast + pass 1)
    int ce_lanes;               // copy streams the copy-engine forms of the ZeRO-1 step spread their copies over
};
Tunables &tunables();

#define B200AMP_CUDA(call)                                                      \
    do                                                                          \
    {                                                                           \
        cudaError_t err_ = (call);                                              \
        if (err_ != cudaSuccess)                                                \
        {                                                                       \
            return b200amp::cuda_fail(err_, #call, __FILE__, __LINE__);         \
        }                                                                       \
    } while (0)

// after a <<<>>> launch: the launch error, if any, becomes the status
#define B200AMP_LAUNCHED()                                                      \
    do                                                                          \
    {                                                                           \
        b200amp::count_launch();                                                \
        B200AMP_CUDA(cudaGetLastError());                                       \
    } while (0)

#define B200AMP_REQUIRE(cond, ...)                                              \
    do                                                                          \
    {                                                                           \
        if (!(cond))                                                            \
        {                                                                       \
            b200amp::set_error(__VA_ARGS__);                                    \
            return B200AMP_ERR_ARG;                                             \
        }                                                                       \
    } while (0)

inline bool aligned(const void *p, size_t a)
{
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

inline cudaStream_t as_stream(b200amp_stream s)
{
    return static_cast<cudaStream_t>(s);
}

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

struct __align__(32) Float8
{
    float v[8];
};

// 256-bit global accesses (PTX ISA 8.8, sm_100): one instruction per 8 floats, so
// a warp touches 1 KB of contiguous memory per request. Load HINT: 0 plain,
// 1 do not allocate in L1, 2 streaming (evict first). These arrays are rewritten by
// the same thread later in the kernel, so the read-only (.nc) path is not used here.
template <int HINT>
__device__ __forceinline__ Float8 load8(const float *p)
{
    Float8 r;
    if (HINT == 1)
    {
        asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]),
                       "=f"(r.v[6]), "=f"(r.v[7])
                     : "l"(p));
    }
    else if (HINT == 2)
    {
        asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]),
                       "=f"(r.v[6]), "=f"(r.v[7])
                     : "l"(p));
    }
    else
    {
        asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]),
                       "=f"(r.v[6]), "=f"(r.v[7])
                     : "l"(p));
    }
    return r;
}

template <int HINT>
__device__ __forceinline__ void store8(float *p, const Float8 &r)
{
    if (HINT == 1)
    {
        asm volatile("st.global.cs.v8.f32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                     :
                     : "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]),
                       "f"(r.v[7]), "l"(p)
                     : "memory");
    }
    else
    {
        asm volatile("st.global.v8.f32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                     :
                     : "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]),
                       "f"(r.v[7]), "l"(p)
                     : "memory");
    }
}

// 8 fp16 values = 16 bytes. The fp16 gradient arena is read-only for the whole
// kernel, so hint 1 may take the non-coherent path.
template <int HINT>
__device__ __forceinline__ uint4 load_h8(const uint4 *p)
{
    uint4 r;
    if (HINT == 1)
    {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                     : "l"(p));
    }
    else if (HINT == 2)
    {
        asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    }
    else
    {
        asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    }
    return r;
}

template <int HINT>
__device__ __forceinline__ void store_h8(uint4 *p, const uint4 &r)
{
    if (HINT == 1)
    {
        asm volatile("st.global.cs.v4.u32 [%4], {%0,%1,%2,%3};" : : "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w), "l"(p)
                     : "memory");
    }
    else
    {
        asm volatile("st.global.v4.u32 [%4], {%0,%1,%2,%3};" : : "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w), "l"(p)
                     : "memory");
    }
}

__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t w)
{
    __half2 h = *reinterpret_cast<__half2 *>(&w);
    return __half22float2(h);
}

// two floats -> two fp16, round to nearest even, low half = a
__device__ __forceinline__ uint32_t float2_to_half2_bits(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// True if either fp16 half of w has all exponent bits set (inf or NaN): adding
// 0x0400 to the 15 magnitude bits carries into bit 15 exactly then, and the
// low half's carry cannot reach the high half.
__device__ __forceinline__ uint32_t half2_nonfinite_bits(uint32_t w)
{
    return ((w & 0x7FFF7FFFu) + 0x04000400u) & 0x80008000u;
}

// xor butterfly: every lane ends with the same bits (the order the reference's
// warp_sum uses, cuda/kernels/reduce.cuh:11-18)
__device__ __forceinline__ float warp_sum_f32(float v)
{
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
    {
        v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    return v;
}

__device__ __forceinline__ double warp_sum_f64(double v)
{
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
    {
        v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    return v;
}

#endif // __CUDACC__

} // namespace b200amp
