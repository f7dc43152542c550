// zero1_sync.cuh: ordering between the ranks of the ZeRO-1 step without a host, a library
// barrier or an endless spin. Every rank owns one small block of 32-bit words that all ranks
// have mapped (b200amp_zero1_sync in b200amp.h). A rank announces "phase p of step e is done
// on my side" by storing e into word [p][my_rank] of EVERY rank's block (plain peer stores with
// release semantics at system scope); a rank that needs phase p of all ranks polls the R words
// [p][*] of its OWN block (local memory) until each has reached e. The step number e lives in
// the block too (word EPOCH, advanced by the last kernel of a step), so nothing on the host
// changes from step to step and a captured graph can be replayed.
//
// Every wait is bounded: after `limit` polls the waiting thread records which phase and which
// rank it was waiting for in word ERROR of its own block (sticky: the first give-up wins), sets
// the device-wide flag that b200amp_device_error() reads, and the kernel RETURNS without doing
// its work. Kernels that find ERROR already set return at once, so one rank that never shows up
// costs every other rank one wait limit, not one per kernel. Nothing traps and nothing spins
// for ever; the context stays usable. The reference has no multi-GPU code to mirror here.
#pragma once

#include "internal.cuh"

namespace b200amp
{

constexpr int MAX_RANKS = 8;

// word indices inside a block (B200AMP_ZERO1_SYNC_BYTES / 4 words)
constexpr int SYNC_PHASE_GRADS = 0;     // [0..7]   every rank's gradients are in its arena
constexpr int SYNC_PHASE_PAIRS = 1;     // [8..15]  rank q has written its {sum, flag} pair into every table
constexpr int SYNC_PHASE_WEIGHTS = 2;   // [16..23] rank q's fp16 weights have landed in every arena
constexpr int SYNC_EPOCH = 24;          // number of the last step this rank completed (only the owner writes it)
constexpr int SYNC_ERROR = 25;          // 0, or what a wait gave up on: (phase + 1) | missing rank << 8
constexpr int SYNC_STAMP = 26;          // the step in flight, written at its start: what a copy engine copies into
                                        // a peer's PIECE word after the data it announces
constexpr int SYNC_PIECE = 32;          // [32 + 8 p + q] piece p of rank q's gradients has landed in my staging rows
constexpr int SYNC_MAX_PIECES = 16;
constexpr int SYNC_PHASE_PIECE = 3;     // phase number recorded when a wait for a piece gives up
// Polls of one wait by default: several seconds (a poll costs 0.5 us at first, about 1 us once it sleeps
// 400 ns between loads). Long enough for the skew a healthy job shows (a rank
// that writes a checkpoint, a slow data loader), short enough that a rank that is gone is reported and not
// waited for; a caller that wants to know sooner passes its own limit.
constexpr unsigned SYNC_DEFAULT_LIMIT = 1u << 23;

// what a launch does with the block
constexpr int SYNC_ENTER_GRADS = 1;     // prologue: announce and await "gradients ready" (rs_pass1)
constexpr int SYNC_SIGNAL_PAIRS = 2;    // epilogue of the last CTA: announce "pairs written" (rs_pass1)
constexpr int SYNC_WAIT_PIECE = 4;      // prologue: await piece `piece` of every peer's pushed gradients

struct SyncArgs
{
    unsigned int *block[MAX_RANKS];     // block[r]: rank r's block as mapped in this process; block[0] == null: off
    int my_rank;
    int mode;
    int piece;
    unsigned int limit;
};

#ifdef __CUDACC__

// Set when a wait gave up. Only zero1.cu includes this header, so there is one copy; it is read
// (and cleared) through sync_timeout_take() below by b200amp_device_error().
static __device__ int g_sync_timeout = 0;

__device__ __forceinline__ unsigned int sync_load_acquire(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void sync_store_release(unsigned int *p, unsigned int v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" : : "l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned int sync_load_relaxed(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ bool sync_on(const SyncArgs &sy)
{
    return sy.block[0] != nullptr;
}

__device__ __forceinline__ unsigned int *sync_local(const SyncArgs &sy)
{
    return sy.block[sy.my_rank];
}

__device__ __forceinline__ bool sync_failed(const SyncArgs &sy)
{
    return sync_load_relaxed(sync_local(sy) + SYNC_ERROR) != 0;
}

// The number of the step in flight: one more than the number of the last completed step, and never
// 0 (the counter wraps from 2^32 - 1 to 1), so a word that is still zero from the set-up never
// matches a live step.
__device__ __forceinline__ unsigned int sync_epoch(const SyncArgs &sy)
{
    const unsigned int e = sync_load_relaxed(sync_local(sy) + SYNC_EPOCH) + 1u;
    return e != 0u ? e : 1u;
}

__device__ __forceinline__ void sync_give_up(const SyncArgs &sy, int phase, int missing_rank)
{
    atomicCAS(sync_local(sy) + SYNC_ERROR, 0u,
              static_cast<unsigned int>(phase + 1) | (static_cast<unsigned int>(missing_rank) << 8));
    g_sync_timeout = 1;
}

// "phase of step e is done here": one store into every rank's block (its own included).
__device__ __forceinline__ void sync_signal(const SyncArgs &sy, int phase, int to_rank, unsigned int e)
{
    sync_store_release(sy.block[to_rank] + phase * MAX_RANKS + sy.my_rank, e);
}

// Polls one word of the own block until it holds e. False when the limit ran out or another
// thread of this GPU has already given up. Equality is all the protocol needs: no rank can announce
// a phase of step e + 1 before every rank has left step e (its own step e ends with a wait for
// everybody's "weights landed" of step e), so a word never runs ahead of its reader; a stale or
// wrapped value simply does not match.
__device__ __forceinline__ bool sync_wait_word(const SyncArgs &sy, int index, unsigned int e)
{
    const unsigned int *word = sync_local(sy) + index;
    const unsigned int limit = sy.limit != 0 ? sy.limit : SYNC_DEFAULT_LIMIT;
    for (unsigned int tries = 0; tries < limit; tries++)
    {
        if (sync_load_acquire(word) == e)
        {
            return true;
        }
        if (tries >= 16)
        {
            __nanosleep(tries < 1024 ? 64 : 400);
        }
        if ((tries & 1023u) == 1023u && sync_failed(sy))
        {
            return false;
        }
    }
    return false;
}

__device__ __forceinline__ bool sync_wait(const SyncArgs &sy, int phase, int from_rank, unsigned int e)
{
    return sync_wait_word(sy, phase * MAX_RANKS + from_rank, e);
}

// Thread q: await piece sy.piece of rank q's pushed gradients (nothing to await from itself).
__device__ __forceinline__ bool sync_await_piece(const SyncArgs &sy, int q)
{
    if (sync_failed(sy))
    {
        return false;
    }
    if (q == sy.my_rank)
    {
        return true;
    }
    if (!sync_wait_word(sy, SYNC_PIECE + sy.piece * MAX_RANKS + q, sync_epoch(sy)))
    {
        sync_give_up(sy, SYNC_PHASE_PIECE, q);
        return false;
    }
    return true;
}

// Thread q < nranks of the calling warp/CTA: announce `phase` to rank q (if signal) and await it
// from rank q. Returns this thread's verdict; the caller combines the threads' verdicts.
__device__ __forceinline__ bool sync_exchange(const SyncArgs &sy, int phase, int q, bool signal, bool wait)
{
    if (sync_failed(sy))
    {
        return false;
    }
    const unsigned int e = sync_epoch(sy);
    if (signal)
    {
        sync_signal(sy, phase, q, e);
    }
    if (wait && !sync_wait(sy, phase, q, e))
    {
        sync_give_up(sy, phase, q);
        return false;
    }
    return true;
}

#endif // __CUDACC__

// host: *out = 1 if a wait gave up on the current device since the last call (clears the flag);
// synchronises the device.
#ifdef __CUDACC__
static inline int sync_timeout_take(int *out)
{
    int flag = 0;
    B200AMP_CUDA(cudaMemcpyFromSymbol(&flag, g_sync_timeout, sizeof(int)));
    if (flag != 0)
    {
        const int zero = 0;
        B200AMP_CUDA(cudaMemcpyToSymbol(g_sync_timeout, &zero, sizeof(int)));
    }
    *out = flag;
    return B200AMP_OK;
}
#endif

} // namespace b200amp
