// Tile scan shared by the brute-force search kernels (ball query, three_nn, kNN, chamfer).
//
// A CTA owns THREADS*Q query points (Q per thread, held in registers) and streams the
// candidate cloud through shared memory in tiles.  The candidate stream is the raw
// (x,y,z) float triples exactly as they lie in global memory, copied with cp.async
// into a double buffer, so the copy of tile t+1 overlaps the arithmetic on tile t.
// Four consecutive candidates are three 16-byte shared-memory loads, every lane
// reading the same address (a broadcast), which leaves the FP32 pipe as the only busy
// unit: per (query, candidate) pair 3 subtractions, 1 multiply, 2 fused multiply-adds
// and one compare.
//
// The per-op rule (radius test, top-3, top-k, arg-min) is a functor:
//   bool op.group(long long k0, const float (&cx)[4], const float (&cy)[4], const float (&cz)[4])
//        consumes candidates k0..k0+3 in index order (slots past the end of the range
//        hold kFarAway coordinates); returns true when this thread needs no further
//        candidates.
#pragma once

#include "tpk_common.cuh"

namespace tpk
{

// Padding coordinate for tile slots past the end of the candidate range: its squared
// distance to any finite query overflows to +inf, which passes no test.
constexpr float kFarAway = 1e30f;

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* gmem_src)
{
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int THREADS>
__device__ __forceinline__ void cta_sync()
{
    if (THREADS == 32)
        __syncwarp();
    else
        __syncthreads();
}

template <int THREADS>
__device__ __forceinline__ bool cta_all(bool pred)
{
    if (THREADS == 32) return __all_sync(kFullMask, pred);
    return __syncthreads_and(pred) != 0;
}

// smem: 2 * 3 * TILE floats, 16-byte aligned.  cand points at the first candidate of
// the range (any 4-byte alignment), ncand may be 0.  All threads of the CTA must call.
template <int THREADS, int TILE, class Op>
__device__ __forceinline__ void scan_candidates(const float* __restrict__ cand, long long ncand,
                                                float* smem, Op& op, bool thread_done)
{
    static_assert(TILE % 64 == 0, "tile must hold whole 64-candidate chunks");
    constexpr int kTileFloats = 3 * TILE;
    const int tid = threadIdx.x;
    const long long ntiles = (ncand + TILE - 1) / TILE;

    auto issue = [&](long long t) {
        float* dst = smem + (t & 1) * kTileFloats;
        const long long f0 = t * kTileFloats;
        long long valid = ncand * 3 - f0;
        if (valid > kTileFloats) valid = kTileFloats;
        const float* src = cand + f0;
#pragma unroll 4
        for (int i = tid; i < kTileFloats; i += THREADS)
        {
            if (i < valid)
                cp_async_f32(dst + i, src + i);
            else
                dst[i] = kFarAway;
        }
        cp_async_commit();
    };

    if (ntiles > 0) issue(0);
    for (long long t = 0; t < ntiles; ++t)
    {
        if (t + 1 < ntiles)
        {
            issue(t + 1);
            cp_async_wait<1>();
        }
        else
        {
            cp_async_wait<0>();
        }
        cta_sync<THREADS>();

        const float4* s4 = reinterpret_cast<const float4*>(smem + (t & 1) * kTileFloats);
        const long long kbase = t * TILE;
        for (int chunk = 0; chunk < TILE / 64; ++chunk)
        {
            if (__all_sync(kFullMask, thread_done)) break;
#pragma unroll 4
            for (int g = chunk * 16; g < chunk * 16 + 16; ++g)
            {
                const float4 a = s4[3 * g + 0];
                const float4 b = s4[3 * g + 1];
                const float4 c = s4[3 * g + 2];
                const float cx[4] = {a.x, a.w, b.z, c.y};
                const float cy[4] = {a.y, b.x, b.w, c.z};
                const float cz[4] = {a.z, b.y, c.x, c.w};
                if (op.group(kbase + 4 * g, cx, cy, cz)) thread_done = true;
            }
        }
        // also keeps the buffer just read from being overwritten by the copy of tile t+2
        if (cta_all<THREADS>(thread_done)) break;
    }
    // an early exit can leave the copy of the next tile in flight
    cp_async_wait<0>();
    cta_sync<THREADS>();
}

// First position in sorted ids[0..n) whose value is >= v (upper = false) or > v (upper = true).
__device__ __forceinline__ long long segment_bound(const int64_t* __restrict__ ids, long long n,
                                                   int64_t v, bool upper)
{
    long long lo = 0, hi = n;
    while (lo < hi)
    {
        const long long mid = (lo + hi) >> 1;
        const int64_t w = __ldg(ids + mid);
        if (upper ? (w <= v) : (w < v))
            lo = mid + 1;
        else
            hi = mid;
    }
    return lo;
}

}  // namespace tpk
