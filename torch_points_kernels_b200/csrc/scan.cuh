// Tile scan shared by the brute-force search kernels (ball query, three_nn, kNN, chamfer).
//
// A CTA owns THREADS*Q query points (Q per thread, in registers) and streams the
// candidate cloud through shared memory in tiles of kScanTile points, double buffered:
// while the CTA works on tile t, every thread already holds the raw coordinates of its
// share of tile t+1 in registers (plain coalesced loads issued before the arithmetic).
//
// Two-level test per (query, candidate) pair:
//   1. filter:  |c|^2 - 2 q.c  <=  T          three fused multiply-adds and one compare,
//      evaluated two candidates at a time with the packed fma.rn.f32x2 of sm_100;
//      |c|^2 (slightly shrunk) is computed once per candidate when the tile is staged,
//      T = thr*(1+2^-17) - |q|^2*(1-2^-17) once per query (and again whenever the
//      query's threshold thr changes).  The slack of 2^-17 = 128 ulp relative to
//      |q|^2 + |c|^2 covers every rounding error of the expanded form, so a pair the exact
//      test accepts always passes the filter; the filter only removes work.
//   2. exact:   for the few pairs that pass, the op's own arithmetic, in the operation
//      order of the reference (so distances and decisions are bit-identical).
//
// Shared-memory tile layout: blocks of four candidates as x[4] y[4] z[4] w[4] (64 B), so
// a block is four 16-byte loads with the same address in every lane (broadcasts) and
// register pairs (x0,x1), (x2,x3) ... feed the packed instructions directly.
//
// The per-op rule is a functor:
//   float threshold(int q)            current admission threshold of query q (squared distance)
//   bool  inclusive()                 true: d2 <= thr admits, false: d2 < thr
//   bool  exact(int q, long long k, float cx, float cy, float cz)
//                                     run the exact test on candidate k (k < ncand is
//                                     guaranteed) and record it; return true if threshold(q) changed
//   bool  finished()                  true when this thread needs no further candidates
#pragma once

#include <math_constants.h>

#include "tpk_common.cuh"

namespace tpk
{

constexpr int kScanTile = 1024;
constexpr int kScanTileFloats = 4 * kScanTile;
constexpr float kFilterSlack = 7.62939453125e-06f;  // 2^-17
#ifndef TPK_SCAN_BATCH
#define TPK_SCAN_BATCH 2
#endif
constexpr int kScanBatch = TPK_SCAN_BATCH;  // blocks of four candidates per filter branch
constexpr int kPendCap = 8 * kScanBatch + 8;  // parked pairs per thread between two exact-test batches

__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ float lo_f32(unsigned long long v)
{
    return __uint_as_float(static_cast<uint32_t>(v));
}
__device__ __forceinline__ float hi_f32(unsigned long long v)
{
    return __uint_as_float(static_cast<uint32_t>(v >> 32));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c)
{
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Filter threshold of a query with squared norm q2 and exact threshold thr.
__device__ __forceinline__ float filter_threshold(float thr, float q2)
{
    const float t = __fmaf_rn(thr, 1.0f + kFilterSlack, -__fmul_rn(q2, 1.0f - kFilterSlack));
    // non-finite input: let everything through, the exact test decides
    return (t == t && fabsf(q2) < CUDART_INF_F) ? t : CUDART_INF_F;
}

// smem: 2 * kScanTileFloats floats, 16-byte aligned.  cand points at the first candidate
// of the range (any 4-byte alignment), ncand may be 0.  All threads of the CTA must call.
template <int THREADS, int Q, class Op>
__device__ __forceinline__ void scan_candidates(const float* __restrict__ cand, long long ncand,
                                                float* smem, const float (&qx)[Q],
                                                const float (&qy)[Q], const float (&qz)[Q], Op& op)
{
    static_assert(kScanTile % THREADS == 0, "every thread stages the same number of candidates");
    constexpr int PER = kScanTile / THREADS;  // candidates staged per thread per tile
    const int tid = threadIdx.x;
    const long long ntiles = (ncand + kScanTile - 1) / kScanTile;

    float raw[PER][3];
    auto fetch = [&](long long t) {
#pragma unroll
        for (int i = 0; i < PER; ++i)
        {
            const long long k = t * kScanTile + i * THREADS + tid;
            const bool ok = k < ncand;
            raw[i][0] = ok ? __ldg(cand + 3 * k + 0) : 0.f;
            raw[i][1] = ok ? __ldg(cand + 3 * k + 1) : 0.f;
            raw[i][2] = ok ? __ldg(cand + 3 * k + 2) : 0.f;
        }
    };
    auto stage = [&](long long t) {
        float* dst = smem + (t & 1) * kScanTileFloats;
#pragma unroll
        for (int i = 0; i < PER; ++i)
        {
            const int j = i * THREADS + tid;  // position in the tile
            const bool ok = t * kScanTile + j < ncand;
            const float x = raw[i][0], y = raw[i][1], z = raw[i][2];
            float w = __fmaf_rn(z, z, __fmaf_rn(y, y, __fmul_rn(x, x)));
            w = __fmul_rn(w, 1.0f - kFilterSlack);
            // slots past the end never pass (+inf); non-finite norms always pass (-inf)
            w = ok ? ((w == w && w < CUDART_INF_F) ? w : -CUDART_INF_F) : CUDART_INF_F;
            float* b = dst + (j >> 2) * 16 + (j & 3);
            b[0] = x;
            b[4] = y;
            b[8] = z;
            b[12] = w;
        }
    };

    // per-query filter constants
    unsigned long long m2x[Q], m2y[Q], m2z[Q];
    float q2[Q], T[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        m2x[q] = pack2(-2.0f * qx[q], -2.0f * qx[q]);
        m2y[q] = pack2(-2.0f * qy[q], -2.0f * qy[q]);
        m2z[q] = pack2(-2.0f * qz[q], -2.0f * qz[q]);
        q2[q] = __fmaf_rn(qz[q], qz[q], __fmaf_rn(qy[q], qy[q], __fmul_rn(qx[q], qx[q])));
        T[q] = filter_threshold(op.threshold(q), q2[q]);
    }

    // pairs that passed the filter and wait for the exact test: entry e of this thread at
    // [e * THREADS + tid].  An entry is (position << 1) | q in 16 bits, and one filter branch can
    // park 4 * kScanBatch * Q pairs before the next flush test: both only hold for these limits.
    static_assert(Q <= 2, "a parked entry keeps the query in one bit");
    static_assert(kScanBatch <= 2, "a parked entry keeps the tile position in 15 bits and a branch's pairs must fit");
    static_assert(kPendCap >= 4 * kScanBatch * Q + 8, "parked pairs of one branch must fit behind the flush threshold");
    __shared__ uint16_t s_pend[kPendCap * THREADS];
    uint16_t* pend = s_pend + tid;
    int npend = 0;
    bool done = op.finished();
    // Exact test of all parked pairs of the warp, every lane in its own (index) order.
    // Must be called by all lanes of the warp together.
    auto flush = [&](long long t) {
        const float* tile = smem + (t & 1) * kScanTileFloats;
        const int most = __reduce_max_sync(kFullMask, npend);
        for (int e = 0; e < most; ++e)
        {
            if (e < npend)
            {
                const uint32_t ent = pend[e * THREADS];
                const int j = static_cast<int>(ent >> 1);
                const long long k = t * kScanTile + j;
                if (k < ncand)
                {
                    const float* c = tile + (j >> 2) * 16 + (j & 3);
                    const float cx = c[0], cy = c[4], cz = c[8];
#pragma unroll
                    for (int q = 0; q < Q; ++q)
                    {
                        if (static_cast<int>(ent & 1u) == q && op.exact(q, k, cx, cy, cz))
                            T[q] = filter_threshold(op.threshold(q), q2[q]);
                    }
                }
            }
        }
        npend = 0;
        done = op.finished();
    };

    if (ntiles > 0)
    {
        fetch(0);
        stage(0);
    }
    __syncthreads();
    for (long long t = 0; t < ntiles; ++t)
    {
        const bool more = t + 1 < ntiles;
        if (more) fetch(t + 1);

        // each 16-byte load yields two packed candidate pairs, ready for fma.rn.f32x2
        const ulonglong2* s2 = reinterpret_cast<const ulonglong2*>(smem + (t & 1) * kScanTileFloats);
        for (int chunk = 0; chunk < kScanTile / 64; ++chunk)
        {
            if (__all_sync(kFullMask, done)) break;
            // kScanBatch blocks of four candidates per branch: independent FMA chains
            // for the scheduler, one vote for all of them
            for (int g0 = chunk * 16; g0 < chunk * 16 + 16; g0 += kScanBatch)
            {
                float a[Q][4 * kScanBatch];
                bool any = false;
#pragma unroll
                for (int u = 0; u < kScanBatch; ++u)
                {
                    const ulonglong2 X = s2[4 * (g0 + u) + 0];
                    const ulonglong2 Y = s2[4 * (g0 + u) + 1];
                    const ulonglong2 Z = s2[4 * (g0 + u) + 2];
                    const ulonglong2 W = s2[4 * (g0 + u) + 3];
#pragma unroll
                    for (int q = 0; q < Q; ++q)
                    {
                        const unsigned long long a01 = fma2(m2x[q], X.x, fma2(m2y[q], Y.x, fma2(m2z[q], Z.x, W.x)));
                        const unsigned long long a23 = fma2(m2x[q], X.y, fma2(m2y[q], Y.y, fma2(m2z[q], Z.y, W.y)));
                        a[q][4 * u + 0] = lo_f32(a01);
                        a[q][4 * u + 1] = hi_f32(a01);
                        a[q][4 * u + 2] = lo_f32(a23);
                        a[q][4 * u + 3] = hi_f32(a23);
                        any |= (a[q][4 * u + 0] <= T[q]) | (a[q][4 * u + 1] <= T[q]) |
                               (a[q][4 * u + 2] <= T[q]) | (a[q][4 * u + 3] <= T[q]);
                    }
                }
                // warp-uniform branch: every lane enters, so the votes inside are convergent
                if (__any_sync(kFullMask, any))
                {
                    // park the pairs that passed (tile position and query, in index order);
                    // they are examined in batches, with most lanes of the warp busy, instead
                    // of one at a time with one lane busy
#pragma unroll
                    for (int i = 0; i < 4 * kScanBatch; ++i)
                    {
#pragma unroll
                        for (int q = 0; q < Q; ++q)
                        {
                            if (a[q][i] <= T[q])
                            {
                                pend[npend * THREADS] = static_cast<uint16_t>(((4 * g0 + i) << 1) | q);
                                ++npend;
                            }
                        }
                    }
                    if (__any_sync(kFullMask, npend > kPendCap - 4 * kScanBatch * Q)) flush(t);
                }
            }
        }
        if (__any_sync(kFullMask, npend > 0)) flush(t);
        if (more) stage(t + 1);
        // one barrier per tile: it publishes tile t+1 and retires tile t, whose buffer is
        // only written again while staging tile t+2, after the next barrier
        if (__syncthreads_and(done)) break;
    }
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
