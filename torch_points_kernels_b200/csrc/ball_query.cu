// Ball query (radius search) for sm_100a: dense (B,N,3) clouds and packed segments.
//
// Brute force in candidate-index order, as the reference's rule demands ("the first
// nsample candidates within the radius"), but query-tiled: a CTA owns THREADS*Q centres
// and streams the candidates through shared memory (scan.cuh), stopping as soon as all
// of its centres are full.  Each thread writes the hits of its own centres as it meets
// them, so index order needs no sorting or compaction pass.
//
// dense   : cuda/src/ball_query_gpu.cu:9-52   d2 <  r^2, idx padded with the first hit
//                                             (0 if none), dist padded with -1
// partial : cuda/src/ball_query_gpu.cu:54-95  d2 <= r^2, idx and dist padded with -1,
//                                             idx = position in the packed x array
#include "scan.cuh"

namespace tpk
{
namespace
{

constexpr int kBqTile = 1024;
constexpr int kBqQ = 2;

template <bool PARTIAL, int Q>
struct BallOp
{
    float qx[Q], qy[Q], qz[Q];
    bool act[Q];
    int cnt[Q];
    long long first[Q];
    int64_t* orow[Q];
    float* drow[Q];
    float r2;
    int nsample;
    long long ncand;
    long long idx_base;

    __device__ __forceinline__ bool group(long long k0, const float (&cx)[4], const float (&cy)[4],
                                          const float (&cz)[4])
    {
        float d[Q][4];
        bool any = false;
#pragma unroll
        for (int q = 0; q < Q; ++q)
        {
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                // dense: (centre - candidate); partial: (candidate - centre).  The sign does
                // not change any of the squares.
                d[q][i] = PARTIAL ? sumsq_loop(cx[i] - qx[q], cy[i] - qy[q], cz[i] - qz[q])
                                  : sumsq_abc(qx[q] - cx[i], qy[q] - cy[i], qz[q] - cz[i]);
                any |= PARTIAL ? (d[q][i] <= r2) : (d[q][i] < r2);
            }
        }
        if (any)
        {
#pragma unroll
            for (int q = 0; q < Q; ++q)
            {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                {
                    const bool hit = PARTIAL ? (d[q][i] <= r2) : (d[q][i] < r2);
                    if (hit && act[q] && cnt[q] < nsample && k0 + i < ncand)
                    {
                        const long long k = k0 + i + idx_base;
                        if (cnt[q] == 0) first[q] = k;
                        orow[q][cnt[q]] = k;
                        drow[q][cnt[q]] = d[q][i];
                        ++cnt[q];
                    }
                }
            }
        }
        bool done = true;
#pragma unroll
        for (int q = 0; q < Q; ++q) done &= (!act[q] || cnt[q] >= nsample);
        return done;
    }
};

template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    ball_query_dense_kernel(int n, int m, int tiles_per_cloud, float radius, int nsample,
                            const float* __restrict__ new_xyz, const float* __restrict__ xyz,
                            int64_t* __restrict__ idx_out, float* __restrict__ dist_out)
{
    __shared__ __align__(16) float smem[2 * 3 * kBqTile];
    const int cloud = blockIdx.x / tiles_per_cloud;
    const int qtile = blockIdx.x - cloud * tiles_per_cloud;
    const float* cand = xyz + static_cast<size_t>(cloud) * n * 3;

    BallOp<false, Q> op;
    op.r2 = __fmul_rn(radius, radius);
    op.nsample = nsample;
    op.ncand = n;
    op.idx_base = 0;
    bool done = true;
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        op.act[q] = j < m;
        op.cnt[q] = 0;
        op.first[q] = 0;
        const size_t row = static_cast<size_t>(cloud) * m + (op.act[q] ? j : 0);
        op.qx[q] = op.act[q] ? __ldg(new_xyz + row * 3 + 0) : 0.f;
        op.qy[q] = op.act[q] ? __ldg(new_xyz + row * 3 + 1) : 0.f;
        op.qz[q] = op.act[q] ? __ldg(new_xyz + row * 3 + 2) : 0.f;
        op.orow[q] = idx_out + row * nsample;
        op.drow[q] = dist_out + row * nsample;
        done &= !op.act[q];
    }
    if (nsample <= 0) done = true;

    scan_candidates<THREADS, kBqTile>(cand, n, smem, op, done);

#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        if (!op.act[q]) continue;
        for (int s = op.cnt[q]; s < nsample; ++s)
        {
            op.orow[q][s] = op.first[q];
            op.drow[q][s] = -1.0f;
        }
    }
}

// One CTA per THREADS*Q consecutive centres of the packed y array.  The centres of a
// CTA usually share one segment; when they straddle several, the CTA walks the
// distinct segment ids in ascending order and scans each segment's candidates with
// only that segment's centres active.
template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    ball_query_partial_kernel(long long size_x, long long size_y, float radius, int nsample,
                              const float* __restrict__ x, const float* __restrict__ y,
                              const int64_t* __restrict__ batch_x,
                              const int64_t* __restrict__ batch_y, int64_t* __restrict__ idx_out,
                              float* __restrict__ dist_out)
{
    __shared__ __align__(16) float smem[2 * 3 * kBqTile];
    __shared__ long long s_range[2];
    __shared__ unsigned long long s_next;

    BallOp<true, Q> op;
    op.r2 = __fmul_rn(radius, radius);
    op.nsample = nsample;
    int64_t seg[Q];
    bool valid[Q];
    const long long j0 = static_cast<long long>(blockIdx.x) * (THREADS * Q);
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const long long j = j0 + q * THREADS + threadIdx.x;
        valid[q] = j < size_y;
        const long long row = valid[q] ? j : 0;
        seg[q] = valid[q] ? __ldg(batch_y + row) : 0;
        op.cnt[q] = 0;
        op.first[q] = -1;
        op.qx[q] = valid[q] ? __ldg(y + row * 3 + 0) : 0.f;
        op.qy[q] = valid[q] ? __ldg(y + row * 3 + 1) : 0.f;
        op.qz[q] = valid[q] ? __ldg(y + row * 3 + 2) : 0.f;
        op.orow[q] = idx_out + row * nsample;
        op.drow[q] = dist_out + row * nsample;
    }

    // sorted ids: the CTA's first centre carries its smallest segment id
    int64_t cur = __ldg(batch_y + j0);
    const unsigned long long kNone = ~0ull;
    while (true)
    {
        if (threadIdx.x == 0)
        {
            s_range[0] = segment_bound(batch_x, size_x, cur, false);
            s_range[1] = segment_bound(batch_x, size_x, cur, true);
            s_next = kNone;
        }
        __syncthreads();
        const long long lo = s_range[0], hi = s_range[1];
        bool done = true;
#pragma unroll
        for (int q = 0; q < Q; ++q)
        {
            op.act[q] = valid[q] && seg[q] == cur;
            done &= !op.act[q];
            // ids are compared as unsigned so that kNone is larger than any real id
            if (valid[q] && seg[q] > cur)
                atomicMin(&s_next, static_cast<unsigned long long>(seg[q]));
        }
        if (nsample <= 0) done = true;
        op.ncand = hi - lo;
        op.idx_base = lo;
        scan_candidates<THREADS, kBqTile>(x + lo * 3, hi - lo, smem, op, done);
        // scan_candidates ends with a CTA barrier: s_next is final here
        const unsigned long long nxt = s_next;
        __syncthreads();
        if (nxt == kNone) break;
        cur = static_cast<int64_t>(nxt);
    }

#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        if (!valid[q]) continue;
        for (int s = op.cnt[q]; s < nsample; ++s)
        {
            op.orow[q][s] = -1;
            op.drow[q][s] = -1.0f;
        }
    }
}

// Smallest CTA (in threads) that still gives every SM several CTAs to balance.
int pick_threads(long long queries, int q_per_thread)
{
    const long long want = 6ll * num_sms();
    if (queries / (128ll * q_per_thread) >= want) return 128;
    if (queries / (64ll * q_per_thread) >= want) return 64;
    return 32;
}

}  // namespace
}  // namespace tpk

extern "C" int tpk_ball_query_dense(int b, int n, int m, float radius, int nsample,
                                    const float* new_xyz, const float* xyz, int64_t* idx,
                                    float* dist, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0 && nsample >= 0,
                "ball_query_dense: negative size (b=%d n=%d m=%d nsample=%d)", b, n, m, nsample);
    if (b == 0 || m == 0 || nsample == 0) return TPK_OK;
    TPK_REQUIRE(new_xyz && idx && dist && (xyz || n == 0), "ball_query_dense: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int threads = pick_threads(static_cast<long long>(b) * m, kBqQ);
    const int tiles = (m + threads * kBqQ - 1) / (threads * kBqQ);
    const long long grid = static_cast<long long>(b) * tiles;
    TPK_REQUIRE(grid < (1ll << 31), "ball_query_dense: too many centres");
    const dim3 g(static_cast<unsigned>(grid));
    if (threads == 128)
        ball_query_dense_kernel<128, kBqQ><<<g, 128, 0, s>>>(n, m, tiles, radius, nsample, new_xyz, xyz, idx, dist);
    else if (threads == 64)
        ball_query_dense_kernel<64, kBqQ><<<g, 64, 0, s>>>(n, m, tiles, radius, nsample, new_xyz, xyz, idx, dist);
    else
        ball_query_dense_kernel<32, kBqQ><<<g, 32, 0, s>>>(n, m, tiles, radius, nsample, new_xyz, xyz, idx, dist);
    return check_launch("ball_query_dense");
}

extern "C" int tpk_ball_query_partial_dense(int64_t size_x, int64_t size_y, float radius,
                                            int nsample, const float* x, const float* y,
                                            const int64_t* batch_x, const int64_t* batch_y,
                                            int64_t* idx, float* dist, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(size_x >= 0 && size_y >= 0 && nsample >= 0,
                "ball_query_partial_dense: negative size");
    if (size_y == 0 || nsample == 0) return TPK_OK;
    TPK_REQUIRE(y && batch_y && idx && dist && ((x && batch_x) || size_x == 0),
                "ball_query_partial_dense: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int threads = pick_threads(size_y, kBqQ);
    const long long grid = (size_y + threads * kBqQ - 1) / (threads * kBqQ);
    TPK_REQUIRE(grid < (1ll << 31), "ball_query_partial_dense: too many centres");
    const dim3 g(static_cast<unsigned>(grid));
    if (threads == 128)
        ball_query_partial_kernel<128, kBqQ><<<g, 128, 0, s>>>(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist);
    else if (threads == 64)
        ball_query_partial_kernel<64, kBqQ><<<g, 64, 0, s>>>(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist);
    else
        ball_query_partial_kernel<32, kBqQ><<<g, 32, 0, s>>>(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist);
    return check_launch("ball_query_partial_dense");
}
