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
#include <math_constants.h>

#include "scan.cuh"

namespace tpk
{
// grid_query.cu
size_t grid_scratch_bytes(int b, int n, int m);
int grid_ball_query_dense(int b, int n, int m, float radius, int nsample, const float* new_xyz,
                          const float* xyz, int64_t* idx, float* dist, void* scratch,
                          const unsigned char** need_scan_out, cudaStream_t s);
// hash_grid.cu
bool hash_grid_fits(long long size_x, long long size_y);
size_t hash_grid_scratch_bytes(long long size_x, long long size_y);
int hash_grid_ball_query(long long size_x, long long size_y, float radius, int nsample, const float* x, const float* y,
                         const int64_t* batch_x, const int64_t* batch_y, int64_t* idx, float* dist, void* scratch,
                         const unsigned char** need_out, cudaStream_t s);
int hash_grid_ball_query_dense(int b, int n, int m, float radius, int nsample, const float* new_xyz, const float* xyz,
                               int64_t* idx, float* dist, void* scratch, const unsigned char** need_out, cudaStream_t s);
// smem_grid.cu
bool sg_ball_query_fits(int b, int n, int nsample);
int sg_ball_query(int b, int n, int m, float radius, int nsample, const float* new_xyz, const float* xyz,
                  int64_t* idx, float* dist, unsigned char* need, cudaStream_t s);

namespace
{

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
    long long idx_base;

    __device__ __forceinline__ bool open(int q) const { return act[q] && cnt[q] < nsample; }
    __device__ __forceinline__ float threshold(int q) const { return open(q) ? r2 : -CUDART_INF_F; }
    __device__ __forceinline__ bool finished() const
    {
        bool done = true;
#pragma unroll
        for (int q = 0; q < Q; ++q) done &= !open(q);
        return done;
    }
    __device__ __forceinline__ bool exact(int q, long long k, float cx, float cy, float cz)
    {
        if (!open(q)) return false;
        // dense: (centre - candidate), strict; partial: (candidate - centre), inclusive.
        // The sign changes none of the squares.
        const float d = PARTIAL ? sumsq_loop(cx - qx[q], cy - qy[q], cz - qz[q])
                                : sumsq_abc(qx[q] - cx, qy[q] - cy, qz[q] - cz);
        const bool hit = PARTIAL ? (d <= r2) : (d < r2);
        if (!hit) return false;
        const long long kk = k + idx_base;
        if (cnt[q] == 0) first[q] = kk;
        orow[q][cnt[q]] = kk;
        drow[q][cnt[q]] = d;
        ++cnt[q];
        return cnt[q] >= nsample;
    }
};

template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    ball_query_dense_kernel(int n, int m, int tiles_per_cloud, float radius, int nsample,
                            const float* __restrict__ new_xyz, const float* __restrict__ xyz,
                            int64_t* __restrict__ idx_out, float* __restrict__ dist_out,
                            const unsigned char* __restrict__ need)
{
    __shared__ __align__(16) float smem[2 * kScanTileFloats];
    const int cloud = blockIdx.x / tiles_per_cloud;
    const int qtile = blockIdx.x - cloud * tiles_per_cloud;
    const float* cand = xyz + static_cast<size_t>(cloud) * n * 3;

    BallOp<false, Q> op;
    op.r2 = __fmul_rn(radius, radius);
    op.nsample = nsample;
    op.idx_base = 0;
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        // `need` (optional): one byte per centre, 0 = already answered by the grid path
        op.act[q] = j < m && (need == nullptr || need[static_cast<size_t>(cloud) * m + j] != 0);
        op.cnt[q] = 0;
        op.first[q] = 0;
        const size_t row = static_cast<size_t>(cloud) * m + (op.act[q] ? j : 0);
        op.qx[q] = op.act[q] ? __ldg(new_xyz + row * 3 + 0) : 0.f;
        op.qy[q] = op.act[q] ? __ldg(new_xyz + row * 3 + 1) : 0.f;
        op.qz[q] = op.act[q] ? __ldg(new_xyz + row * 3 + 2) : 0.f;
        op.orow[q] = idx_out + row * nsample;
        op.drow[q] = dist_out + row * nsample;
    }

    if (need != nullptr)
    {
        // nothing left over for this CTA (the usual case behind the grid kernels): leave
        // before staging a single tile
        bool any = false;
#pragma unroll
        for (int q = 0; q < Q; ++q) any |= op.act[q];
        if (!__syncthreads_or(any ? 1 : 0)) return;
    }
    scan_candidates<THREADS, Q>(cand, n, smem, op.qx, op.qy, op.qz, op);

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
                              float* __restrict__ dist_out, const unsigned char* __restrict__ need)
{
    __shared__ __align__(16) float smem[2 * kScanTileFloats];
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
        // `need` (optional): one byte per centre, 0 = already answered by the grid path
        valid[q] = j < size_y && (need == nullptr || need[j] != 0);
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

    // sorted ids: the CTA's first centre still to be answered carries its smallest segment id
    long long first_valid = 0x7fffffffffffffffll;
#pragma unroll
    for (int q = 0; q < Q; ++q)
        if (valid[q]) first_valid = min(first_valid, j0 + q * THREADS + static_cast<long long>(threadIdx.x));
    {
        __shared__ unsigned long long s_first;
        if (threadIdx.x == 0) s_first = ~0ull;
        __syncthreads();
        if (first_valid != 0x7fffffffffffffffll) atomicMin(&s_first, static_cast<unsigned long long>(first_valid));
        __syncthreads();
        if (s_first == ~0ull) return;  // nothing left over for this CTA
        first_valid = static_cast<long long>(s_first);
    }
    int64_t cur = __ldg(batch_y + first_valid);
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
#pragma unroll
        for (int q = 0; q < Q; ++q)
        {
            op.act[q] = valid[q] && seg[q] == cur;
            // ids are compared as unsigned so that kNone is larger than any real id
            if (valid[q] && seg[q] > cur)
                atomicMin(&s_next, static_cast<unsigned long long>(seg[q]));
        }
        op.idx_base = lo;
        scan_candidates<THREADS, Q>(x + lo * 3, hi - lo, smem, op.qx, op.qy, op.qz, op);
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

// Launch shape for `queries` centres: two centres per thread only when there are
// enough of them to fill the GPU several times over, smaller CTAs for small problems.
void pick_shape(long long queries, int* threads, int* q)
{
    *q = queries >= 300000 ? 2 : 1;
    *threads = queries >= 32768 ? 128 : 64;
}

}  // namespace
}  // namespace tpk

#define TPK_BQ_DISPATCH(KERNEL, ...)                                                               \
    do                                                                                             \
    {                                                                                              \
        if (threads == 128 && q == 2)                                                              \
        {                                                                                          \
            prefer_max_shared(KERNEL<128, 2>);                                                     \
            count_launches(1), KERNEL<128, 2><<<g, 128, 0, s>>>(__VA_ARGS__);                                         \
        }                                                                                          \
        else if (threads == 128)                                                                   \
        {                                                                                          \
            prefer_max_shared(KERNEL<128, 1>);                                                     \
            count_launches(1), KERNEL<128, 1><<<g, 128, 0, s>>>(__VA_ARGS__);                                         \
        }                                                                                          \
        else if (q == 2)                                                                           \
        {                                                                                          \
            prefer_max_shared(KERNEL<64, 2>);                                                      \
            count_launches(1), KERNEL<64, 2><<<g, 64, 0, s>>>(__VA_ARGS__);                                           \
        }                                                                                          \
        else                                                                                       \
        {                                                                                          \
            prefer_max_shared(KERNEL<64, 1>);                                                      \
            count_launches(1), KERNEL<64, 1><<<g, 64, 0, s>>>(__VA_ARGS__);                                           \
        }                                                                                          \
    } while (0)

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
    int threads, q;
    pick_shape(static_cast<long long>(b) * m, &threads, &q);
    const int tiles = (m + threads * q - 1) / (threads * q);
    const long long grid = static_cast<long long>(b) * tiles;
    TPK_REQUIRE(grid < (1ll << 31), "ball_query_dense: too many centres");
    const dim3 g(static_cast<unsigned>(grid));
    const unsigned char* need = nullptr;
    TPK_BQ_DISPATCH(ball_query_dense_kernel, n, m, tiles, radius, nsample, new_xyz, xyz, idx, dist, need);
    return check_launch("ball_query_dense");
}

// the test hook "ball_query_global_grid" selects the grid in global memory where the
// shared-memory grid would be used
static bool use_smem_grid(int b, int n, int nsample)
{
    return tpk::sg_ball_query_fits(b, n, nsample) && !tpk::test_path("ball_query_global_grid");
}

// Clouds the shared-memory grid does not take (2^18 points and more): the hashed grid in
// global scratch.  The test hook "ball_query_global_grid" selects the older bounding-box grid in
// global memory instead of either.
static bool use_hash_grid(int b, int n, int m)
{
    return n >= 8192 && tpk::hash_grid_fits(static_cast<long long>(b) * n, static_cast<long long>(b) * m) &&
           !tpk::test_path("ball_query_global_grid");
}

extern "C" int64_t tpk_ball_query_dense_scratch_bytes(int b, int n, int m, int nsample)
{
    if (b <= 0 || m <= 0 || nsample <= 0) return 0;
    if (tpk::test_path("ball_query_scan")) return 0;  // test hook: the index-order scan alone
    // shared-memory grid: one flag per centre
    if (use_smem_grid(b, n, nsample)) return (static_cast<int64_t>(b) * m + 255) / 256 * 256;
    if (use_hash_grid(b, n, m))
        return static_cast<int64_t>(tpk::hash_grid_scratch_bytes(static_cast<long long>(b) * n, static_cast<long long>(b) * m));
    // the grid in global memory needs clouds worth binning and a hit list that fits shared memory
    if (n < 8192 || nsample > 128) return 0;
    return static_cast<int64_t>(tpk::grid_scratch_bytes(b, n, m));
}

extern "C" int tpk_ball_query_dense_ws(int b, int n, int m, float radius, int nsample,
                                       const float* new_xyz, const float* xyz, int64_t* idx,
                                       float* dist, void* scratch, int64_t scratch_bytes,
                                       void* stream)
{
    using namespace tpk;
    const int64_t want = tpk_ball_query_dense_scratch_bytes(b, n, m, nsample);
    if (want == 0 || scratch == nullptr)
        return tpk_ball_query_dense(b, n, m, radius, nsample, new_xyz, xyz, idx, dist, stream);
    if (scratch_bytes < want)
    {
        set_error("ball_query_dense: scratch of %lld bytes given, %lld needed",
                  static_cast<long long>(scratch_bytes), static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE(new_xyz && xyz && idx && dist, "ball_query_dense: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ball_query_dense: scratch must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned char* need = nullptr;
    int rc;
    if (use_smem_grid(b, n, nsample))
    {
        need = static_cast<const unsigned char*>(scratch);
        rc = sg_ball_query(b, n, m, radius, nsample, new_xyz, xyz, idx, dist, static_cast<unsigned char*>(scratch), s);
    }
    else if (use_hash_grid(b, n, m) && radius > 0.f && radius < 1.0e18f)
    {
        rc = hash_grid_ball_query_dense(b, n, m, radius, nsample, new_xyz, xyz, idx, dist, scratch, &need, s);
    }
    else if (use_hash_grid(b, n, m))
    {
        rc = TPK_OK;  // a radius without a grid: the scan answers every centre
    }
    else
    {
        rc = grid_ball_query_dense(b, n, m, radius, nsample, new_xyz, xyz, idx, dist, scratch, &need, s);
    }
    if (rc != TPK_OK) return rc;
    // centres the grid left over (dense neighbourhoods, degenerate clouds): index-order scan
    int threads, q;
    pick_shape(static_cast<long long>(b) * m, &threads, &q);
    const int tiles = (m + threads * q - 1) / (threads * q);
    const long long grid = static_cast<long long>(b) * tiles;
    TPK_REQUIRE(grid < (1ll << 31), "ball_query_dense: too many centres");
    const dim3 g(static_cast<unsigned>(grid));
    TPK_BQ_DISPATCH(ball_query_dense_kernel, n, m, tiles, radius, nsample, new_xyz, xyz, idx, dist, need);
    return check_launch("ball_query_dense");
}

static int launch_partial_scan(long long size_x, long long size_y, float radius, int nsample, const float* x,
                               const float* y, const int64_t* batch_x, const int64_t* batch_y, int64_t* idx,
                               float* dist, const unsigned char* need, cudaStream_t s)
{
    using namespace tpk;
    int threads, q;
    pick_shape(size_y, &threads, &q);
    const long long grid = (size_y + threads * q - 1) / (threads * q);
    TPK_REQUIRE(grid < (1ll << 31), "ball_query_partial_dense: too many centres");
    const dim3 g(static_cast<unsigned>(grid));
    TPK_BQ_DISPATCH(ball_query_partial_kernel, size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist, need);
    return check_launch("ball_query_partial_dense");
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
    return launch_partial_scan(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist, nullptr,
                               static_cast<cudaStream_t>(stream));
}

// the test hook "ball_query_scan" keeps packed queries on the scan
static bool partial_wants_grid(int64_t size_x, int64_t size_y, float radius)
{
    return tpk::hash_grid_fits(size_x, size_y) && radius > 0.f && radius < 1.0e18f &&
           !tpk::test_path("ball_query_scan");
}

extern "C" int64_t tpk_ball_query_partial_dense_scratch_bytes(int64_t size_x, int64_t size_y, float radius)
{
    if (!partial_wants_grid(size_x, size_y, radius)) return 0;
    return static_cast<int64_t>(tpk::hash_grid_scratch_bytes(size_x, size_y));
}

extern "C" int tpk_ball_query_partial_dense_ws(int64_t size_x, int64_t size_y, float radius, int nsample,
                                               const float* x, const float* y, const int64_t* batch_x,
                                               const int64_t* batch_y, int64_t* idx, float* dist, void* scratch,
                                               int64_t scratch_bytes, void* stream)
{
    using namespace tpk;
    const int64_t want = tpk_ball_query_partial_dense_scratch_bytes(size_x, size_y, radius);
    if (want == 0 || scratch == nullptr || nsample <= 0)
        return tpk_ball_query_partial_dense(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist, stream);
    if (scratch_bytes < want)
    {
        set_error("ball_query_partial_dense: scratch of %lld bytes given, %lld needed",
                  static_cast<long long>(scratch_bytes), static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE(x && y && batch_x && batch_y && idx && dist, "ball_query_partial_dense: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ball_query_partial_dense: scratch must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned char* need = nullptr;
    const int rc = hash_grid_ball_query(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist, scratch, &need, s);
    if (rc != TPK_OK) return rc;
    // queries the grid left over (crowded neighbourhoods, non-finite coordinates): index-order scan
    return launch_partial_scan(size_x, size_y, radius, nsample, x, y, batch_x, batch_y, idx, dist, need, s);
}
