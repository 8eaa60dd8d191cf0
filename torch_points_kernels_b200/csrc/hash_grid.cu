// Ball query on a hashed uniform grid (sm_100a): the packed (partial_dense) layout, and dense
// clouds too large for the grids in shared memory.
//
// The packed layout holds many scenes of different sizes, each with its own extent, so
// there is no common bounding box to lay a grid over.  Points are instead binned by the
// hash of (segment id, cell coordinates) with cells one radius wide: a bucket holds the
// points of one cell, plus, rarely, those of other cells that hash to the same bucket;
// the exact test (same segment, squared distance <= r^2 in the reference's arithmetic,
// cuda/src/ball_query_gpu.cu:54-95) rejects the strangers.  A query looks at the 27
// buckets of the cells around it, one warp per query, 32 candidates at a time; a hit's
// output position is its rank by point index among the hits, so the first `nsample`
// neighbours in index order come out without a sort.  Queries the grid cannot answer
// (non-finite coordinates, too many candidates or hits) are flagged and left to the scan.
//
// Pipeline on the caller's stream: zero counters, count, prefix sum (three launches),
// fill, query.
#include <math_constants.h>

#include "tpk_common.cuh"

namespace tpk
{
namespace
{

constexpr int kHgThreads = 256;
constexpr int kHgWarps = kHgThreads / 32;
constexpr int kHgHitCap = 512;        // hits per query the buffer takes
constexpr int kHgCoordLimit = 1 << 20;

__device__ __forceinline__ int hg_cell(float v, float inv_h)
{
    const float t = floorf(__fmul_rn(v, inv_h));
    return static_cast<int>(fminf(fmaxf(t, -static_cast<float>(kHgCoordLimit)), static_cast<float>(kHgCoordLimit)));
}

__device__ __forceinline__ uint32_t hg_bucket(long long seg, int cx, int cy, int cz, uint32_t mask)
{
    uint32_t h = static_cast<uint32_t>(seg) * 0x9E3779B1u;
    h ^= static_cast<uint32_t>(cx) * 0x85EBCA77u;
    h = (h << 13) | (h >> 19);
    h ^= static_cast<uint32_t>(cy) * 0xC2B2AE3Du;
    h = (h << 13) | (h >> 19);
    h ^= static_cast<uint32_t>(cz) * 0x27D4EB2Fu;
    h ^= h >> 15;
    h *= 0x2C1B3C6Du;
    h ^= h >> 12;
    return h & mask;
}

__device__ __forceinline__ bool hg_finite(float x, float y, float z)
{
    return fabsf(x) < 1.0e18f && fabsf(y) < 1.0e18f && fabsf(z) < 1.0e18f;
}

// FILL == false: count points per bucket (counter of bucket c at counts[c + 1]);
// FILL == true: the prefix sum left the first slot of bucket c in counts[c + 1]; handing
// slots out advances it to the bucket's end, which is the beginning of bucket c + 1.
// Points with non-finite coordinates are not binned (no ball contains them).
template <bool FILL>
__global__ void __launch_bounds__(kHgThreads)
    hg_bin_kernel(long long size_x, long long per_cloud, float inv_h, uint32_t mask, const float* __restrict__ x,
                  const int64_t* __restrict__ batch_x, int* __restrict__ counts, float4* __restrict__ sorted,
                  int* __restrict__ sorted_seg)
{
    const long long k = static_cast<long long>(blockIdx.x) * kHgThreads + threadIdx.x;
    if (k >= size_x) return;
    const float px = __ldg(x + 3 * k + 0), py = __ldg(x + 3 * k + 1), pz = __ldg(x + 3 * k + 2);
    if (!hg_finite(px, py, pz)) return;
    // packed layout: the segment id of the point; dense layout (batch_x == NULL): its cloud
    const long long seg = batch_x ? __ldg(batch_x + k) : k / per_cloud;
    const uint32_t bkt = hg_bucket(seg, hg_cell(px, inv_h), hg_cell(py, inv_h), hg_cell(pz, inv_h), mask);
    const int pos = atomicAdd(counts + bkt + 1, 1);
    if (FILL)
    {
        sorted[pos] = make_float4(px, py, pz, __int_as_float(static_cast<int>(k)));
        sorted_seg[pos] = static_cast<int>(seg);
    }
}

// Exclusive prefix sum over data[0..n), three launches: per-block scan + block totals,
// scan of the totals (one block), add.
__global__ void __launch_bounds__(1024) hg_scan_blocks_kernel(int* __restrict__ data, long long n, int* __restrict__ totals)
{
    __shared__ int s_warp[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long i = static_cast<long long>(blockIdx.x) * 1024 + threadIdx.x;
    const int v = i < n ? data[i] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
    {
        const int t = __shfl_up_sync(kFullMask, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0)
    {
        int w = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            const int t = __shfl_up_sync(kFullMask, w, o);
            if (lane >= o) w += t;
        }
        s_warp[lane] = w;
    }
    __syncthreads();
    const int before = (warp ? s_warp[warp - 1] : 0) + incl - v;
    if (i < n) data[i] = before;
    if (threadIdx.x == 1023) totals[blockIdx.x] = before + v;
}

__global__ void __launch_bounds__(1024) hg_scan_totals_kernel(int* __restrict__ totals, int nblocks)
{
    __shared__ int s_warp[32];
    __shared__ int s_carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < nblocks; base += 1024)
    {
        const int i = base + threadIdx.x;
        const int v = i < nblocks ? totals[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            const int t = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0)
        {
            int w = s_warp[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1)
            {
                const int t = __shfl_up_sync(kFullMask, w, o);
                if (lane >= o) w += t;
            }
            s_warp[lane] = w;
        }
        __syncthreads();
        const int before = s_carry + (warp ? s_warp[warp - 1] : 0) + incl - v;
        if (i < nblocks) totals[i] = before;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = before + v;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(1024) hg_scan_add_kernel(int* __restrict__ data, long long n, const int* __restrict__ totals)
{
    const long long i = static_cast<long long>(blockIdx.x) * 1024 + threadIdx.x;
    if (i < n) data[i] += totals[blockIdx.x];
}

struct HgWarpScratch
{
    uint32_t hit_idx[kHgHitCap];  // original index of the hit
    int hit_pos[kHgHitCap];       // its slot in the sorted copy
    int run_end[32];              // inclusive prefix of the 27 bucket lengths
    int run_shift[32];            // slot of candidate v of run r = run_shift[r] + v
    int first;                    // dense layout: index of the first hit, repeated in unused slots
};

// DENSE: (b, n, 3) clouds and (b, m, 3) centres instead of packed segments: the segment of a
// query is its cloud, the test is the dense kernel's (strict, ball_query_gpu.cu:35-36),
// indices are local to the cloud and unused slots repeat the first hit.
template <bool DENSE>
__global__ void __launch_bounds__(kHgThreads)
    hg_query_kernel(long long size_y, long long per_cloud_x, long long per_cloud_y, float radius, int nsample, int max_candidates,
                    float inv_h, uint32_t mask,
                    const float* __restrict__ y, const int64_t* __restrict__ batch_y, const int* __restrict__ counts,
                    const float4* __restrict__ sorted, const int* __restrict__ sorted_seg,
                    int64_t* __restrict__ idx_out, float* __restrict__ dist_out, unsigned char* __restrict__ need)
{
    __shared__ HgWarpScratch s_scr[kHgWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    HgWarpScratch& ws = s_scr[warp];
    const float r2 = __fmul_rn(radius, radius);
    const long long nwarps_total = static_cast<long long>(gridDim.x) * kHgWarps;
    for (long long j = static_cast<long long>(blockIdx.x) * kHgWarps + warp; j < size_y; j += nwarps_total)
    {
        // the query is the same in all lanes: everything up to the candidate loop is warp-uniform
        const float qx = __ldg(y + 3 * j + 0), qy = __ldg(y + 3 * j + 1), qz = __ldg(y + 3 * j + 2);
        if (!hg_finite(qx, qy, qz))
        {
            if (lane == 0) need[j] = 1;
            continue;
        }
        const long long seg = DENSE ? j / per_cloud_y : __ldg(batch_y + j);
        // the ball, enlarged by the rounding of the exact test and of q +- r, must stay inside the
        // three cells per axis around the query's cell; it does unless q sits on a cell face
        const float pad = radius * 1.00001f + 1.0e-30f;
        const int cx = hg_cell(qx, inv_h), cy = hg_cell(qy, inv_h), cz = hg_cell(qz, inv_h);
        const float ex = pad + fabsf(qx) * 2.0e-7f, ey = pad + fabsf(qy) * 2.0e-7f, ez = pad + fabsf(qz) * 2.0e-7f;
        const bool inside = hg_cell(qx - ex, inv_h) >= cx - 1 && hg_cell(qx + ex, inv_h) <= cx + 1 &&
                            hg_cell(qy - ey, inv_h) >= cy - 1 && hg_cell(qy + ey, inv_h) <= cy + 1 &&
                            hg_cell(qz - ez, inv_h) >= cz - 1 && hg_cell(qz + ez, inv_h) <= cz + 1 &&
                            abs(cx) < kHgCoordLimit - 1 && abs(cy) < kHgCoordLimit - 1 && abs(cz) < kHgCoordLimit - 1;
        if (!inside)
        {
            if (lane == 0) need[j] = 1;
            continue;
        }
        // lane l < 27: bucket of neighbour cell l; a bucket reached through two cells counts once
        uint32_t bkt = 0xFFFFFFFFu - static_cast<uint32_t>(lane);  // distinct dummies for lanes 27..31
        if (lane < 27) bkt = hg_bucket(seg, cx + lane % 3 - 1, cy + (lane / 3) % 3 - 1, cz + lane / 9 - 1, mask);
        const uint32_t same = __match_any_sync(kFullMask, bkt);
        int beg = 0, len = 0;
        if (lane < 27 && (same & ((1u << lane) - 1u)) == 0u)
        {
            beg = __ldg(counts + bkt);
            len = __ldg(counts + bkt + 1) - beg;
        }
        int incl = len;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            const int v = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += v;
        }
        const int total = __shfl_sync(kFullMask, incl, 31);
        if (total > max_candidates)  // crowded: the scan, which stops at the nsample-th hit, is cheaper
        {
            if (lane == 0) need[j] = 1;
            continue;
        }
        __syncwarp();  // the previous query's reads of the scratch are done
        ws.run_end[lane] = incl;
        ws.run_shift[lane] = beg - (incl - len);
        __syncwarp();
        int nh = 0;
        for (int v0 = 0; v0 < total; v0 += 32)
        {
            const int v = v0 + lane;
            const bool valid = v < total;
            int r = 0;
#pragma unroll
            for (int k = 0; k < 26; ++k) r += ws.run_end[k] <= v ? 1 : 0;
            const int p = valid ? ws.run_shift[r] + v : 0;
            const float4 c = __ldg(sorted + p);
            const int cseg = __ldg(sorted_seg + p);
            // the packed kernel's arithmetic (ball_query_gpu.cu:78-82) and its inclusive test, or the dense one's
            const float d = DENSE ? sumsq_abc(qx - c.x, qy - c.y, qz - c.z) : sumsq_loop(qx - c.x, qy - c.y, qz - c.z);
            const bool hit = valid && cseg == static_cast<int>(seg) && (DENSE ? d < r2 : d <= r2);
            const uint32_t bal = __ballot_sync(kFullMask, hit);
            if (hit)
            {
                const int pos = nh + __popc(bal & ((1u << lane) - 1u));
                if (pos < kHgHitCap)
                {
                    ws.hit_idx[pos] = static_cast<uint32_t>(__float_as_int(c.w));
                    ws.hit_pos[pos] = p;
                }
            }
            nh += __popc(bal);
        }
        if (nh > kHgHitCap)
        {
            if (lane == 0) need[j] = 1;
            continue;
        }
        __syncwarp();
        int64_t* orow = idx_out + j * nsample;
        float* drow = dist_out + j * nsample;
        const long long base = DENSE ? seg * per_cloud_x : 0;  // dense indices are local to the cloud
        __syncwarp();
        for (int h0 = 0; h0 < nh; h0 += 32)
        {
            const int h = h0 + lane;
            if (h < nh)
            {
                const uint32_t e = ws.hit_idx[h];
                int rank = 0;
                for (int k = 0; k < nh; ++k) rank += ws.hit_idx[k] < e ? 1 : 0;
                if (rank < nsample)
                {
                    const float4 c = __ldg(sorted + ws.hit_pos[h]);
                    orow[rank] = static_cast<int64_t>(e) - base;
                    drow[rank] = DENSE ? sumsq_abc(qx - c.x, qy - c.y, qz - c.z) : sumsq_loop(qx - c.x, qy - c.y, qz - c.z);
                    if (rank == 0) ws.first = static_cast<int>(static_cast<long long>(e) - base);
                }
            }
        }
        __syncwarp();
        const int64_t fill = DENSE ? (nh ? static_cast<int64_t>(ws.first) : 0) : -1;
        for (int s = min(nh, nsample) + lane; s < nsample; s += 32)
        {
            orow[s] = fill;
            drow[s] = -1.0f;
        }
        if (lane == 0) need[j] = 0;
    }
}

size_t hg_round(size_t v) { return (v + 255) / 256 * 256; }

uint32_t hg_buckets(long long size_x)
{
    uint32_t h = 1024;
    while (h < (1u << 30) && static_cast<long long>(h) * 2 < size_x) h <<= 1;
    return h;  // a power of two, at least size_x / 2
}

}  // namespace

// Whether the hashed grid serves a packed problem (indices must fit 31 bits, one int per segment id).
bool hash_grid_fits(long long size_x, long long size_y)
{
    return size_x >= 4096 && size_x < (1ll << 31) && size_y > 0;
}

size_t hash_grid_scratch_bytes(long long size_x, long long size_y)
{
    const size_t h = hg_buckets(size_x);
    return hg_round((h + 1) * sizeof(int)) + hg_round(((h + 1 + 1023) / 1024) * sizeof(int)) +
           hg_round(static_cast<size_t>(size_x) * sizeof(float4)) + hg_round(static_cast<size_t>(size_x) * sizeof(int)) +
           hg_round(static_cast<size_t>(size_y));
}

// Answers the queries the grid is good for; *need_out: one byte per query, 1 = left to the scan.
// Packed layout: batch_x / batch_y give the segments.  Dense layout (both NULL): size_x = b * n,
// size_y = b * m, per_cloud_x = n, per_cloud_y = m.
static int hash_grid_run(long long size_x, long long size_y, long long per_cloud_x, long long per_cloud_y, float radius,
                         int nsample, const float* x, const float* y, const int64_t* batch_x, const int64_t* batch_y,
                         int64_t* idx, float* dist, void* scratch, const unsigned char** need_out, cudaStream_t s)
{
    const uint32_t h = hg_buckets(size_x);
    const uint32_t mask = h - 1u;
    const long long ncount = static_cast<long long>(h) + 1;
    const int nblocks = static_cast<int>((ncount + 1023) / 1024);
    unsigned char* p = static_cast<unsigned char*>(scratch);
    int* counts = reinterpret_cast<int*>(p);
    p += hg_round((static_cast<size_t>(h) + 1) * sizeof(int));
    int* totals = reinterpret_cast<int*>(p);
    p += hg_round(static_cast<size_t>(nblocks) * sizeof(int));
    float4* sorted = reinterpret_cast<float4*>(p);
    p += hg_round(static_cast<size_t>(size_x) * sizeof(float4));
    int* sorted_seg = reinterpret_cast<int*>(p);
    p += hg_round(static_cast<size_t>(size_x) * sizeof(int));
    unsigned char* need = p;

    // cells a shade wider than the radius: the ball never reaches past the neighbouring cells
    const float inv_h = 1.0f / (radius * 1.0001f);
    cudaError_t err = cudaMemsetAsync(counts, 0, (static_cast<size_t>(h) + 1) * sizeof(int), s);
    if (err != cudaSuccess)
    {
        set_error("ball_query hash grid: memset: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    const unsigned gp = static_cast<unsigned>((size_x + kHgThreads - 1) / kHgThreads);
    count_launches(1), hg_bin_kernel<false><<<gp, kHgThreads, 0, s>>>(size_x, per_cloud_x, inv_h, mask, x, batch_x, counts, sorted, sorted_seg);
    count_launches(1), hg_scan_blocks_kernel<<<nblocks, 1024, 0, s>>>(counts, ncount, totals);
    count_launches(1), hg_scan_totals_kernel<<<1, 1024, 0, s>>>(totals, nblocks);
    count_launches(1), hg_scan_add_kernel<<<nblocks, 1024, 0, s>>>(counts, ncount, totals);
    count_launches(1), hg_bin_kernel<true><<<gp, kHgThreads, 0, s>>>(size_x, per_cloud_x, inv_h, mask, x, batch_x, counts, sorted, sorted_seg);
    // above this many candidates around a query the early-exit scan is cheaper (the rule of the
    // other grids for dense clouds; packed segments have no common size)
    int max_cand = 16384;
    if (batch_y == nullptr)
    {
        const double v = 2.0 * sqrt(6.45 * static_cast<double>(per_cloud_x) * nsample);
        max_cand = v < 4096.0 ? 4096 : (v > 1.0e6 ? 1000000 : static_cast<int>(v));
    }
    long long gq = (size_y + kHgWarps - 1) / kHgWarps;
    const long long cap = 32ll * num_sms();
    if (gq > cap) gq = cap;
    if (batch_y == nullptr)
    {
        prefer_max_shared(hg_query_kernel<true>);
        count_launches(1), hg_query_kernel<true><<<static_cast<unsigned>(gq), kHgThreads, 0, s>>>(
            size_y, per_cloud_x, per_cloud_y, radius, nsample, max_cand, inv_h, mask, y, batch_y, counts, sorted, sorted_seg, idx, dist, need);
    }
    else
    {
        prefer_max_shared(hg_query_kernel<false>);
        count_launches(1), hg_query_kernel<false><<<static_cast<unsigned>(gq), kHgThreads, 0, s>>>(
            size_y, per_cloud_x, per_cloud_y, radius, nsample, max_cand, inv_h, mask, y, batch_y, counts, sorted, sorted_seg, idx, dist, need);
    }
    *need_out = need;
    return check_launch("ball_query hash grid");
}

int hash_grid_ball_query(long long size_x, long long size_y, float radius, int nsample, const float* x, const float* y,
                         const int64_t* batch_x, const int64_t* batch_y, int64_t* idx, float* dist, void* scratch,
                         const unsigned char** need_out, cudaStream_t s)
{
    return hash_grid_run(size_x, size_y, 1, 1, radius, nsample, x, y, batch_x, batch_y, idx, dist, scratch, need_out, s);
}

// Dense clouds (b, n, 3) / centres (b, m, 3) on the hashed grid (for clouds too large for the
// grids in shared memory).
int hash_grid_ball_query_dense(int b, int n, int m, float radius, int nsample, const float* new_xyz, const float* xyz,
                               int64_t* idx, float* dist, void* scratch, const unsigned char** need_out, cudaStream_t s)
{
    return hash_grid_run(static_cast<long long>(b) * n, static_cast<long long>(b) * m, n, m, radius, nsample, xyz, new_xyz,
                         nullptr, nullptr, idx, dist, scratch, need_out, s);
}

}  // namespace tpk
