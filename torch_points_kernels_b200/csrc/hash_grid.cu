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
#include <climits>
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
// inv_h_dev (optional): the reciprocal cell width in device memory, where an earlier kernel of the
// same call computed it (kNN, which has no radius to size the cells by).
template <bool FILL>
__global__ void __launch_bounds__(kHgThreads)
    hg_bin_kernel(long long size_x, long long per_cloud, float inv_h, const float* __restrict__ inv_h_dev, uint32_t mask,
                  const float* __restrict__ x, const int64_t* __restrict__ batch_x, int* __restrict__ counts,
                  float4* __restrict__ sorted, int* __restrict__ sorted_seg)
{
    const long long k = static_cast<long long>(blockIdx.x) * kHgThreads + threadIdx.x;
    if (k >= size_x) return;
    if (inv_h_dev != nullptr) inv_h = __ldg(inv_h_dev);
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


// ------------------------------------------------------------------ k nearest neighbours
//
// kNN on the same hashed grid.  There is no radius to size the cells by, so the call first
// measures the bounding box of all support points and picks a cell width that puts about
// max(k, 8) / 4 points into a cell of an average segment (hg_knn_params_kernel; the width
// stays in device memory, no host round trip).  A query (one warp) then examines the 27
// cells around its own cell, keeps the k best candidates in (distance, index) order in
// registers (slot s of the list in lane s & 31), and is done when the k-th best distance is
// no larger than the distance to the nearest face of the block it has searched; otherwise
// it searches the next shell of cells (up to kHgKnnMaxRing shells), and what is still open
// after that (sparse regions, segments with fewer than k points, coordinates that are not
// finite) is flagged for the scan kernel.  A candidate is taken only from the bucket of its
// own cell, so a bucket that two cells of the search hash to never yields a point twice.
// Distances use the arithmetic of the reference's kd-tree metric (sumsq_unfused).
constexpr int kHgKnnMaxRing = 3;  // shells beyond the first 3 x 3 x 3 block

struct HgKnnParams
{
    float inv_h, h;
    int box[6];  // ordered-int images of min x, y, z and max x, y, z
    int pad[8];
};

__device__ __forceinline__ int hg_ordered(float v)
{
    const int b = __float_as_int(v);
    return b >= 0 ? b : b ^ 0x7FFFFFFF;
}
__device__ __forceinline__ float hg_unordered(int o) { return __int_as_float(o >= 0 ? o : o ^ 0x7FFFFFFF); }

__global__ void hg_knn_init_kernel(HgKnnParams* prm)
{
    if (threadIdx.x < 3) prm->box[threadIdx.x] = INT_MAX;
    if (threadIdx.x >= 3 && threadIdx.x < 6) prm->box[threadIdx.x] = INT_MIN;
}

__global__ void __launch_bounds__(kHgThreads)
    hg_knn_bbox_kernel(long long size_x, const float* __restrict__ x, HgKnnParams* prm)
{
    __shared__ float s_lo[3][kHgWarps], s_hi[3][kHgWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float lo[3] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};
    float hi[3] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
    for (long long k = static_cast<long long>(blockIdx.x) * kHgThreads + threadIdx.x; k < size_x;
         k += static_cast<long long>(gridDim.x) * kHgThreads)
    {
        const float p[3] = {__ldg(x + 3 * k + 0), __ldg(x + 3 * k + 1), __ldg(x + 3 * k + 2)};
        if (!hg_finite(p[0], p[1], p[2])) continue;
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            lo[a] = fminf(lo[a], p[a]);
            hi[a] = fmaxf(hi[a], p[a]);
        }
    }
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
        {
            lo[a] = fminf(lo[a], __shfl_xor_sync(kFullMask, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(kFullMask, hi[a], o));
        }
        if (lane == 0)
        {
            s_lo[a][warp] = lo[a];
            s_hi[a][warp] = hi[a];
        }
    }
    __syncthreads();
    if (threadIdx.x < 3)
    {
        float l = s_lo[threadIdx.x][0], h = s_hi[threadIdx.x][0];
        for (int w = 1; w < kHgWarps; ++w)
        {
            l = fminf(l, s_lo[threadIdx.x][w]);
            h = fmaxf(h, s_hi[threadIdx.x][w]);
        }
        if (l <= h)
        {
            atomicMin(&prm->box[threadIdx.x], hg_ordered(l));
            atomicMax(&prm->box[3 + threadIdx.x], hg_ordered(h));
        }
    }
}

// Cell width from the mean density of a segment inside the common bounding box (segments of
// a packed batch usually share their coordinate range; where they do not, cells come out
// wider than needed, which costs candidates, not correctness).
__global__ void hg_knn_params_kernel(long long size_x, long long nclouds, int k, const int64_t* __restrict__ batch_x,
                                     HgKnnParams* prm)
{
    if (threadIdx.x != 0) return;
    float ext[3], longest = 0.f;
    for (int a = 0; a < 3; ++a)
    {
        ext[a] = prm->box[a] <= prm->box[3 + a] ? hg_unordered(prm->box[3 + a]) - hg_unordered(prm->box[a]) : 0.f;
        longest = fmaxf(longest, ext[a]);
    }
    if (!(longest > 0.f) || !(longest < 1.0e18f)) longest = 1.0f;
    float volume = 1.f;
    for (int a = 0; a < 3; ++a) volume *= fmaxf(ext[a], longest * 1.0e-3f);  // flat clouds still have a volume
    const long long nseg = batch_x ? __ldg(batch_x + size_x - 1) + 1 : nclouds;
    const float per_seg = static_cast<float>(size_x) / static_cast<float>(nseg > 0 ? nseg : 1);
    const float per_cell = static_cast<float>(k > 8 ? k : 8) * 0.25f;
    float h = cbrtf(volume * per_cell / fmaxf(per_seg, 1.f));
    h = fminf(fmaxf(h, longest * 1.0e-5f), longest);
    prm->h = h;
    prm->inv_h = 1.0f / h;
}

struct HgKnnWarpScratch
{
    int run_end[32];    // inclusive prefix of the bucket lengths of the cells in flight
    int run_shift[32];  // slot of candidate v of run r = run_shift[r] + v
    int run_cell[32];   // the run's cell, packed relative to the query's cell
};

// Sorted list of the best candidates, slot s in lane s & 31 (d0/i0: slots 0..31, d1/i1: 32..63).
// Inserts (nd, ni), the same in all lanes, dropping the last slot.
template <bool K32>
__device__ __forceinline__ void hg_knn_insert(float nd, int ni, int lane, float& d0, int& i0, float& d1, int& i1)
{
    const bool less0 = d0 < nd || (d0 == nd && i0 < ni);
    int pos = __popc(__ballot_sync(kFullMask, less0));
    const float u0d = __shfl_up_sync(kFullMask, d0, 1);
    const int u0i = __shfl_up_sync(kFullMask, i0, 1);
    if (!K32)
    {
        const bool less1 = d1 < nd || (d1 == nd && i1 < ni);
        pos += __popc(__ballot_sync(kFullMask, less1));
        const float last_d = __shfl_sync(kFullMask, d0, 31);
        const int last_i = __shfl_sync(kFullMask, i0, 31);
        const float u1d = __shfl_up_sync(kFullMask, d1, 1);
        const int u1i = __shfl_up_sync(kFullMask, i1, 1);
        const int s1 = lane + 32;
        if (s1 > pos)
        {
            d1 = lane == 0 ? last_d : u1d;
            i1 = lane == 0 ? last_i : u1i;
        }
        else if (s1 == pos)
        {
            d1 = nd;
            i1 = ni;
        }
    }
    if (lane > pos)
    {
        d0 = u0d;
        i0 = u0i;
    }
    else if (lane == pos)
    {
        d0 = nd;
        i0 = ni;
    }
}

template <bool DENSE, bool K32>
__global__ void __launch_bounds__(kHgThreads)
    hg_knn_kernel(long long size_q, long long per_cloud_s, long long per_cloud_q, int k, const HgKnnParams* __restrict__ prm,
                  uint32_t mask, const float* __restrict__ query, const int64_t* __restrict__ batch_q,
                  const int* __restrict__ counts, const float4* __restrict__ sorted, const int* __restrict__ sorted_seg,
                  int64_t* __restrict__ idx_out, float* __restrict__ dist_out, unsigned char* __restrict__ need)
{
    __shared__ HgKnnWarpScratch s_scr[kHgWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    HgKnnWarpScratch& ws = s_scr[warp];
    const float inv_h = __ldg(&prm->inv_h), h = __ldg(&prm->h);
    const long long nwarps_total = static_cast<long long>(gridDim.x) * kHgWarps;
    for (long long j = static_cast<long long>(blockIdx.x) * kHgWarps + warp; j < size_q; j += nwarps_total)
    {
        // the query is the same in all lanes: everything outside the candidate loop is warp-uniform
        const float qx = __ldg(query + 3 * j + 0), qy = __ldg(query + 3 * j + 1), qz = __ldg(query + 3 * j + 2);
        const int cx = hg_cell(qx, inv_h), cy = hg_cell(qy, inv_h), cz = hg_cell(qz, inv_h);
        if (!hg_finite(qx, qy, qz) || abs(cx) >= kHgCoordLimit - 8 || abs(cy) >= kHgCoordLimit - 8 ||
            abs(cz) >= kHgCoordLimit - 8)
        {
            if (lane == 0) need[j] = 1;
            continue;
        }
        const long long seg = DENSE ? j / per_cloud_q : __ldg(batch_q + j);
        float d0 = CUDART_INF_F, d1 = CUDART_INF_F;  // empty slots: (+inf, INT_MAX)
        int i0 = INT_MAX, i1 = INT_MAX;
        float kd = CUDART_INF_F;  // the k-th best so far
        int ki = INT_MAX;
        bool done = false;
        for (int ring = 0; ring <= kHgKnnMaxRing && !done; ++ring)
        {
            // ring 0: the 3 x 3 x 3 block; ring r >= 1: the shell of cells at Chebyshev distance r + 1
            const int rad = ring + 1, side = 2 * rad + 1;
            const int ncell = side * side * side;
            for (int t0 = 0; t0 < ncell; t0 += 32)
            {
                int t = t0 + lane;
                if (ring == 0) t = lane == 0 ? 13 : (lane <= 13 ? lane - 1 : lane);  // the query's own cell first
                const int ox = t % side - rad, oy = (t / side) % side - rad, oz = t / (side * side) - rad;
                const bool shell = t < ncell && (ring == 0 || max(max(abs(ox), abs(oy)), abs(oz)) == rad);
                int beg = 0, len = 0;
                if (shell)
                {
                    const uint32_t bkt = hg_bucket(seg, cx + ox, cy + oy, cz + oz, mask);
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
                if (total == 0) continue;
                __syncwarp();  // earlier reads of the scratch are done
                ws.run_end[lane] = incl;
                ws.run_shift[lane] = beg - (incl - len);
                ws.run_cell[lane] = ((ox + 8) << 8) | ((oy + 8) << 4) | (oz + 8);
                __syncwarp();
                for (int v0 = 0; v0 < total; v0 += 32)
                {
                    const int v = v0 + lane;
                    const bool valid = v < total;
                    int r = 0;
#pragma unroll
                    for (int q = 0; q < 31; ++q) r += ws.run_end[q] <= v ? 1 : 0;
                    const int p = valid ? ws.run_shift[r] + v : 0;
                    const float4 c = __ldg(sorted + p);
                    const float d = sumsq_unfused(qx - c.x, qy - c.y, qz - c.z);
                    const int ci = __float_as_int(c.w);
                    bool want = valid && d < CUDART_INF_F && (d < kd || (d == kd && ci < ki));
                    if (want)
                    {
                        // a candidate counts in the bucket of its own cell and segment only
                        const int rc = ws.run_cell[r];
                        want = __ldg(sorted_seg + p) == static_cast<int>(seg) &&
                               hg_cell(c.x, inv_h) == cx + ((rc >> 8) & 15) - 8 &&
                               hg_cell(c.y, inv_h) == cy + ((rc >> 4) & 15) - 8 && hg_cell(c.z, inv_h) == cz + (rc & 15) - 8;
                    }
                    uint32_t bal = __ballot_sync(kFullMask, want);
                    while (bal != 0u)
                    {
                        const int src = __ffs(bal) - 1;
                        bal &= bal - 1u;
                        const float nd = __shfl_sync(kFullMask, d, src);
                        const int ni = __shfl_sync(kFullMask, ci, src);
                        if (nd < kd || (nd == kd && ni < ki))
                        {
                            hg_knn_insert<K32>(nd, ni, lane, d0, i0, d1, i1);
                            const int ks = k - 1;
                            kd = __shfl_sync(kFullMask, (K32 || ks < 32) ? d0 : d1, ks & 31);
                            ki = __shfl_sync(kFullMask, (K32 || ks < 32) ? i0 : i1, ks & 31);
                        }
                    }
                }
            }
            // every point closer than the nearest face of the searched block has been seen
            const float fx = fminf(qx - static_cast<float>(cx - rad) * h, static_cast<float>(cx + rad + 1) * h - qx);
            const float fy = fminf(qy - static_cast<float>(cy - rad) * h, static_cast<float>(cy + rad + 1) * h - qy);
            const float fz = fminf(qz - static_cast<float>(cz - rad) * h, static_cast<float>(cz + rad + 1) * h - qz);
            const float reach = fminf(fminf(fx, fy), fz) * 0.9999f - (fabsf(qx) + fabsf(qy) + fabsf(qz) + h) * 2.0e-6f;
            done = reach > 0.f && kd <= reach * reach;
        }
        if (!done)
        {
            if (lane == 0) need[j] = 1;
            continue;
        }
        const long long base = DENSE ? seg * per_cloud_s : 0;  // dense indices are local to the cloud
        int64_t* orow = idx_out + j * k;
        float* drow = dist_out + j * k;
        if (lane < k)
        {
            orow[lane] = static_cast<int64_t>(i0) - base;
            drow[lane] = d0;
        }
        if (!K32 && lane + 32 < k)
        {
            orow[lane + 32] = static_cast<int64_t>(i1) - base;
            drow[lane + 32] = d1;
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
    count_launches(1), hg_bin_kernel<false><<<gp, kHgThreads, 0, s>>>(size_x, per_cloud_x, inv_h, nullptr, mask, x, batch_x, counts, sorted, sorted_seg);
    count_launches(1), hg_scan_blocks_kernel<<<nblocks, 1024, 0, s>>>(counts, ncount, totals);
    count_launches(1), hg_scan_totals_kernel<<<1, 1024, 0, s>>>(totals, nblocks);
    count_launches(1), hg_scan_add_kernel<<<nblocks, 1024, 0, s>>>(counts, ncount, totals);
    count_launches(1), hg_bin_kernel<true><<<gp, kHgThreads, 0, s>>>(size_x, per_cloud_x, inv_h, nullptr, mask, x, batch_x, counts, sorted, sorted_seg);
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

// ---- kNN on the hashed grid: scratch = parameters, then the ball query's layout
size_t hash_grid_knn_scratch_bytes(long long size_s, long long size_q)
{
    return 256 + hash_grid_scratch_bytes(size_s, size_q);
}

// Answers the queries the grid is good for; *need_out: one byte per query, 1 = left to the scan.
// Packed layout: batch_s / batch_q give the segments.  Dense layout (both NULL): size_s = b * n,
// size_q = b * m, per_cloud_s = n, per_cloud_q = m.
int hash_grid_knn(long long size_s, long long size_q, long long per_cloud_s, long long per_cloud_q, int k,
                  const float* support, const float* query, const int64_t* batch_s, const int64_t* batch_q, int64_t* idx,
                  float* dist2, void* scratch, const unsigned char** need_out, cudaStream_t s)
{
    const uint32_t h = hg_buckets(size_s);
    const uint32_t mask = h - 1u;
    const long long ncount = static_cast<long long>(h) + 1;
    const int nblocks = static_cast<int>((ncount + 1023) / 1024);
    unsigned char* p = static_cast<unsigned char*>(scratch);
    HgKnnParams* prm = reinterpret_cast<HgKnnParams*>(p);
    p += 256;
    int* counts = reinterpret_cast<int*>(p);
    p += hg_round((static_cast<size_t>(h) + 1) * sizeof(int));
    int* totals = reinterpret_cast<int*>(p);
    p += hg_round(static_cast<size_t>(nblocks) * sizeof(int));
    float4* sorted = reinterpret_cast<float4*>(p);
    p += hg_round(static_cast<size_t>(size_s) * sizeof(float4));
    int* sorted_seg = reinterpret_cast<int*>(p);
    p += hg_round(static_cast<size_t>(size_s) * sizeof(int));
    unsigned char* need = p;

    cudaError_t err = cudaMemsetAsync(counts, 0, (static_cast<size_t>(h) + 1) * sizeof(int), s);
    if (err != cudaSuccess)
    {
        set_error("knn hash grid: memset: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    const unsigned gp = static_cast<unsigned>((size_s + kHgThreads - 1) / kHgThreads);
    long long gb = (size_s + 8ll * kHgThreads - 1) / (8ll * kHgThreads);
    if (gb > 8ll * num_sms()) gb = 8ll * num_sms();
    const long long nclouds = per_cloud_s > 0 ? size_s / per_cloud_s : 1;
    count_launches(3);
    hg_knn_init_kernel<<<1, 32, 0, s>>>(prm);
    hg_knn_bbox_kernel<<<static_cast<unsigned>(gb), kHgThreads, 0, s>>>(size_s, support, prm);
    hg_knn_params_kernel<<<1, 32, 0, s>>>(size_s, nclouds, k, batch_s, prm);
    count_launches(1), hg_bin_kernel<false><<<gp, kHgThreads, 0, s>>>(size_s, per_cloud_s, 0.f, &prm->inv_h, mask, support, batch_s, counts, sorted, sorted_seg);
    count_launches(1), hg_scan_blocks_kernel<<<nblocks, 1024, 0, s>>>(counts, ncount, totals);
    count_launches(1), hg_scan_totals_kernel<<<1, 1024, 0, s>>>(totals, nblocks);
    count_launches(1), hg_scan_add_kernel<<<nblocks, 1024, 0, s>>>(counts, ncount, totals);
    count_launches(1), hg_bin_kernel<true><<<gp, kHgThreads, 0, s>>>(size_s, per_cloud_s, 0.f, &prm->inv_h, mask, support, batch_s, counts, sorted, sorted_seg);
    long long gq = (size_q + kHgWarps - 1) / kHgWarps;
    const long long cap = 32ll * num_sms();
    if (gq > cap) gq = cap;
    const unsigned g = static_cast<unsigned>(gq);
    count_launches(1);
#define TPK_HG_KNN(DENSE, K32)                                                                                          \
    prefer_max_shared(hg_knn_kernel<DENSE, K32>),                                                                       \
        hg_knn_kernel<DENSE, K32><<<g, kHgThreads, 0, s>>>(size_q, per_cloud_s, per_cloud_q, k, prm, mask, query, batch_q, \
                                                           counts, sorted, sorted_seg, idx, dist2, need)
    if (batch_q == nullptr)
    {
        if (k <= 32)
            TPK_HG_KNN(true, true);
        else
            TPK_HG_KNN(true, false);
    }
    else
    {
        if (k <= 32)
            TPK_HG_KNN(false, true);
        else
            TPK_HG_KNN(false, false);
    }
#undef TPK_HG_KNN
    *need_out = need;
    return check_launch("knn hash grid");
}

}  // namespace tpk
