// Uniform-grid acceleration of the dense ball query (sm_100a).
//
// The brute-force kernel has to look at every candidate of a cloud for a centre with
// fewer than nsample neighbours.  Here each cloud is binned into a uniform grid whose
// cells are at least one radius wide, so all neighbours of a centre lie in the 27 cells
// around it.  The result must still be "the first nsample neighbours in index order":
// a centre collects the hits of its 27 cells in a list sorted by original index, capped
// at nsample entries (a larger index than the list's last never enters), and writes the
// list.  The distance test is the reference's exact arithmetic, so the set of hits - and
// with the index sort the whole output - is bit-identical to the scan.
//
// The grid only pays for centres with few candidates.  A centre inside a dense blob is
// cheaper for the scan, which stops at the nsample-th hit; such centres (and whole
// clouds whose bounding box is only a few radii wide, or holds non-finite coordinates)
// are flagged and left to the scan kernel, which runs right after on the flagged
// centres only.
//
// Pipeline (all on the caller's stream, no host synchronisation):
//   grid_setup  : bounding box, cell size, grid dimensions, zeroed cell counters (1 CTA per cloud)
//   grid_count  : points per cell (atomics)
//   grid_scan   : exclusive prefix sum of the counters (1 CTA per cloud)
//   grid_fill   : points copied cell by cell as (x, y, z, index)
//   grid_query  : one thread per centre
#include <math_constants.h>

#include "tpk_common.cuh"

namespace tpk
{

struct GridInfo
{
    float minx, miny, minz, inv_h;
    int dx, dy, dz, use;
};

constexpr int kGridMaxDim = 64;
constexpr int kGridThreads = 256;
constexpr int kGridQueryThreads = 128;

size_t grid_cells_capacity(int n)
{
    // about two points per cell, at most 64^3 cells
    int dim = 4;
    while (dim < kGridMaxDim && static_cast<long long>(dim + 1) * (dim + 1) * (dim + 1) * 2 <= n) ++dim;
    return static_cast<size_t>(dim) * dim * dim;
}

int grid_max_dim(int n)
{
    int dim = 4;
    while (dim < kGridMaxDim && static_cast<long long>(dim + 1) * (dim + 1) * (dim + 1) * 2 <= n) ++dim;
    return dim;
}

namespace
{

__device__ __forceinline__ int cell_coord(float v, float mn, float inv_h, int d)
{
    // monotone in v: the same function bins points and bounds a centre's cell range
    const float t = floorf(__fmul_rn(__fsub_rn(v, mn), inv_h));
    return max(0, min(d - 1, static_cast<int>(fminf(fmaxf(t, -1.0f), 1.0e6f))));
}

__global__ void __launch_bounds__(kGridThreads)
    grid_setup_kernel(int n, float radius, int max_dim, size_t cells_cap, const float* __restrict__ xyz_all,
                      GridInfo* __restrict__ info, int* __restrict__ cells_all)
{
    __shared__ float s_min[3][kGridThreads / 32], s_max[3][kGridThreads / 32];
    const int b = blockIdx.x;
    const float* xyz = xyz_all + static_cast<size_t>(b) * n * 3;
    float mn[3] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};
    float mx[3] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
    bool finite = true;
    for (int k = threadIdx.x; k < n; k += kGridThreads)
    {
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            const float v = __ldg(xyz + 3 * static_cast<size_t>(k) + a);
            finite &= fabsf(v) < 1.0e18f;  // false for inf and NaN too
            mn[a] = fminf(mn[a], v);
            mx[a] = fmaxf(mx[a], v);
        }
    }
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
        {
            mn[a] = fminf(mn[a], __shfl_xor_sync(kFullMask, mn[a], o));
            mx[a] = fmaxf(mx[a], __shfl_xor_sync(kFullMask, mx[a], o));
        }
        if ((threadIdx.x & 31) == 0)
        {
            s_min[a][threadIdx.x >> 5] = mn[a];
            s_max[a][threadIdx.x >> 5] = mx[a];
        }
    }
    const int all_finite = __syncthreads_and(finite ? 1 : 0);
    int* cells = cells_all + static_cast<size_t>(b) * (cells_cap + 1);
    for (size_t i = threadIdx.x; i <= cells_cap; i += kGridThreads) cells[i] = 0;
    if (threadIdx.x == 0)
    {
        GridInfo g;
        float lo[3], ext = 0.f, e[3];
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            float vmin = s_min[a][0], vmax = s_max[a][0];
            for (int w = 1; w < kGridThreads / 32; ++w)
            {
                vmin = fminf(vmin, s_min[a][w]);
                vmax = fmaxf(vmax, s_max[a][w]);
            }
            lo[a] = vmin;
            e[a] = vmax - vmin;
            ext = fmaxf(ext, e[a]);
        }
        // cells at least a (slightly enlarged) radius wide
        const float r1 = radius * 1.00001f + 1.0e-30f;
        const float h = fmaxf(r1, ext / static_cast<float>(max_dim));
        g.minx = lo[0];
        g.miny = lo[1];
        g.minz = lo[2];
        g.inv_h = 1.0f / h;
        g.dx = min(max_dim, static_cast<int>(e[0] * g.inv_h) + 1);
        g.dy = min(max_dim, static_cast<int>(e[1] * g.inv_h) + 1);
        g.dz = min(max_dim, static_cast<int>(e[2] * g.inv_h) + 1);
        const long long ncell = static_cast<long long>(g.dx) * g.dy * g.dz;
        g.use = (n > 0 && all_finite && radius > 0.f && radius < 1.0e18f && h > 0.f && h < CUDART_INF_F &&
                 ncell >= 64 && ncell <= static_cast<long long>(cells_cap))
                    ? 1
                    : 0;
        info[b] = g;
    }
}

__device__ __forceinline__ int cell_of(const GridInfo& g, float x, float y, float z)
{
    const int cx = cell_coord(x, g.minx, g.inv_h, g.dx);
    const int cy = cell_coord(y, g.miny, g.inv_h, g.dy);
    const int cz = cell_coord(z, g.minz, g.inv_h, g.dz);
    return (cz * g.dy + cy) * g.dx + cx;
}

// FILL == false: count points per cell (counter of cell c lives at cells[c + 1], so that the
// prefix sum leaves cells[c] = first slot of cell c).  FILL == true: copy the points.
template <bool FILL>
__global__ void __launch_bounds__(kGridThreads)
    grid_bin_kernel(int b, int n, size_t cells_cap, const float* __restrict__ xyz_all,
                    const GridInfo* __restrict__ info, int* __restrict__ cells_all,
                    float4* __restrict__ sorted_all)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGridThreads + threadIdx.x;
    if (t >= static_cast<long long>(b) * n) return;
    const int bi = static_cast<int>(t / n);
    const int k = static_cast<int>(t - static_cast<long long>(bi) * n);
    const GridInfo g = info[bi];
    if (!g.use) return;
    const float x = __ldg(xyz_all + 3 * t + 0), y = __ldg(xyz_all + 3 * t + 1), z = __ldg(xyz_all + 3 * t + 2);
    int* cells = cells_all + static_cast<size_t>(bi) * (cells_cap + 1);
    const int c = cell_of(g, x, y, z);
    if (!FILL)
        atomicAdd(cells + c + 1, 1);
    else
    {
        // the prefix sum left the first slot of cell c in cells[c + 1]; handing slots out
        // advances it to the cell's end, which is also the beginning of cell c + 1
        const int pos = atomicAdd(cells + c + 1, 1);
        sorted_all[static_cast<size_t>(bi) * n + pos] = make_float4(x, y, z, __int_as_float(k));
    }
}

// In place: cells[c + 1] (count of cell c) becomes the first slot of cell c; cells[0] = 0.
// After grid_bin_kernel<true> cells[c + 1] is the end of cell c and cells[c] its beginning.
__global__ void __launch_bounds__(1024)
    grid_scan_kernel(size_t cells_cap, const GridInfo* __restrict__ info, int* __restrict__ cells_all)
{
    __shared__ int s_warp[32];
    __shared__ int s_carry;
    const int b = blockIdx.x;
    const GridInfo g = info[b];
    if (!g.use) return;
    int* cells = cells_all + static_cast<size_t>(b) * (cells_cap + 1) + 1;
    const int ncell = g.dx * g.dy * g.dz;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < ncell; base += 1024)
    {
        const int i = base + threadIdx.x;
        const int v = i < ncell ? cells[i] : 0;
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
            s_warp[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int carry = s_carry;
        const int before = carry + (warp ? s_warp[warp - 1] : 0) + incl - v;  // exclusive prefix
        if (i < ncell) cells[i] = before;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = before + v;
        __syncthreads();
    }
}

// One thread per centre.  Sorted hit list (by original index) in shared memory: entry e of
// this thread at [e * THREADS + tid].
__global__ void __launch_bounds__(kGridQueryThreads)
    grid_query_kernel(int b, int n, int m, float radius, int nsample, float max_candidates, size_t cells_cap,
                      const float* __restrict__ new_xyz, const GridInfo* __restrict__ info,
                      const int* __restrict__ cells_all, const float4* __restrict__ sorted_all,
                      int64_t* __restrict__ idx_out, float* __restrict__ dist_out,
                      unsigned char* __restrict__ need_scan)
{
    extern __shared__ __align__(16) unsigned char lists_raw[];
    int* lidx = reinterpret_cast<int*>(lists_raw) + threadIdx.x;
    float* ldst = reinterpret_cast<float*>(lists_raw) + static_cast<size_t>(nsample) * kGridQueryThreads + threadIdx.x;
    const long long t = static_cast<long long>(blockIdx.x) * kGridQueryThreads + threadIdx.x;
    if (t >= static_cast<long long>(b) * m) return;
    const int bi = static_cast<int>(t / m);
    const GridInfo g = info[bi];
    if (!g.use)
    {
        need_scan[t] = 1;
        return;
    }
    const float qx = __ldg(new_xyz + 3 * t + 0), qy = __ldg(new_xyz + 3 * t + 1), qz = __ldg(new_xyz + 3 * t + 2);
    if (!(fabsf(qx) < 1.0e18f && fabsf(qy) < 1.0e18f && fabsf(qz) < 1.0e18f))
    {
        need_scan[t] = 1;
        return;
    }
    const float r1 = radius * 1.00001f + 1.0e-30f;
    const float r2 = __fmul_rn(radius, radius);
    const int* cells = cells_all + static_cast<size_t>(bi) * (cells_cap + 1);
    const float4* pts = sorted_all + static_cast<size_t>(bi) * n;
    // cell range of the ball, enlarged by the rounding of the exact test (1e-5 relative) and
    // of q +- r itself (2e-7 |q|); cell_coord is monotone, so every point the exact test can
    // accept lies in a cell of the range
    const float rx = r1 + fabsf(qx) * 2.0e-7f, ry = r1 + fabsf(qy) * 2.0e-7f, rz = r1 + fabsf(qz) * 2.0e-7f;
    const int x0 = cell_coord(qx - rx, g.minx, g.inv_h, g.dx), x1 = cell_coord(qx + rx, g.minx, g.inv_h, g.dx);
    const int y0 = cell_coord(qy - ry, g.miny, g.inv_h, g.dy), y1 = cell_coord(qy + ry, g.miny, g.inv_h, g.dy);
    const int z0 = cell_coord(qz - rz, g.minz, g.inv_h, g.dz), z1 = cell_coord(qz + rz, g.minz, g.inv_h, g.dz);

    int cnt = 0;
    {
        // candidates in the cell block; too many: the early-exit scan is cheaper
        float cand = 0.f;
        for (int cz = z0; cz <= z1; ++cz)
            for (int cy = y0; cy <= y1; ++cy)
            {
                const int row = (cz * g.dy + cy) * g.dx;
                cand += static_cast<float>(__ldg(cells + row + x1 + 1) - __ldg(cells + row + x0));
            }
        if (cand > max_candidates)
        {
            need_scan[t] = 1;
            return;
        }
        for (int cz = z0; cz <= z1; ++cz)
            for (int cy = y0; cy <= y1; ++cy)
            {
                const int row = (cz * g.dy + cy) * g.dx;
                const int beg = __ldg(cells + row + x0), end = __ldg(cells + row + x1 + 1);
                for (int p = beg; p < end; ++p)
                {
                    const float4 c = __ldg(pts + p);
                    const float d = sumsq_abc(qx - c.x, qy - c.y, qz - c.z);
                    if (d < r2)
                    {
                        const int k = __float_as_int(c.w);
                        if (cnt < nsample || k < lidx[(nsample - 1) * kGridQueryThreads])
                        {
                            int i = cnt < nsample ? cnt : nsample - 1;
                            for (; i > 0 && lidx[(i - 1) * kGridQueryThreads] > k; --i)
                            {
                                lidx[i * kGridQueryThreads] = lidx[(i - 1) * kGridQueryThreads];
                                ldst[i * kGridQueryThreads] = ldst[(i - 1) * kGridQueryThreads];
                            }
                            lidx[i * kGridQueryThreads] = k;
                            ldst[i * kGridQueryThreads] = d;
                            if (cnt < nsample) ++cnt;
                        }
                    }
                }
            }
    }
    need_scan[t] = 0;
    int64_t* orow = idx_out + t * nsample;
    float* drow = dist_out + t * nsample;
    const int first = cnt ? lidx[0] : 0;
    for (int s = 0; s < nsample; ++s)
    {
        orow[s] = s < cnt ? lidx[s * kGridQueryThreads] : first;
        drow[s] = s < cnt ? ldst[s * kGridQueryThreads] : -1.0f;
    }
}

// K (1 or 3) nearest known points per unknown point on the grid of the known cloud: search
// the 3x3x3 cell block around the query, then grow the block ring by ring until the K-th
// best squared distance is smaller than the squared distance to the nearest face of the
// block that still has cells behind it (or the block covers the grid).  Candidates are
// compared as (distance, index) pairs, which is the order the reference's index-ordered
// strict-'<' scans produce (three_nn: interpolate_gpu.cu:30-49; chamfer: chamfer_dist_gpu.cu:25-60).
// Output: K distances and K indices per unknown point.
template <int K>
__global__ void __launch_bounds__(kGridQueryThreads)
    grid_nn_kernel(int b, int n, int m, size_t cells_cap, const float* __restrict__ unknown,
                   const GridInfo* __restrict__ info, const int* __restrict__ cells_all,
                   const float4* __restrict__ sorted_all, float* __restrict__ dist2,
                   int32_t* __restrict__ idx, unsigned char* __restrict__ need_scan)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGridQueryThreads + threadIdx.x;
    if (t >= static_cast<long long>(b) * n) return;
    const int bi = static_cast<int>(t / n);
    const GridInfo g = info[bi];
    const float qx = __ldg(unknown + 3 * t + 0), qy = __ldg(unknown + 3 * t + 1), qz = __ldg(unknown + 3 * t + 2);
    if (!g.use || !(fabsf(qx) < 1.0e18f && fabsf(qy) < 1.0e18f && fabsf(qz) < 1.0e18f))
    {
        need_scan[t] = 1;
        return;
    }
    const int* cells = cells_all + static_cast<size_t>(bi) * (cells_cap + 1);
    const float4* pts = sorted_all + static_cast<size_t>(bi) * m;
    const float h = 1.0f / g.inv_h;
    const int cx = cell_coord(qx, g.minx, g.inv_h, g.dx);
    const int cy = cell_coord(qy, g.miny, g.inv_h, g.dy);
    const int cz = cell_coord(qz, g.minz, g.inv_h, g.dz);

    float b1 = CUDART_INF_F, b2 = CUDART_INF_F, b3 = CUDART_INF_F;
    int i1 = 0x7fffffff, i2 = 0x7fffffff, i3 = 0x7fffffff;
    int px0 = 0, px1 = -1, py0 = 0, py1 = -1, pz0 = 0, pz1 = -1;  // block already searched (empty)
    const int max_ring = max(g.dx, max(g.dy, g.dz));
    for (int ring = 1; ring <= max_ring; ++ring)
    {
        const int x0 = max(cx - ring, 0), x1 = min(cx + ring, g.dx - 1);
        const int y0 = max(cy - ring, 0), y1 = min(cy + ring, g.dy - 1);
        const int z0 = max(cz - ring, 0), z1 = min(cz + ring, g.dz - 1);
        for (int z = z0; z <= z1; ++z)
            for (int y = y0; y <= y1; ++y)
            {
                const bool inner_row = z >= pz0 && z <= pz1 && y >= py0 && y <= py1;
                const int row = (z * g.dy + y) * g.dx;
                // cells of this row not searched before: all of [x0,x1], or the two ends
                for (int part = 0; part < 2; ++part)
                {
                    int xa, xb;
                    if (!inner_row)
                    {
                        if (part == 1) break;
                        xa = x0;
                        xb = x1;
                    }
                    else if (part == 0)
                    {
                        xa = x0;
                        xb = px0 - 1;
                    }
                    else
                    {
                        xa = px1 + 1;
                        xb = x1;
                    }
                    if (xa > xb) continue;
                    const int beg = __ldg(cells + row + xa), end = __ldg(cells + row + xb + 1);
                    // Four candidates per step: the loads (L2) and distances are independent; a
                    // candidate that cannot beat the K-th best (one compare) costs nothing more,
                    // the others update the best list in order.
                    auto consider = [&](float d, int k) {
                        if (K == 1)
                        {
                            if (d < b1 || k < i1)  // reached only with d <= b1
                            {
                                b1 = d;
                                i1 = k;
                            }
                        }
                        else if (d < b3 || k < i3)  // reached only with d <= b3
                        {
                            if (d < b1 || (d == b1 && k < i1))
                            {
                                b3 = b2; i3 = i2;
                                b2 = b1; i2 = i1;
                                b1 = d;  i1 = k;
                            }
                            else if (d < b2 || (d == b2 && k < i2))
                            {
                                b3 = b2; i3 = i2;
                                b2 = d;  i2 = k;
                            }
                            else
                            {
                                b3 = d; i3 = k;
                            }
                        }
                    };
                    int p = beg;
                    for (; p + 4 <= end; p += 4)
                    {
                        float4 c[4];
                        float d[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) c[u] = __ldg(pts + p + u);
#pragma unroll
                        for (int u = 0; u < 4; ++u) d[u] = sumsq_abc(qx - c[u].x, qy - c[u].y, qz - c[u].z);
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (d[u] <= (K == 1 ? b1 : b3)) consider(d[u], __float_as_int(c[u].w));
                    }
                    for (; p < end; ++p)
                    {
                        const float4 c = __ldg(pts + p);
                        const float d = sumsq_abc(qx - c.x, qy - c.y, qz - c.z);
                        if (d <= (K == 1 ? b1 : b3)) consider(d, __float_as_int(c.w));
                    }
                }
            }
        px0 = x0; px1 = x1; py0 = y0; py1 = y1; pz0 = z0; pz1 = z1;
        const bool whole = x0 == 0 && y0 == 0 && z0 == 0 && x1 == g.dx - 1 && y1 == g.dy - 1 && z1 == g.dz - 1;
        if (whole) break;
        // distance to the nearest face of the block with unsearched cells behind it
        float rho = CUDART_INF_F;
        if (x0 > 0) rho = fminf(rho, qx - (g.minx + x0 * h));
        if (x1 < g.dx - 1) rho = fminf(rho, (g.minx + (x1 + 1) * h) - qx);
        if (y0 > 0) rho = fminf(rho, qy - (g.miny + y0 * h));
        if (y1 < g.dy - 1) rho = fminf(rho, (g.miny + (y1 + 1) * h) - qy);
        if (z0 > 0) rho = fminf(rho, qz - (g.minz + z0 * h));
        if (z1 < g.dz - 1) rho = fminf(rho, (g.minz + (z1 + 1) * h) - qz);
        // faces are computed in floating point and points near a face may be binned on either
        // side of it: take a margin of a thousandth of a cell plus the coordinate rounding
        rho -= 1.0e-3f * h + 4.0e-7f * (fabsf(qx) + fabsf(qy) + fabsf(qz) + fabsf(g.minx) + fabsf(g.miny) + fabsf(g.minz));
        const float kth = K == 1 ? b1 : b3;
        if (rho > 0.f && kth < rho * rho * 0.9999f) break;
    }
    need_scan[t] = 0;
    dist2[K * t + 0] = b1;
    idx[K * t + 0] = i1 == 0x7fffffff ? 0 : i1;
    if (K == 3)
    {
        dist2[3 * t + 1] = b2;
        dist2[3 * t + 2] = b3;
        idx[3 * t + 1] = i2 == 0x7fffffff ? 0 : i2;
        idx[3 * t + 2] = i3 == 0x7fffffff ? 0 : i3;
    }
}

}  // namespace

size_t grid_scratch_bytes(int b, int n, int m)
{
    const size_t cap = grid_cells_capacity(n);
    size_t bytes = 0;
    bytes += (static_cast<size_t>(b) * sizeof(GridInfo) + 255) / 256 * 256;
    bytes += (static_cast<size_t>(b) * (cap + 1) * sizeof(int) + 255) / 256 * 256;
    bytes += (static_cast<size_t>(b) * n * sizeof(float4) + 255) / 256 * 256;
    bytes += (static_cast<size_t>(b) * m + 255) / 256 * 256;
    return bytes;
}

// Builds the grids and answers the centres the grid is good for; *need_scan_out points at
// one byte per centre (1 = still to be answered by the scan kernel).
int grid_ball_query_dense(int b, int n, int m, float radius, int nsample, const float* new_xyz,
                          const float* xyz, int64_t* idx, float* dist, void* scratch,
                          const unsigned char** need_scan_out, cudaStream_t s)
{
    const size_t cap = grid_cells_capacity(n);
    unsigned char* p = static_cast<unsigned char*>(scratch);
    GridInfo* info = reinterpret_cast<GridInfo*>(p);
    p += (static_cast<size_t>(b) * sizeof(GridInfo) + 255) / 256 * 256;
    int* cells = reinterpret_cast<int*>(p);
    p += (static_cast<size_t>(b) * (cap + 1) * sizeof(int) + 255) / 256 * 256;
    float4* sorted = reinterpret_cast<float4*>(p);
    p += (static_cast<size_t>(b) * n * sizeof(float4) + 255) / 256 * 256;
    unsigned char* need = p;

    const long long npts = static_cast<long long>(b) * n;
    const unsigned gp = static_cast<unsigned>((npts + kGridThreads - 1) / kGridThreads);
    count_launches(1), grid_setup_kernel<<<b, kGridThreads, 0, s>>>(n, radius, grid_max_dim(n), cap, xyz, info, cells);
    count_launches(1), grid_bin_kernel<false><<<gp, kGridThreads, 0, s>>>(b, n, cap, xyz, info, cells, sorted);
    count_launches(1), grid_scan_kernel<<<b, 1024, 0, s>>>(cap, info, cells);
    count_launches(1), grid_bin_kernel<true><<<gp, kGridThreads, 0, s>>>(b, n, cap, xyz, info, cells, sorted);
    const size_t smem = static_cast<size_t>(nsample) * kGridQueryThreads * 8;
    auto qk = grid_query_kernel;
    prefer_max_shared(qk);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(qk, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("ball_query grid: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    // above this many candidates in a centre's cell block the early-exit scan is cheaper
    const float max_cand = 2.0f * sqrtf(6.45f * static_cast<float>(n) * static_cast<float>(nsample));
    const long long nq = static_cast<long long>(b) * m;
    const unsigned gq = static_cast<unsigned>((nq + kGridQueryThreads - 1) / kGridQueryThreads);
    count_launches(1), qk<<<gq, kGridQueryThreads, smem, s>>>(b, n, m, radius, nsample, max_cand, cap, new_xyz, info, cells, sorted, idx,
                                           dist, need);
    *need_scan_out = need;
    return check_launch("ball_query grid");
}

}  // namespace tpk

namespace tpk
{

// Grid of the `m` known points of every cloud; answers, with the k (1 or 3) nearest known
// points, the unknown points the grid is good for.
int grid_nn(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2,
            int32_t* idx, void* scratch, const unsigned char** need_scan_out, cudaStream_t s)
{
    const size_t cap = grid_cells_capacity(m);
    unsigned char* p = static_cast<unsigned char*>(scratch);
    GridInfo* info = reinterpret_cast<GridInfo*>(p);
    p += (static_cast<size_t>(b) * sizeof(GridInfo) + 255) / 256 * 256;
    int* cells = reinterpret_cast<int*>(p);
    p += (static_cast<size_t>(b) * (cap + 1) * sizeof(int) + 255) / 256 * 256;
    float4* sorted = reinterpret_cast<float4*>(p);
    p += (static_cast<size_t>(b) * m * sizeof(float4) + 255) / 256 * 256;
    unsigned char* need = p;

    const long long npts = static_cast<long long>(b) * m;
    const unsigned gp = static_cast<unsigned>((npts + kGridThreads - 1) / kGridThreads);
    // no radius here: cells as small as the capacity allows (radius argument just above zero)
    count_launches(1), grid_setup_kernel<<<b, kGridThreads, 0, s>>>(m, 1.0e-30f, grid_max_dim(m), cap, known, info, cells);
    count_launches(1), grid_bin_kernel<false><<<gp, kGridThreads, 0, s>>>(b, m, cap, known, info, cells, sorted);
    count_launches(1), grid_scan_kernel<<<b, 1024, 0, s>>>(cap, info, cells);
    count_launches(1), grid_bin_kernel<true><<<gp, kGridThreads, 0, s>>>(b, m, cap, known, info, cells, sorted);
    const long long nq = static_cast<long long>(b) * n;
    const unsigned gq = static_cast<unsigned>((nq + kGridQueryThreads - 1) / kGridQueryThreads);
    if (k == 1)
    {
        prefer_max_shared(grid_nn_kernel<1>);
        count_launches(1), grid_nn_kernel<1><<<gq, kGridQueryThreads, 0, s>>>(b, n, m, cap, unknown, info, cells, sorted, dist2, idx, need);
    }
    else
    {
        prefer_max_shared(grid_nn_kernel<3>);
        count_launches(1), grid_nn_kernel<3><<<gq, kGridQueryThreads, 0, s>>>(b, n, m, cap, unknown, info, cells, sorted, dist2, idx, need);
    }
    *need_scan_out = need;
    return check_launch("nearest neighbours on the grid");
}

int grid_three_nn(int b, int n, int m, const float* unknown, const float* known, float* dist2,
                  int32_t* idx, void* scratch, const unsigned char** need_scan_out, cudaStream_t s)
{
    return grid_nn(3, b, n, m, unknown, known, dist2, idx, scratch, need_scan_out, s);
}

// scratch for grid_nn: grid of m known points, one flag per unknown point
size_t grid_three_nn_scratch_bytes(int b, int n, int m) { return grid_scratch_bytes(b, m, n); }

}  // namespace tpk
