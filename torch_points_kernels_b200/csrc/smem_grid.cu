// Uniform-grid search with the grid in shared memory (sm_100a).
//
// The global-memory grid kernels of grid_query.cu spend their time waiting: a query walks
// its cells with one dependent L2 access after the other.  Here a CTA builds the part of
// the grid its queries need in shared memory and then answers them from there, in one
// launch and without grid scratch:
//
//   three_nn   : every CTA of a cloud bins all known points (at most kSgMaxPoints) and
//                answers a contiguous chunk of the unknown points;
//   ball query : CTA `part` of a cloud owns the centres of one z-layer of cells, bins the
//                points of that layer and its two neighbours, collects the layer's
//                centres in a list and answers them.
//
// Every CTA recomputes the cloud's bounding box and bins from the raw coordinates (they
// come out of L2; the passes are a few microseconds).  Results are bit-identical to the
// brute-force kernels: the exact tests use the reference's arithmetic, three_nn orders
// candidates by (distance, index), the ball query keeps the nsample lowest indices.
// Queries a CTA cannot answer (non-finite coordinates, more staged points than fit,
// neighbourhoods so crowded that the early-exit scan is cheaper) are flagged in a byte
// array and left to the scan kernels, which run right after on the flagged queries only.
#include <math_constants.h>

#include "tpk_common.cuh"

namespace tpk
{

size_t grid_cells_capacity(int n);  // grid_query.cu
int grid_max_dim(int n);


namespace
{

constexpr int kSgThreads = 512;
constexpr int kSgMaxPoints = 8192;       // three_nn: known points per cloud
constexpr size_t kSgSmemBudget = 200 * 1024;
constexpr int kSgSlotBits = 14;          // ball query: staged points per CTA < 2^14
constexpr int kSgQueryChunk = 1024;      // ball query: centres examined per list pass

struct SgGrid
{
    float minx, miny, minz, inv_h, h;
    int dx, dy, dz;
    bool ok;
};

__device__ __forceinline__ int sg_cell_coord(float v, float mn, float inv_h, int d)
{
    // monotone in v: the same function bins points and bounds a query's cell range
    const float t = floorf(__fmul_rn(__fsub_rn(v, mn), inv_h));
    return max(0, min(d - 1, static_cast<int>(fminf(fmaxf(t, -1.0f), 1.0e6f))));
}

// Calls f(k, x, y, z) for the points k = this thread's share of the cloud.  Four points per
// step from three 16-byte loads when the cloud is 16-byte aligned and n a multiple of four.
template <class F>
__device__ __forceinline__ void sg_for_points(const float* __restrict__ xyz, int n, F&& f)
{
    if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(xyz) & 15u) == 0)
    {
        const float4* v = reinterpret_cast<const float4*>(xyz);
#pragma unroll 2
        for (int gi = threadIdx.x; gi < (n >> 2); gi += kSgThreads)
        {
            const float4 a = __ldg(v + 3 * gi), b = __ldg(v + 3 * gi + 1), c = __ldg(v + 3 * gi + 2);
            f(4 * gi + 0, a.x, a.y, a.z);
            f(4 * gi + 1, a.w, b.x, b.y);
            f(4 * gi + 2, b.z, b.w, c.x);
            f(4 * gi + 3, c.y, c.z, c.w);
        }
    }
    else
    {
        for (int k = threadIdx.x; k < n; k += kSgThreads)
            f(k, __ldg(xyz + 3 * static_cast<size_t>(k) + 0), __ldg(xyz + 3 * static_cast<size_t>(k) + 1),
              __ldg(xyz + 3 * static_cast<size_t>(k) + 2));
    }
}

// Bounding box of a cloud and the grid over it: cells at least `min_h` wide, at most
// max_dim per axis.  Every thread of the CTA returns the same struct.
__device__ __forceinline__ SgGrid sg_make_grid(const float* __restrict__ xyz, int n, float min_h, int max_dim, size_t cells_cap)
{
    __shared__ float s_min[3][kSgThreads / 32], s_max[3][kSgThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mn[3] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};
    float mx[3] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
    bool finite = true;
    sg_for_points(xyz, n, [&](int, float x, float y, float z) {
        finite &= fabsf(x) < 1.0e18f && fabsf(y) < 1.0e18f && fabsf(z) < 1.0e18f;  // false for inf and NaN too
        mn[0] = fminf(mn[0], x);
        mx[0] = fmaxf(mx[0], x);
        mn[1] = fminf(mn[1], y);
        mx[1] = fmaxf(mx[1], y);
        mn[2] = fminf(mn[2], z);
        mx[2] = fmaxf(mx[2], z);
    });
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
        {
            mn[a] = fminf(mn[a], __shfl_xor_sync(kFullMask, mn[a], o));
            mx[a] = fmaxf(mx[a], __shfl_xor_sync(kFullMask, mx[a], o));
        }
        if (lane == 0)
        {
            s_min[a][warp] = mn[a];
            s_max[a][warp] = mx[a];
        }
    }
    const int all_finite = __syncthreads_and(finite ? 1 : 0);
    SgGrid g;
    float lo[3], e[3], ext = 0.f;
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
        float vmin = s_min[a][0], vmax = s_max[a][0];
        for (int w = 1; w < kSgThreads / 32; ++w)
        {
            vmin = fminf(vmin, s_min[a][w]);
            vmax = fmaxf(vmax, s_max[a][w]);
        }
        lo[a] = vmin;
        e[a] = vmax - vmin;
        ext = fmaxf(ext, e[a]);
    }
    g.h = fmaxf(min_h, ext / static_cast<float>(max_dim));
    g.minx = lo[0];
    g.miny = lo[1];
    g.minz = lo[2];
    g.inv_h = 1.0f / g.h;
    g.dx = min(max_dim, static_cast<int>(e[0] * g.inv_h) + 1);
    g.dy = min(max_dim, static_cast<int>(e[1] * g.inv_h) + 1);
    g.dz = min(max_dim, static_cast<int>(e[2] * g.inv_h) + 1);
    const long long ncell = static_cast<long long>(g.dx) * g.dy * g.dz;
    g.ok = n > 0 && all_finite && g.h > 0.f && g.h < CUDART_INF_F && ncell <= static_cast<long long>(cells_cap);
    __syncthreads();  // the reduction buffers may be reused by the next call
    return g;
}

// Exclusive prefix sum in place over a[0..len) in shared memory; returns the total.
__device__ __forceinline__ int sg_block_scan(int* a, int len)
{
    __shared__ int s_warp[kSgThreads / 32];
    __shared__ int s_carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < len; base += kSgThreads)
    {
        const int i = base + tid;
        const int v = i < len ? a[i] : 0;
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
            int w = lane < kSgThreads / 32 ? s_warp[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1)
            {
                const int t = __shfl_up_sync(kFullMask, w, o);
                if (lane >= o) w += t;
            }
            if (lane < kSgThreads / 32) s_warp[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int before = s_carry + (warp ? s_warp[warp - 1] : 0) + incl - v;
        if (i < len) a[i] = before;
        __syncthreads();
        if (tid == kSgThreads - 1) s_carry = before + v;
        __syncthreads();
    }
    return s_carry;
}

// Bins the points whose z cell lies in [za, zb] into shared memory: cells[c] .. cells[c+1]
// is the run of local cell c = ((cz - za) * dy + cy) * dx + cx in spts, entries
// (x, y, z, original index).  Returns the number of staged points, or -1 if they exceed
// `pcap` (nothing usable is left in spts then).
__device__ __forceinline__ int sg_bin(const float* __restrict__ xyz, int n, const SgGrid& g, int za, int zb, int* cells,
                      float4* spts, int pcap)
{
    const int tid = threadIdx.x;
    const int ncell = (zb - za + 1) * g.dy * g.dx;
    for (int c = tid; c <= ncell; c += kSgThreads) cells[c] = 0;
    __syncthreads();
    sg_for_points(xyz, n, [&](int, float x, float y, float z) {
        const int cz = sg_cell_coord(z, g.minz, g.inv_h, g.dz);
        if (cz < za || cz > zb) return;
        const int cy = sg_cell_coord(y, g.miny, g.inv_h, g.dy);
        const int cx = sg_cell_coord(x, g.minx, g.inv_h, g.dx);
        atomicAdd(&cells[((cz - za) * g.dy + cy) * g.dx + cx + 1], 1);
    });
    __syncthreads();
    const int total = sg_block_scan(cells + 1, ncell);
    if (total > pcap) return -1;
    sg_for_points(xyz, n, [&](int k, float x, float y, float z) {
        const int cz = sg_cell_coord(z, g.minz, g.inv_h, g.dz);
        if (cz < za || cz > zb) return;
        const int cy = sg_cell_coord(y, g.miny, g.inv_h, g.dy);
        const int cx = sg_cell_coord(x, g.minx, g.inv_h, g.dx);
        // the scan left the first slot of cell c in cells[c + 1]; handing slots out advances
        // it to the end of the cell, which is the beginning of cell c + 1
        const int pos = atomicAdd(&cells[((cz - za) * g.dy + cy) * g.dx + cx + 1], 1);
        spts[pos] = make_float4(x, y, z, __int_as_float(k));
    });
    __syncthreads();
    return total;
}

// The K (1 or 3) nearest staged points of (qx, qy, qz) by (distance, index): the 3x3x3 cells
// around the query, then ring by ring until the K-th best squared distance is below the
// squared distance to the nearest face of the searched block that has unsearched cells behind
// it.  `cells` / `spts` hold the z layers [za, zb] of the grid.  Returns false if a ring
// would need layers outside [za, zb] before the search could stop (the best list is then
// incomplete).
template <int K>
__device__ __forceinline__ bool sg_nn_search(const SgGrid& g, const int* cells, const float4* spts, int za, int zb,
                                             float qx, float qy, float qz, float& b1, float& b2, float& b3,
                                             int& i1, int& i2, int& i3)
{
    const int cx = sg_cell_coord(qx, g.minx, g.inv_h, g.dx);
    const int cy = sg_cell_coord(qy, g.miny, g.inv_h, g.dy);
    const int cz = sg_cell_coord(qz, g.minz, g.inv_h, g.dz);
    b1 = b2 = b3 = CUDART_INF_F;
    i1 = i2 = i3 = 0x7fffffff;
    int px0 = 0, px1 = -1, py0 = 0, py1 = -1, pz0 = 0, pz1 = -1;  // block searched so far
    const int max_ring = max(g.dx, max(g.dy, g.dz));
    for (int ring = 1; ring <= max_ring; ++ring)
    {
        const int x0 = max(cx - ring, 0), x1 = min(cx + ring, g.dx - 1);
        const int y0 = max(cy - ring, 0), y1 = min(cy + ring, g.dy - 1);
        const int z0 = max(cz - ring, 0), z1 = min(cz + ring, g.dz - 1);
        if (z0 < za || z1 > zb) return false;  // this ring leaves the staged layers
        for (int z = z0; z <= z1; ++z)
            for (int y = y0; y <= y1; ++y)
            {
                const bool inner_row = z >= pz0 && z <= pz1 && y >= py0 && y <= py1;
                const int row = ((z - za) * g.dy + y) * g.dx;
                // cells of the row not searched before: all of [x0, x1], or its two ends
                for (int side = 0; side < 2; ++side)
                {
                    int xa, xb;
                    if (!inner_row)
                    {
                        if (side == 1) break;
                        xa = x0;
                        xb = x1;
                    }
                    else if (side == 0)
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
                    const int beg = cells[row + xa], end = cells[row + xb + 1];
                    // Four candidates per step: the loads and distances are independent; a
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
                        for (int u = 0; u < 4; ++u) c[u] = spts[p + u];
#pragma unroll
                        for (int u = 0; u < 4; ++u) d[u] = sumsq_abc(qx - c[u].x, qy - c[u].y, qz - c[u].z);
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (d[u] <= (K == 1 ? b1 : b3)) consider(d[u], __float_as_int(c[u].w));
                    }
                    for (; p < end; ++p)
                    {
                        const float4 c = spts[p];
                        const float d = sumsq_abc(qx - c.x, qy - c.y, qz - c.z);
                        if (d <= (K == 1 ? b1 : b3)) consider(d, __float_as_int(c.w));
                    }
                }
            }
        px0 = x0; px1 = x1; py0 = y0; py1 = y1; pz0 = z0; pz1 = z1;
        if (x0 == 0 && y0 == 0 && z0 == 0 && x1 == g.dx - 1 && y1 == g.dy - 1 && z1 == g.dz - 1) return true;
        // distance to the nearest face of the block with unsearched cells behind it
        float rho = CUDART_INF_F;
        if (x0 > 0) rho = fminf(rho, qx - (g.minx + x0 * g.h));
        if (x1 < g.dx - 1) rho = fminf(rho, (g.minx + (x1 + 1) * g.h) - qx);
        if (y0 > 0) rho = fminf(rho, qy - (g.miny + y0 * g.h));
        if (y1 < g.dy - 1) rho = fminf(rho, (g.miny + (y1 + 1) * g.h) - qy);
        if (z0 > 0) rho = fminf(rho, qz - (g.minz + z0 * g.h));
        if (z1 < g.dz - 1) rho = fminf(rho, (g.minz + (z1 + 1) * g.h) - qz);
        // faces are computed in floating point and a point next to a face may be binned on
        // either side: a thousandth of a cell plus the coordinate rounding as margin
        rho -= 1.0e-3f * g.h + 4.0e-7f * (fabsf(qx) + fabsf(qy) + fabsf(qz) + fabsf(g.minx) + fabsf(g.miny) + fabsf(g.minz));
        const float kth = K == 1 ? b1 : b3;
        if (rho > 0.f && kth < rho * rho * 0.9999f) return true;
    }
    return true;
}

// ------------------------------------------------------------------------------ three_nn
//
// Grid: blockIdx.x = cloud * parts + part.  Every CTA of a cloud bins all known points.
// The cells in x-fastest order cut the known points into `parts` runs of equal length;
// the CTA owns the unknown points that fall into the cells of run `part` (as many
// unknown points per CTA as the known density predicts).  It collects them from one pass
// over the cloud's unknown points and sorts them by cell, so that the lanes of a warp
// search the same or adjacent cells: same loop counts, same shared-memory rows.
constexpr int kSgQueryCapMin = 1024;

template <int K>  // K = 3: three_nn, K = 1: nearest neighbour (chamfer); K outputs per unknown point
__global__ void __launch_bounds__(kSgThreads, 2)
    sg_three_nn_kernel(int n, int m, int parts, int qcap, int max_dim, int cells_cap,
                       const float* __restrict__ unknown_all, const float* __restrict__ known_all,
                       float* __restrict__ dist2_all, int32_t* __restrict__ idx_all,
                       unsigned char* __restrict__ need_all)
{
    extern __shared__ __align__(16) unsigned char sg_raw[];
    __shared__ int s_nq;
    float4* spts = reinterpret_cast<float4*>(sg_raw);
    int* cells = reinterpret_cast<int*>(spts + m);
    int* qj = cells + cells_cap + 1;   // collected unknown points, in arrival order
    int* qsorted = qj + qcap;          // the same, sorted by key
    int* counts = qsorted + qcap;      // per key: run length + 1 entries
    unsigned short* qkey = reinterpret_cast<unsigned short*>(counts + (m / parts + 3));

    const int tid = threadIdx.x;
    const int cloud = blockIdx.x / parts, part = blockIdx.x - cloud * parts;
    const float* known = known_all + static_cast<size_t>(cloud) * m * 3;
    const float* unknown = unknown_all + static_cast<size_t>(cloud) * n * 3;
    const size_t qbase = static_cast<size_t>(cloud) * n;

    const SgGrid g = sg_make_grid(known, m, 1.0e-30f, max_dim, static_cast<size_t>(cells_cap));
    int staged = -1;
    if (g.ok) staged = sg_bin(known, m, g, 0, g.dz - 1, cells, spts, m);
    if (staged < 0)
    {
        if (part == 0)
            for (int j = tid; j < n; j += kSgThreads) need_all[qbase + j] = 1;
        return;
    }
    // run of known points this CTA owns: a cell belongs to the run its first slot lies in
    // (the last run also takes the empty cells behind the last point)
    const int lo = static_cast<int>(static_cast<long long>(part) * m / parts);
    const int hi = part == parts - 1 ? m + 1 : static_cast<int>(static_cast<long long>(part + 1) * m / parts);
    const int nkeys = hi - lo;  // at most m / parts + 2
    if (tid == 0) s_nq = 0;
    for (int k = tid; k <= nkeys; k += kSgThreads) counts[k] = 0;
    __syncthreads();
    sg_for_points(unknown, n, [&](int j, float qx, float qy, float qz) {
        if (!(fabsf(qx) < 1.0e18f && fabsf(qy) < 1.0e18f && fabsf(qz) < 1.0e18f))
        {
            if (part == 0) need_all[qbase + j] = 1;  // no cell: the first CTA hands it to the scan
            return;
        }
        const int cx = sg_cell_coord(qx, g.minx, g.inv_h, g.dx);
        const int cy = sg_cell_coord(qy, g.miny, g.inv_h, g.dy);
        const int cz = sg_cell_coord(qz, g.minz, g.inv_h, g.dz);
        const int first_slot = cells[(cz * g.dy + cy) * g.dx + cx];
        if (first_slot < lo || first_slot >= hi) return;
        const int pos = atomicAdd(&s_nq, 1);
        if (pos < qcap)
        {
            qj[pos] = j;
            qkey[pos] = static_cast<unsigned short>(first_slot - lo);
            atomicAdd(&counts[first_slot - lo + 1], 1);
        }
        else
        {
            need_all[qbase + j] = 1;  // far more unknown points here than known ones: left to the scan
        }
    });
    __syncthreads();
    const int nq = min(s_nq, qcap);
    sg_block_scan(counts + 1, nkeys);
    for (int i = tid; i < nq; i += kSgThreads) qsorted[atomicAdd(&counts[qkey[i] + 1], 1)] = qj[i];
    __syncthreads();

    for (int i = tid; i < nq; i += kSgThreads)
    {
        const int j = qsorted[i];
        const size_t t = qbase + j;
        const float qx = __ldg(unknown + 3 * j + 0), qy = __ldg(unknown + 3 * j + 1), qz = __ldg(unknown + 3 * j + 2);
        float b1, b2, b3;
        int i1, i2, i3;
        sg_nn_search<K>(g, cells, spts, 0, g.dz - 1, qx, qy, qz, b1, b2, b3, i1, i2, i3);
        need_all[t] = 0;
        dist2_all[K * t + 0] = b1;
        idx_all[K * t + 0] = i1 == 0x7fffffff ? 0 : i1;
        if (K == 3)
        {
            dist2_all[3 * t + 1] = b2;
            dist2_all[3 * t + 2] = b3;
            idx_all[3 * t + 1] = i2 == 0x7fffffff ? 0 : i2;
            idx_all[3 * t + 2] = i3 == 0x7fffffff ? 0 : i3;
        }
    }
}

// ----------------------------------------------------------- nearest neighbours, by layers
//
// The same search for known clouds too large for one CTA's shared memory.  Grid:
// blockIdx.x = cloud * parts + part; the CTA owns the unknown points whose z cell lies in
// layers [part * lpp, (part + 1) * lpp) of the grid of the known points and stages those
// layers plus `pad` layers on either side.  It collects its unknown points from one pass
// over the cloud, sorts them by cell and answers one per thread.  A search that would have
// to leave the staged layers (its ring-1 block never does) is flagged for the scan.
template <int K>
__global__ void __launch_bounds__(kSgThreads, 2)
    sg_nn_slab_kernel(int n, int m, int parts, int lpp, int pad, int qcap, int max_dim, int cells_cap,
                      int slab_cells_cap, int own_cells_cap, int pcap, const float* __restrict__ unknown_all,
                      const float* __restrict__ known_all, float* __restrict__ dist2_all,
                      int32_t* __restrict__ idx_all, unsigned char* __restrict__ need_all)
{
    extern __shared__ __align__(16) unsigned char sg_raw[];
    __shared__ int s_nq;
    float4* spts = reinterpret_cast<float4*>(sg_raw);
    int* cells = reinterpret_cast<int*>(spts + pcap);
    int* counts = cells + slab_cells_cap + 1;   // per owned cell: run of collected unknown points
    int* qj = counts + own_cells_cap + 2;       // collected unknown points, in arrival order
    int* qsorted = qj + qcap;                   // the same, sorted by cell
    unsigned short* qkey = reinterpret_cast<unsigned short*>(qsorted + qcap);

    const int tid = threadIdx.x;
    const int cloud = blockIdx.x / parts, part = blockIdx.x - cloud * parts;
    const float* known = known_all + static_cast<size_t>(cloud) * m * 3;
    const float* unknown = unknown_all + static_cast<size_t>(cloud) * n * 3;
    const size_t qbase = static_cast<size_t>(cloud) * n;

    const SgGrid g = sg_make_grid(known, m, 1.0e-30f, max_dim, static_cast<size_t>(cells_cap));
    if (!g.ok)
    {
        if (part == 0)
            for (int j = tid; j < n; j += kSgThreads) need_all[qbase + j] = 1;
        return;
    }
    const int own_lo = part * lpp, own_hi = min(g.dz, own_lo + lpp) - 1;
    if (own_lo > own_hi) return;
    const int za = max(own_lo - pad, 0), zb = min(own_hi + pad, g.dz - 1);
    const int staged = sg_bin(known, m, g, za, zb, cells, spts, pcap);
    const int nkeys = (own_hi - own_lo + 1) * g.dy * g.dx;  // at most own_cells_cap, below 65536
    if (tid == 0) s_nq = 0;
    for (int k = tid; k <= nkeys; k += kSgThreads) counts[k] = 0;
    __syncthreads();
    sg_for_points(unknown, n, [&](int j, float qx, float qy, float qz) {
        if (!(fabsf(qx) < 1.0e18f && fabsf(qy) < 1.0e18f && fabsf(qz) < 1.0e18f))
        {
            if (part == 0) need_all[qbase + j] = 1;  // no cell: the first CTA hands it to the scan
            return;
        }
        const int cz = sg_cell_coord(qz, g.minz, g.inv_h, g.dz);
        if (cz < own_lo || cz > own_hi) return;
        const int cy = sg_cell_coord(qy, g.miny, g.inv_h, g.dy);
        const int cx = sg_cell_coord(qx, g.minx, g.inv_h, g.dx);
        const int key = ((cz - own_lo) * g.dy + cy) * g.dx + cx;
        const int pos = staged < 0 ? qcap : atomicAdd(&s_nq, 1);
        if (pos < qcap)
        {
            qj[pos] = j;
            qkey[pos] = static_cast<unsigned short>(key);
            atomicAdd(&counts[key + 1], 1);
        }
        else
        {
            need_all[qbase + j] = 1;  // more known or unknown points around these layers than fit
        }
    });
    __syncthreads();
    const int nq = min(s_nq, qcap);
    sg_block_scan(counts + 1, nkeys);
    for (int i = tid; i < nq; i += kSgThreads) qsorted[atomicAdd(&counts[qkey[i] + 1], 1)] = qj[i];
    __syncthreads();

    for (int i = tid; i < nq; i += kSgThreads)
    {
        const int j = qsorted[i];
        const size_t t = qbase + j;
        const float qx = __ldg(unknown + 3 * j + 0), qy = __ldg(unknown + 3 * j + 1), qz = __ldg(unknown + 3 * j + 2);
        float b1, b2, b3;
        int i1, i2, i3;
        if (!sg_nn_search<K>(g, cells, spts, za, zb, qx, qy, qz, b1, b2, b3, i1, i2, i3))
        {
            need_all[t] = 1;
            continue;
        }
        need_all[t] = 0;
        dist2_all[K * t + 0] = b1;
        idx_all[K * t + 0] = i1 == 0x7fffffff ? 0 : i1;
        if (K == 3)
        {
            dist2_all[3 * t + 1] = b2;
            dist2_all[3 * t + 2] = b3;
            idx_all[3 * t + 1] = i2 == 0x7fffffff ? 0 : i2;
            idx_all[3 * t + 2] = i3 == 0x7fffffff ? 0 : i3;
        }
    }
}

// ---------------------------------------------------------------------------- ball query
//
// Grid: blockIdx.x = cloud * parts + part; the CTA owns the centres whose z cell lies in
// layers [part * lpp, (part + 1) * lpp) and stages those layers plus one on either side.
// One warp per centre: the cells of the ball are at most 16 runs of staged points (one per
// (z, y) row of cells); the lanes walk the concatenation of the runs 32 candidates at a
// time, hits are appended to a per-warp buffer as (original index << kSgSlotBits) | slot,
// and a hit's output position is its rank among the hits (the number of smaller entries),
// so the nsample lowest indices land in index order without a sort.  The distance written
// out is recomputed from the staged coordinates with the arithmetic of the test.
constexpr int kSgWarps = kSgThreads / 32;
constexpr int kSgHitCap = 256;   // hits per centre the buffer takes; more: left to the scan
constexpr int kSgMaxRows = 16;

struct SgWarpScratch
{
    uint32_t hits[kSgHitCap];
    int row_end[kSgMaxRows];    // inclusive prefix of the run lengths
    int row_shift[kSgMaxRows];  // slot of candidate v of row r = row_shift[r] + v
    int first;
};

__global__ void __launch_bounds__(kSgThreads, 2)
    sg_ball_query_kernel(int n, int m, int parts, int lpp, float radius, int nsample, float max_candidates,
                         int max_dim, int cells_cap, int slab_cells_cap, int pcap,
                         const float* __restrict__ new_xyz_all, const float* __restrict__ xyz_all,
                         int64_t* __restrict__ idx_out, float* __restrict__ dist_out,
                         unsigned char* __restrict__ need_all)
{
    extern __shared__ __align__(16) unsigned char sg_raw[];
    __shared__ int s_count;
    float4* spts = reinterpret_cast<float4*>(sg_raw);
    int* cells = reinterpret_cast<int*>(spts + pcap);
    int* qlist = cells + slab_cells_cap + 1;
    SgWarpScratch* wscr = reinterpret_cast<SgWarpScratch*>(qlist + kSgQueryChunk);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cloud = blockIdx.x / parts, part = blockIdx.x - cloud * parts;
    const float* xyz = xyz_all + static_cast<size_t>(cloud) * n * 3;
    const float* new_xyz = new_xyz_all + static_cast<size_t>(cloud) * m * 3;
    const size_t qbase = static_cast<size_t>(cloud) * m;

    const float r1 = radius * 1.00001f + 1.0e-30f;
    const float r2 = __fmul_rn(radius, radius);
    const SgGrid g = sg_make_grid(xyz, n, r1, max_dim, static_cast<size_t>(cells_cap));
    // too few cells: the scan is as good; a radius that is not a positive finite number: the scan decides
    const bool use = g.ok && radius > 0.f && radius < 1.0e18f && g.dx * g.dy * g.dz >= 64;
    if (!use)
    {
        if (part == 0)
            for (int j = tid; j < m; j += kSgThreads) need_all[qbase + j] = 1;
        return;
    }
    const int own_lo = part * lpp, own_hi = min(g.dz, own_lo + lpp) - 1;
    if (own_lo > own_hi) return;
    const int za = max(own_lo - 1, 0), zb = min(own_hi + 1, g.dz - 1);
    const int staged = sg_bin(xyz, n, g, za, zb, cells, spts, pcap);

    SgWarpScratch& ws = wscr[warp];
    for (int base = 0; base < m; base += kSgQueryChunk)
    {
        if (tid == 0) s_count = 0;
        __syncthreads();
        const int jend = min(m, base + kSgQueryChunk);
        // (a chunk starts at a multiple of four centres, so the 16-byte path stays aligned)
        sg_for_points(new_xyz + 3 * static_cast<size_t>(base), jend - base, [&](int jj, float qx, float qy, float qz) {
            const int j = base + jj;
            if (!(fabsf(qx) < 1.0e18f && fabsf(qy) < 1.0e18f && fabsf(qz) < 1.0e18f))
            {
                if (part == 0) need_all[qbase + j] = 1;  // no cell: the first CTA hands it to the scan
                return;
            }
            const int qcz = sg_cell_coord(qz, g.minz, g.inv_h, g.dz);
            if (qcz < own_lo || qcz > own_hi) return;
            if (staged < 0)
                need_all[qbase + j] = 1;  // more points around these layers than fit
            else
                qlist[atomicAdd(&s_count, 1)] = j;
        });
        __syncthreads();
        const int nq = s_count;
        // the next centre's coordinates are requested one centre ahead (they come from L2)
        int j_next = warp < nq ? qlist[warp] : 0;
        float nx = __ldg(new_xyz + 3 * j_next + 0), ny_ = __ldg(new_xyz + 3 * j_next + 1), nz = __ldg(new_xyz + 3 * j_next + 2);
        for (int i = warp; i < nq; i += kSgWarps)
        {
            // everything up to the candidate loop is the same in all lanes of the warp
            const int j = j_next;
            const size_t t = qbase + j;
            const float qx = nx, qy = ny_, qz = nz;
            if (i + kSgWarps < nq)
            {
                j_next = qlist[i + kSgWarps];
                nx = __ldg(new_xyz + 3 * j_next + 0);
                ny_ = __ldg(new_xyz + 3 * j_next + 1);
                nz = __ldg(new_xyz + 3 * j_next + 2);
            }
            // cell range of the ball, enlarged by the rounding of the exact test (1e-5 relative)
            // and of q +- r itself (2e-7 |q|); the cell function is monotone, so every point the
            // exact test can accept lies in a cell of the range
            const float rx = r1 + fabsf(qx) * 2.0e-7f, ry = r1 + fabsf(qy) * 2.0e-7f, rz = r1 + fabsf(qz) * 2.0e-7f;
            const int x0 = sg_cell_coord(qx - rx, g.minx, g.inv_h, g.dx), x1 = sg_cell_coord(qx + rx, g.minx, g.inv_h, g.dx);
            const int y0 = sg_cell_coord(qy - ry, g.miny, g.inv_h, g.dy), y1 = sg_cell_coord(qy + ry, g.miny, g.inv_h, g.dy);
            const int z0 = sg_cell_coord(qz - rz, g.minz, g.inv_h, g.dz), z1 = sg_cell_coord(qz + rz, g.minz, g.inv_h, g.dz);
            const int ny = y1 - y0 + 1, nrows = ny * (z1 - z0 + 1);
            if (z0 < za || z1 > zb || nrows > kSgMaxRows)
            {
                // reaches beyond the staged layers (cells exactly one radius wide)
                if (lane == 0) need_all[t] = 1;
                continue;
            }
            int len = 0, beg = 0;
            if (lane < nrows)
            {
                const int cz = z0 + lane / ny, cy = y0 + lane - (lane / ny) * ny;
                const int row = ((cz - za) * g.dy + cy) * g.dx;
                beg = cells[row + x0];
                len = cells[row + x1 + 1] - beg;
            }
            int incl = len;
#pragma unroll
            for (int o = 1; o < kSgMaxRows; o <<= 1)
            {
                const int v = __shfl_up_sync(kFullMask, incl, o);
                if (lane >= o) incl += v;
            }
            const int total = __shfl_sync(kFullMask, incl, kSgMaxRows - 1);
            if (static_cast<float>(total) > max_candidates)
            {
                // crowded: the scan, which stops at the nsample-th hit, is cheaper
                if (lane == 0) need_all[t] = 1;
                continue;
            }
            __syncwarp();  // the previous centre's reads of the scratch are done
            if (lane < kSgMaxRows)
            {
                ws.row_end[lane] = incl;
                ws.row_shift[lane] = beg - (incl - len);
            }
            __syncwarp();
            int nh = 0;
            for (int v0 = 0; v0 < total; v0 += 32)
            {
                const int v = v0 + lane;
                const bool valid = v < total;
                int r = 0;
                for (int k = 0; k < nrows - 1; ++k) r += ws.row_end[k] <= v ? 1 : 0;
                const int p = valid ? ws.row_shift[r] + v : 0;
                const float4 c = spts[p];
                const float d = sumsq_abc(qx - c.x, qy - c.y, qz - c.z);
                const bool hit = valid && d < r2;
                const uint32_t bal = __ballot_sync(kFullMask, hit);
                if (hit)
                {
                    const int pos = nh + __popc(bal & ((1u << lane) - 1u));
                    if (pos < kSgHitCap)
                        ws.hits[pos] = (static_cast<uint32_t>(__float_as_int(c.w)) << kSgSlotBits) | static_cast<uint32_t>(p);
                }
                nh += __popc(bal);
            }
            if (nh > kSgHitCap)
            {
                if (lane == 0) need_all[t] = 1;
                continue;
            }
            __syncwarp();
            int64_t* orow = idx_out + t * nsample;
            float* drow = dist_out + t * nsample;
            for (int h0 = 0; h0 < nh; h0 += 32)
            {
                const int h = h0 + lane;
                if (h < nh)
                {
                    const uint32_t e = ws.hits[h];
                    int rank = 0;
                    for (int k = 0; k < nh; ++k) rank += ws.hits[k] < e ? 1 : 0;
                    if (rank < nsample)
                    {
                        const float4 c = spts[e & ((1u << kSgSlotBits) - 1u)];
                        orow[rank] = static_cast<int64_t>(e >> kSgSlotBits);
                        drow[rank] = sumsq_abc(qx - c.x, qy - c.y, qz - c.z);
                        if (rank == 0) ws.first = static_cast<int>(e >> kSgSlotBits);
                    }
                }
            }
            __syncwarp();
            const int64_t first = nh ? static_cast<int64_t>(ws.first) : 0;
            for (int s = min(nh, nsample) + lane; s < nsample; s += 32)
            {
                orow[s] = first;
                drow[s] = -1.0f;
            }
            if (lane == 0) need_all[t] = 0;
        }
        __syncthreads();
    }
}

}  // namespace

// ------------------------------------------------------------------------------- host side

// Whether the shared-memory grid serves a three_nn call with m known points per cloud.
bool sg_three_nn_fits(int m) { return m >= 256 && m <= kSgMaxPoints; }

// k = 3: three_nn; k = 1: the nearest neighbour only (one distance and one index per unknown point)
int sg_nn(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
          unsigned char* need, cudaStream_t s)
{
    const int max_dim = grid_max_dim(m);
    const int cap = static_cast<int>(grid_cells_capacity(m));
    // CTAs per cloud: at most two per SM over the batch (one wave), at least 256 unknown points each, and runs of
    // known points short enough for a 16-bit sort key
    int parts = 2 * num_sms() / b;
    if (parts > n / 256) parts = n / 256;
    if (parts > m / 8) parts = m / 8;
    if (parts < 1) parts = 1;
    const size_t base = static_cast<size_t>(m) * sizeof(float4) + (static_cast<size_t>(cap) + 1) * sizeof(int) +
                        (static_cast<size_t>(m / parts) + 3) * sizeof(int);
    // unknown points a CTA takes: 2.5 times its share, whatever still fits
    long long qcap = 5ll * n / (2 * parts) + 64;
    if (qcap < kSgQueryCapMin) qcap = kSgQueryCapMin;
    if (qcap > n) qcap = n;
    const long long room = (static_cast<long long>(kSgSmemBudget) - static_cast<long long>(base)) / 10;
    if (qcap > room) qcap = room;
    qcap = (qcap + 1) / 2 * 2;
    TPK_REQUIRE(qcap >= 2, "three_nn grid: no room for the query list");
    const size_t smem = base + static_cast<size_t>(qcap) * 10;
    auto kernel = k == 1 ? sg_three_nn_kernel<1> : sg_three_nn_kernel<3>;
    prefer_max_shared(kernel);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("three_nn grid: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long grid = static_cast<long long>(b) * parts;
    TPK_REQUIRE(grid < (1ll << 31), "three_nn: too many queries");
    count_launches(1), kernel<<<static_cast<unsigned>(grid), kSgThreads, smem, s>>>(n, m, parts, static_cast<int>(qcap), max_dim, cap, unknown,
                                                                 known, dist2, idx, need);
    return check_launch("three_nn grid");
}

int sg_three_nn(int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
                unsigned char* need, cudaStream_t s)
{
    return sg_nn(3, b, n, m, unknown, known, dist2, idx, need, s);
}

namespace
{
struct SgSlabPlan
{
    int max_dim, cells_cap, slab_cells_cap, own_cells_cap, pcap, qcap, lpp, pad, parts;
    size_t smem;
    bool ok;
};

// Layers per CTA for the nearest-neighbour search by layers: the same trade as for the ball
// query (every CTA passes over both clouds; CTAs beyond what the SMs hold wait), one layer
// of padding on either side.
SgSlabPlan sg_slab_plan(int b, int n, int m)
{
    SgSlabPlan best = {};
    best.ok = false;
    if (b < 1 || n < 1 || m < 1024) return best;
    const int max_dim = grid_max_dim(m);
    const int pad = 1;
    double best_cost = 0.0;
    for (int lpp = 1; lpp <= max_dim; ++lpp)
    {
        const int parts = (max_dim + lpp - 1) / lpp;
        if (lpp > 1 && parts == (max_dim + lpp - 2) / (lpp - 1)) continue;  // same parts with fewer layers each
        const int layers = lpp + 2 * pad < max_dim ? lpp + 2 * pad : max_dim;
        const size_t slab_cells = static_cast<size_t>(layers) * max_dim * max_dim;
        const size_t own_cells = static_cast<size_t>(lpp) * max_dim * max_dim;
        if (own_cells >= 65536) continue;  // 16-bit sort keys
        size_t qcap = static_cast<size_t>(2.5 * n * lpp / max_dim) + 256;
        if (qcap > static_cast<size_t>(n)) qcap = n;
        qcap = (qcap + 1) / 2 * 2;
        const size_t fixed = (slab_cells + 1 + own_cells + 2) * sizeof(int) + qcap * 10 + 64;
        if (fixed + 1024 * sizeof(float4) > kSgSmemBudget) continue;
        size_t want = static_cast<size_t>(2.0 * m * layers / max_dim) + 256;
        if (want > static_cast<size_t>(m)) want = m;
        const size_t room = (kSgSmemBudget - fixed) / sizeof(float4);
        if (want > room)
        {
            // single layers: take what fits (crowded layers go to the scan), unless even an
            // average layer would not fit
            if (lpp > 1 || static_cast<double>(m) * layers / max_dim > static_cast<double>(room)) continue;
            want = room;
        }
        SgSlabPlan p = {};
        p.max_dim = max_dim;
        p.cells_cap = static_cast<int>(grid_cells_capacity(m));
        p.lpp = lpp;
        p.pad = pad;
        p.parts = parts;
        p.slab_cells_cap = static_cast<int>(slab_cells);
        p.own_cells_cap = static_cast<int>(own_cells);
        p.qcap = static_cast<int>(qcap);
        p.pcap = static_cast<int>((want + 3) / 4 * 4);
        p.smem = static_cast<size_t>(p.pcap) * sizeof(float4) + fixed;
        p.ok = true;
        const int per_sm = (p.smem + 1024) * 2 <= 228 * 1024 ? 2 : 1;
        const double slots = static_cast<double>(num_sms()) * per_sm;
        // about 1 ns per point for the passes over both clouds, 25 ns per unknown point answered
        const double passes = 1.0 * m + 0.4 * n, per_layer = 25.0 * n / max_dim;
        const double total = static_cast<double>(b) * (parts * passes + max_dim * per_layer);
        const double heaviest = passes + 1.5 * lpp * per_layer;
        const double cost = total / slots > heaviest ? total / slots : heaviest;
        if (!best.ok || cost < best_cost)
        {
            best = p;
            best_cost = cost;
        }
    }
    return best;
}
}  // namespace

// Whether the search by layers serves m known points per cloud (above the whole-cloud limit).
bool sg_nn_slab_fits(int b, int n, int m) { return m > kSgMaxPoints && sg_slab_plan(b, n, m).ok; }

int sg_nn_slab(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
               unsigned char* need, cudaStream_t s)
{
    const SgSlabPlan p = sg_slab_plan(b, n, m);
    if (!p.ok)
    {
        set_error("nearest neighbours by layers: sizes do not fit shared memory (n=%d m=%d)", n, m);
        return TPK_ERR_UNSUPPORTED;
    }
    auto kernel = k == 1 ? sg_nn_slab_kernel<1> : sg_nn_slab_kernel<3>;
    prefer_max_shared(kernel);
    if (p.smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(p.smem));
        if (err != cudaSuccess)
        {
            set_error("nearest neighbours by layers: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long grid = static_cast<long long>(b) * p.parts;
    TPK_REQUIRE(grid < (1ll << 31), "nearest neighbours: too many clouds");
    count_launches(1), kernel<<<static_cast<unsigned>(grid), kSgThreads, p.smem, s>>>(n, m, p.parts, p.lpp, p.pad, p.qcap, p.max_dim,
                                                                   p.cells_cap, p.slab_cells_cap, p.own_cells_cap, p.pcap,
                                                                   unknown, known, dist2, idx, need);
    return check_launch("nearest neighbours by layers");
}

namespace
{
struct SgBallPlan
{
    int max_dim, cells_cap, slab_cells_cap, pcap, lpp, parts;
    size_t smem;
    bool ok;
};

// Layers per CTA.  Every CTA passes over the whole cloud three times to bin its layers
// (a fixed cost) and then answers the centres of the layers it owns.  The plan minimises
// the larger of the heaviest CTA and the total work divided by the CTAs the SMs hold at once.
SgBallPlan sg_ball_plan(int b, int n, int m, int nsample)
{
    SgBallPlan best = {};
    best.ok = false;
    if (b < 1 || n < 1024 || n >= (1 << (32 - kSgSlotBits)) || nsample < 1 || nsample > kSgHitCap) return best;
    const int max_dim = grid_max_dim(n);
    double best_cost = 0.0;
    for (int lpp = 1; lpp <= max_dim; ++lpp)
    {
        const int parts = (max_dim + lpp - 1) / lpp;
        if (lpp > 1 && parts == (max_dim + lpp - 2) / (lpp - 1)) continue;  // same parts with fewer layers each
        const int layers = lpp + 2 < max_dim ? lpp + 2 : max_dim;
        const size_t slab_cells = static_cast<size_t>(layers) * max_dim * max_dim;
        const size_t fixed = (slab_cells + 1) * sizeof(int) + static_cast<size_t>(kSgQueryChunk) * sizeof(int) +
                             kSgWarps * sizeof(SgWarpScratch) + 64;
        if (fixed + 1024 * sizeof(float4) > kSgSmemBudget) continue;
        size_t want = static_cast<size_t>(2.0 * n * layers / max_dim) + 256;
        if (want > static_cast<size_t>(n)) want = n;
        size_t room = (kSgSmemBudget - fixed) / sizeof(float4);
        if (room > (1u << kSgSlotBits)) room = 1u << kSgSlotBits;
        if (want > room)
        {
            // single layers: take what fits (crowded layers go to the scan), unless even an
            // average layer would not fit
            if (lpp > 1 || static_cast<double>(n) * layers / max_dim > static_cast<double>(room)) continue;
            want = room;
        }
        SgBallPlan p = {};
        p.max_dim = max_dim;
        p.cells_cap = static_cast<int>(grid_cells_capacity(n));
        p.lpp = lpp;
        p.parts = parts;
        p.slab_cells_cap = static_cast<int>(slab_cells);
        p.pcap = static_cast<int>((want + 3) / 4 * 4);
        p.smem = static_cast<size_t>(p.pcap) * sizeof(float4) + fixed;
        p.ok = true;
        // 228 KB of shared memory per SM, 1 KB reserved per CTA; registers allow two CTAs
        const int per_sm = (p.smem + 1024) * 2 <= 228 * 1024 ? 2 : 1;
        const double slots = static_cast<double>(num_sms()) * per_sm;
        // measured: about 1 ns per point for the three passes, 75 ns per centre (one warp each,
        // sixteen at a time); the middle layers of a round cloud hold 1.5 times the average
        const double passes = 1.0 * n, per_layer = 75.0 * m / max_dim;
        const double total = static_cast<double>(b) * (parts * passes + max_dim * per_layer);
        const double heaviest = passes + 1.5 * lpp * per_layer;
        const double cost = total / slots > heaviest ? total / slots : heaviest;
        if (!best.ok || cost < best_cost)
        {
            best = p;
            best_cost = cost;
        }
    }
    return best;
}
}  // namespace

bool sg_ball_query_fits(int b, int n, int nsample) { return sg_ball_plan(b, n, n, nsample).ok; }

int sg_ball_query(int b, int n, int m, float radius, int nsample, const float* new_xyz, const float* xyz,
                  int64_t* idx, float* dist, unsigned char* need, cudaStream_t s)
{
    const SgBallPlan p = sg_ball_plan(b, n, m, nsample);
    if (!p.ok)
    {
        set_error("ball_query grid: sizes do not fit shared memory (n=%d nsample=%d)", n, nsample);
        return TPK_ERR_UNSUPPORTED;
    }
    auto kernel = sg_ball_query_kernel;
    prefer_max_shared(kernel);
    if (p.smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(p.smem));
        if (err != cudaSuccess)
        {
            set_error("ball_query grid: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const float max_cand = 2.0f * sqrtf(6.45f * static_cast<float>(n) * static_cast<float>(nsample));
    const long long grid = static_cast<long long>(b) * p.parts;
    TPK_REQUIRE(grid < (1ll << 31), "ball_query_dense: too many clouds");
    count_launches(1), kernel<<<static_cast<unsigned>(grid), kSgThreads, p.smem, s>>>(n, m, p.parts, p.lpp, radius, nsample, max_cand,
                                                                   p.max_dim, p.cells_cap, p.slab_cells_cap, p.pcap,
                                                                   new_xyz, xyz, idx, dist, need);
    return check_launch("ball_query grid");
}

}  // namespace tpk

