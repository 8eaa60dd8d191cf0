/*
 * CPU oracle for the spatial-search path of torch-points-kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the smoke
 * test and the CPU-baseline leg of the benchmark compare the CUDA library against.
 * Nothing in the shipped package links, loads or calls it.
 *
 * Every function restates, in plain C, the rule of one reference kernel.  The
 * reference CUDA sources are compiled with nvcc's default -fmad=true, which
 * contracts the left-associated sum a*a + b*b + c*c into
 *     fma(c, c, fma(a, a, b*b))
 * and the partial_dense accumulation loop (dist = 0; dist += t*t) into
 *     fma(c, c, fma(b, b, fma(a, a, 0))).
 * The oracle writes those forms out with fmaf() and is built with
 * -ffp-contract=off so that the host compiler adds no contraction of its own.
 * The reference CPU (nanoflann) path is built without FMA and evaluates
 * ((a*a) + b*b) + c*c unfused; orc_knn follows that.
 *
 * Parity pinning: orc_knn, orc_three_interpolate and the set content of the ball
 * queries are checked against the reference's own CPU extension and against the
 * known-answer vectors of the reference's unit tests (tests/golden).  The CUDA-only
 * rules (FPS tie-break, index-order ball query, chamfer argmin, fma patterns) are
 * checked on a GPU against the reference's CUDA extension compiled from its own
 * sources (oracle/Makefile, target ref_cuda).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* a*a + b*b + c*c as nvcc contracts it (dense ball query, three_nn, chamfer, FPS). */
static inline float sumsq_abc(float a, float b, float c)
{
    return fmaf(c, c, fmaf(a, a, b * b));
}

/* dist = 0; dist += a*a; dist += b*b; dist += c*c  as nvcc contracts it (partial_dense). */
static inline float sumsq_loop(float a, float b, float c)
{
    return fmaf(c, c, fmaf(b, b, fmaf(a, a, 0.0f)));
}

/* Largest power of two <= n, capped at 512, at least 1.
 * Follows opt_n_threads, cuda/include/cuda_utils.h:16-21. */
int orc_opt_n_threads(int work_size)
{
    const int pow_2 = (int)(log((double)work_size) / log(2.0));
    int v = 1 << pow_2;
    if (v > 512) v = 512;
    if (v < 1) v = 1;
    return v;
}

/*
 * Furthest point sampling, cuda/src/sampling_gpu.cu:16-144 with the launch of
 * :146-198 (block size = opt_n_threads(n)) and the scratch initialisation of
 * cuda/src/sampling.cpp:14-18 (output zeros, temp = 1e10).
 * The per-thread strided scan and the shared-memory tree are replayed literally
 * because together they define which index wins among equal distances.
 */
void orc_fps(int b, int n, int m, const float* dataset_all, int32_t* idxs_all)
{
    const int bs = orc_opt_n_threads(n);
#pragma omp parallel for schedule(dynamic, 1)
    for (int bi = 0; bi < b; ++bi)
    {
        float* temp = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
        float* dists = (float*)malloc(sizeof(float) * (size_t)bs);
        int* dists_i = (int*)malloc(sizeof(int) * (size_t)bs);
        const float* dataset = dataset_all + (size_t)bi * n * 3;
        int32_t* idxs = idxs_all + (size_t)bi * m;
        for (int j = 0; j < m; ++j) idxs[j] = 0;
        for (int k = 0; k < n; ++k) temp[k] = 1e10f;
        int old = 0;
        if (m > 0) idxs[0] = old;
        for (int j = 1; j < m; ++j)
        {
            const float x1 = dataset[old * 3 + 0];
            const float y1 = dataset[old * 3 + 1];
            const float z1 = dataset[old * 3 + 2];
            for (int tid = 0; tid < bs; ++tid)
            {
                int besti = 0;
                float best = -1;
                for (int k = tid; k < n; k += bs)
                {
                    const float x2 = dataset[k * 3 + 0];
                    const float y2 = dataset[k * 3 + 1];
                    const float z2 = dataset[k * 3 + 2];
                    const float mag = sumsq_abc(x2, y2, z2);
                    if ((double)mag <= 1e-3) continue;
                    const float d = sumsq_abc(x2 - x1, y2 - y1, z2 - z1);
                    const float d2 = d < temp[k] ? d : temp[k];
                    temp[k] = d2;
                    besti = d2 > best ? k : besti;
                    best = d2 > best ? d2 : best;
                }
                dists[tid] = best;
                dists_i[tid] = besti;
            }
            for (int s = bs / 2; s >= 1; s >>= 1)
            {
                for (int tid = 0; tid < s; ++tid)
                {
                    const float v1 = dists[tid], v2 = dists[tid + s];
                    const int i1 = dists_i[tid], i2 = dists_i[tid + s];
                    dists[tid] = v1 > v2 ? v1 : v2;
                    dists_i[tid] = v2 > v1 ? i2 : i1;
                }
            }
            old = dists_i[0];
            idxs[j] = old;
        }
        free(temp);
        free(dists);
        free(dists_i);
    }
}

/*
 * Dense ball query, cuda/src/ball_query_gpu.cu:9-52, output initialisation of
 * cuda/src/ball_query.cpp:26-29 (idx zeros, dist -1).
 * pairs_out (optional) receives the number of (centre, candidate) distance
 * evaluations the index-order rule forces: the scan stops after the nsample-th hit.
 */
void orc_ball_query_dense(int b, int n, int m, float radius, int nsample, const float* new_xyz_all,
                          const float* xyz_all, int64_t* idx_all, float* dist_all,
                          int64_t* pairs_out)
{
    const float radius2 = radius * radius;
    int64_t pairs = 0;
#pragma omp parallel for reduction(+ : pairs) schedule(dynamic, 64) collapse(2)
    for (int bi = 0; bi < b; ++bi)
    {
        for (int j = 0; j < m; ++j)
        {
            const float* xyz = xyz_all + (size_t)bi * n * 3;
            const float* q = new_xyz_all + ((size_t)bi * m + j) * 3;
            int64_t* idx_out = idx_all + ((size_t)bi * m + j) * nsample;
            float* dist_out = dist_all + ((size_t)bi * m + j) * nsample;
            for (int l = 0; l < nsample; ++l)
            {
                idx_out[l] = 0;
                dist_out[l] = -1.0f;
            }
            int cnt = 0, k = 0;
            for (; k < n && cnt < nsample; ++k)
            {
                const float d2 = sumsq_abc(q[0] - xyz[k * 3 + 0], q[1] - xyz[k * 3 + 1],
                                           q[2] - xyz[k * 3 + 2]);
                if (d2 < radius2)
                {
                    if (cnt == 0)
                        for (int l = 0; l < nsample; ++l) idx_out[l] = k;
                    idx_out[cnt] = k;
                    dist_out[cnt] = d2;
                    ++cnt;
                }
            }
            pairs += k;
        }
    }
    if (pairs_out) *pairs_out = pairs;
}

/*
 * Partial-dense ball query, cuda/src/ball_query_gpu.cu:54-95.  The reference host
 * code (cuda/src/ball_query.cpp:58-73) fills idx and dist with -1, takes the number
 * of segments from batch_x[-1] + 1 and derives segment offsets from per-segment
 * counts, so batch ids must be sorted.  Test is dist <= r*r, indices are positions
 * in the packed x array.
 */
void orc_ball_query_partial(int64_t size_x, int64_t size_y, float radius, int nsample,
                            const float* x, const float* y, const int64_t* batch_x,
                            const int64_t* batch_y, int64_t* idx_all, float* dist_all,
                            int64_t* pairs_out)
{
    const float radius2 = radius * radius;
    for (int64_t i = 0; i < size_y * nsample; ++i)
    {
        idx_all[i] = -1;
        dist_all[i] = -1.0f;
    }
    if (size_x <= 0)
    {
        if (pairs_out) *pairs_out = 0;
        return;
    }
    const int64_t nseg = batch_x[size_x - 1] + 1;
    int64_t* off_x = (int64_t*)calloc((size_t)nseg + 1, sizeof(int64_t));
    int64_t* off_y = (int64_t*)calloc((size_t)nseg + 1, sizeof(int64_t));
    for (int64_t i = 0; i < size_x; ++i) off_x[batch_x[i] + 1]++;
    for (int64_t i = 0; i < size_y; ++i)
        if (batch_y[i] < nseg) off_y[batch_y[i] + 1]++;
    for (int64_t s = 0; s < nseg; ++s)
    {
        off_x[s + 1] += off_x[s];
        off_y[s + 1] += off_y[s];
    }
    int64_t pairs = 0;
    for (int64_t s = 0; s < nseg; ++s)
    {
#pragma omp parallel for reduction(+ : pairs) schedule(dynamic, 64)
        for (int64_t n_y = off_y[s]; n_y < off_y[s + 1]; ++n_y)
        {
            int64_t count = 0, n_x = off_x[s];
            for (; n_x < off_x[s + 1]; ++n_x)
            {
                const float dist = sumsq_loop(x[n_x * 3 + 0] - y[n_y * 3 + 0],
                                              x[n_x * 3 + 1] - y[n_y * 3 + 1],
                                              x[n_x * 3 + 2] - y[n_y * 3 + 2]);
                if (dist <= radius2)
                {
                    idx_all[n_y * nsample + count] = n_x;
                    dist_all[n_y * nsample + count] = dist;
                    count++;
                }
                if (count >= nsample)
                {
                    ++n_x;
                    break;
                }
            }
            pairs += n_x - off_x[s];
        }
    }
    free(off_x);
    free(off_y);
    if (pairs_out) *pairs_out = pairs;
}

/*
 * three_nn, cuda/src/interpolate_gpu.cu:9-65.  The reference keeps the running
 * bests in doubles initialised to 1e40 but only ever stores float values in them, so
 * float bests initialised to +inf (what (float)1e40 is) compare identically.
 * Returns squared distances; the Python layer takes the square root
 * (torch_points_kernels/torchpoints.py:64).
 */
void orc_three_nn(int b, int n, int m, const float* unknown_all, const float* known_all,
                  float* dist2_all, int32_t* idx_all)
{
#pragma omp parallel for schedule(dynamic, 64) collapse(2)
    for (int bi = 0; bi < b; ++bi)
    {
        for (int j = 0; j < n; ++j)
        {
            const float* known = known_all + (size_t)bi * m * 3;
            const float* u = unknown_all + ((size_t)bi * n + j) * 3;
            float best1 = INFINITY, best2 = INFINITY, best3 = INFINITY;
            int besti1 = 0, besti2 = 0, besti3 = 0;
            for (int k = 0; k < m; ++k)
            {
                const float d = sumsq_abc(u[0] - known[k * 3 + 0], u[1] - known[k * 3 + 1],
                                          u[2] - known[k * 3 + 2]);
                if (d < best1)
                {
                    best3 = best2; besti3 = besti2;
                    best2 = best1; besti2 = besti1;
                    best1 = d;     besti1 = k;
                }
                else if (d < best2)
                {
                    best3 = best2; besti3 = besti2;
                    best2 = d;     besti2 = k;
                }
                else if (d < best3)
                {
                    best3 = d; besti3 = k;
                }
            }
            float* d2 = dist2_all + ((size_t)bi * n + j) * 3;
            int32_t* id = idx_all + ((size_t)bi * n + j) * 3;
            d2[0] = best1; d2[1] = best2; d2[2] = best3;
            id[0] = besti1; id[1] = besti2; id[2] = besti3;
        }
    }
}

/*
 * k nearest neighbours: the result nanoflann's knnSearch returns for
 * cpu/src/knn.cpp:40-59 -> cpu/src/neighbors.cpp:295-339, restated as a brute-force
 * scan.  Distance is L2_Simple_Adaptor's unfused ((dx*dx)+dy*dy)+dz*dz
 * (cpu/include/nanoflann.hpp:488-497); results ascend by distance
 * (KNNResultSet::addPoint, nanoflann.hpp:178-216).  Among exactly equal distances
 * nanoflann keeps kd-tree visit order; this restatement keeps index order, so the
 * two agree on inputs without distance ties.
 * Returns 0, or 1 when k > n_support (the reference raises, cpu/src/knn.cpp:12-14).
 */
int orc_knn(int b, int n_support, int m_query, int k, const float* support_all,
            const float* query_all, int64_t* idx_all, float* dist2_all)
{
    if (k > n_support) return 1;
#pragma omp parallel for schedule(dynamic, 64) collapse(2)
    for (int bi = 0; bi < b; ++bi)
    {
        for (int j = 0; j < m_query; ++j)
        {
            const float* sup = support_all + (size_t)bi * n_support * 3;
            const float* q = query_all + ((size_t)bi * m_query + j) * 3;
            int64_t* idx = idx_all + ((size_t)bi * m_query + j) * k;
            float* dst = dist2_all + ((size_t)bi * m_query + j) * k;
            int cnt = 0;
            for (int s = 0; s < n_support; ++s)
            {
                const float dx = q[0] - sup[s * 3 + 0];
                const float dy = q[1] - sup[s * 3 + 1];
                const float dz = q[2] - sup[s * 3 + 2];
                const float d = ((0.0f + dx * dx) + dy * dy) + dz * dz;
                if (cnt == k && !(d < dst[k - 1])) continue;
                int i = cnt < k ? cnt : k - 1;
                for (; i > 0 && dst[i - 1] > d; --i)
                {
                    dst[i] = dst[i - 1];
                    idx[i] = idx[i - 1];
                }
                dst[i] = d;
                idx[i] = s;
                if (cnt < k) ++cnt;
            }
        }
    }
    return 0;
}

/*
 * three_interpolate forward, cuda/src/interpolate_gpu.cu:78-107:
 * out[b,c,j] = p1*w1 + p2*w2 + p3*w3, contracted by nvcc to fma(p3,w3, fma(p1,w1, p2*w2)).
 */
void orc_three_interpolate(int b, int c, int m, int n, const float* points, const int32_t* idx,
                           const float* weight, float* out)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int bi = 0; bi < b; ++bi)
        for (int l = 0; l < c; ++l)
        {
            const float* p = points + ((size_t)bi * c + l) * m;
            for (int j = 0; j < n; ++j)
            {
                const float* w = weight + ((size_t)bi * n + j) * 3;
                const int32_t* id = idx + ((size_t)bi * n + j) * 3;
                out[((size_t)bi * c + l) * n + j] =
                    fmaf(p[id[2]], w[2], fmaf(p[id[0]], w[0], p[id[1]] * w[1]));
            }
        }
}

/*
 * three_interpolate backward, cuda/src/interpolate_gpu.cu:122-152.  The reference
 * accumulates with fp32 atomics in an unspecified order; the oracle accumulates each
 * fp32 product grad_out*w in double and rounds once, which any order of fp32 adds
 * matches to well within 1e-4.
 */
void orc_three_interpolate_grad(int b, int c, int n, int m, const float* grad_out,
                                const int32_t* idx, const float* weight, float* grad_points)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int bi = 0; bi < b; ++bi)
        for (int l = 0; l < c; ++l)
        {
            double* acc = (double*)calloc((size_t)m, sizeof(double));
            const float* g = grad_out + ((size_t)bi * c + l) * n;
            for (int j = 0; j < n; ++j)
            {
                const float* w = weight + ((size_t)bi * n + j) * 3;
                const int32_t* id = idx + ((size_t)bi * n + j) * 3;
                acc[id[0]] += (double)(g[j] * w[0]);
                acc[id[1]] += (double)(g[j] * w[1]);
                acc[id[2]] += (double)(g[j] * w[2]);
            }
            for (int i = 0; i < m; ++i) grad_points[((size_t)bi * c + l) * m + i] = (float)acc[i];
            free(acc);
        }
}

/*
 * grouping_operation forward, torch_points_kernels/torchpoints.py:129-146:
 * out[b,c,p,s] = features[b,c,idx[b,p,s]]  (a pure copy).
 */
void orc_grouping(int b, int c, int n, int npoint, int nsample, const float* features,
                  const int64_t* idx, float* out)
{
    const size_t ps = (size_t)npoint * nsample;
#pragma omp parallel for schedule(static) collapse(2)
    for (int bi = 0; bi < b; ++bi)
        for (int l = 0; l < c; ++l)
        {
            const float* f = features + ((size_t)bi * c + l) * n;
            const int64_t* id = idx + (size_t)bi * ps;
            float* o = out + ((size_t)bi * c + l) * ps;
            for (size_t i = 0; i < ps; ++i) o[i] = f[id[i]];
        }
}

/*
 * grouping_operation backward: autograd's gather backward for
 * torch_points_kernels/torchpoints.py:145, grad_features[b,c,idx[b,p,s]] += grad_out[b,c,p,s],
 * accumulated in double and rounded once.
 */
void orc_grouping_grad(int b, int c, int n, int npoint, int nsample, const float* grad_out,
                       const int64_t* idx, float* grad_features)
{
    const size_t ps = (size_t)npoint * nsample;
#pragma omp parallel for schedule(static) collapse(2)
    for (int bi = 0; bi < b; ++bi)
        for (int l = 0; l < c; ++l)
        {
            double* acc = (double*)calloc((size_t)n, sizeof(double));
            const float* g = grad_out + ((size_t)bi * c + l) * ps;
            const int64_t* id = idx + (size_t)bi * ps;
            for (size_t i = 0; i < ps; ++i) acc[id[i]] += (double)g[i];
            for (int i = 0; i < n; ++i) grad_features[((size_t)bi * c + l) * n + i] = (float)acc[i];
            free(acc);
        }
}

/*
 * One direction of the chamfer kernel, cuda/src/chamfer_dist_gpu.cu:8-155: for each
 * point of cloud 1 the smallest squared distance to cloud 2 and its index.  Within a
 * 512-point tile the comparison is strict (<) from the tile's first element, and a
 * later tile replaces the stored result only when strictly smaller (:146), so the
 * lowest index wins among equal minima.  Differences are taken as (p2 - p1) (:38-41).
 * With m == 0 the reference writes nothing and the zero-initialised outputs remain.
 */
void orc_chamfer_dir(int b, int n, const float* xyz1, int m, const float* xyz2, float* dist,
                     int32_t* indexes)
{
#pragma omp parallel for schedule(dynamic, 64) collapse(2)
    for (int bi = 0; bi < b; ++bi)
        for (int j = 0; j < n; ++j)
        {
            const float* p1 = xyz1 + ((size_t)bi * n + j) * 3;
            const float* c2 = xyz2 + (size_t)bi * m * 3;
            float best = 0;
            int besti = 0;
            for (int k = 0; k < m; ++k)
            {
                const float d = sumsq_abc(c2[k * 3 + 0] - p1[0], c2[k * 3 + 1] - p1[1],
                                          c2[k * 3 + 2] - p1[2]);
                if (k == 0 || d < best)
                {
                    best = d;
                    besti = k;
                }
            }
            dist[(size_t)bi * n + j] = best;
            indexes[(size_t)bi * n + j] = besti;
        }
}

/* Same in double precision (the reference dispatches float and double,
 * cuda/src/chamfer_dist_gpu.cu:167-176; its gradcheck test runs in double). */
void orc_chamfer_dir_f64(int b, int n, const double* xyz1, int m, const double* xyz2, double* dist,
                         int32_t* indexes)
{
    for (int bi = 0; bi < b; ++bi)
        for (int j = 0; j < n; ++j)
        {
            const double* p1 = xyz1 + ((size_t)bi * n + j) * 3;
            const double* c2 = xyz2 + (size_t)bi * m * 3;
            double best = 0;
            int besti = 0;
            for (int k = 0; k < m; ++k)
            {
                const double a = c2[k * 3 + 0] - p1[0], bb = c2[k * 3 + 1] - p1[1],
                             cc = c2[k * 3 + 2] - p1[2];
                const double d = fma(cc, cc, fma(a, a, bb * bb));
                if (k == 0 || d < best)
                {
                    best = d;
                    besti = k;
                }
            }
            dist[(size_t)bi * n + j] = best;
            indexes[(size_t)bi * n + j] = besti;
        }
}

/*
 * Chamfer backward, cuda/src/chamfer_dist_gpu.cu:186-245: both launches folded into
 * one pass.  g = 2*grad_dist[j]; grad_xyz1[j] += g*(p1-p2); grad_xyz2[idx1[j]] -= g*(p1-p2),
 * then the same with the clouds swapped.  Products are fp32 as in the kernel; the sums
 * are taken in double and rounded once.
 */
void orc_chamfer_grad(int b, int n, const float* xyz1, int m, const float* xyz2,
                      const int32_t* idx1, const int32_t* idx2, const float* grad_dist1,
                      const float* grad_dist2, float* grad_xyz1, float* grad_xyz2)
{
    for (int bi = 0; bi < b; ++bi)
    {
        double* a1 = (double*)calloc((size_t)n * 3 + 1, sizeof(double));
        double* a2 = (double*)calloc((size_t)m * 3 + 1, sizeof(double));
        const float* p1 = xyz1 + (size_t)bi * n * 3;
        const float* p2 = xyz2 + (size_t)bi * m * 3;
        for (int j = 0; j < n; ++j)
        {
            const int j2 = idx1[(size_t)bi * n + j];
            const float g = grad_dist1[(size_t)bi * n + j] * 2;
            for (int d = 0; d < 3; ++d)
            {
                const float t = g * (p1[j * 3 + d] - p2[j2 * 3 + d]);
                a1[j * 3 + d] += (double)t;
                a2[j2 * 3 + d] += (double)(-t);
            }
        }
        for (int j = 0; j < m; ++j)
        {
            const int j2 = idx2[(size_t)bi * m + j];
            const float g = grad_dist2[(size_t)bi * m + j] * 2;
            for (int d = 0; d < 3; ++d)
            {
                const float t = g * (p2[j * 3 + d] - p1[j2 * 3 + d]);
                a2[j * 3 + d] += (double)t;
                a1[j2 * 3 + d] += (double)(-t);
            }
        }
        for (int i = 0; i < n * 3; ++i) grad_xyz1[(size_t)bi * n * 3 + i] = (float)a1[i];
        for (int i = 0; i < m * 3; ++i) grad_xyz2[(size_t)bi * m * 3 + i] = (float)a2[i];
        free(a1);
        free(a2);
    }
}

/* ------------------------------------------------------------------ region growing
 *
 * torch_points_kernels/cluster.py:8-37 (_grow_proximity_core), literally: seeds in index
 * order, a stack ("queue.pop()" takes the last element), a neighbour list ends at the first
 * -1.  Writes the members of the clusters that reach min_cluster_size one after the other
 * into `members`, in the order the traversal met them, and cluster c's range into
 * offsets[c], offsets[c + 1].  Returns the number of clusters kept.
 */
int64_t orc_grow_proximity(int64_t n, int nsample, const int64_t* neighbours, int64_t min_cluster_size,
                           int64_t* members, int64_t* offsets)
{
    unsigned char* visited = (unsigned char*)calloc((size_t)n + 1, 1);
    int64_t* stack = (int64_t*)malloc(sizeof(int64_t) * ((size_t)n + 1));
    int64_t* cluster = (int64_t*)malloc(sizeof(int64_t) * ((size_t)n + 1));
    int64_t nclusters = 0, written = 0;
    offsets[0] = 0;
    for (int64_t i = 0; i < n; ++i)
    {
        if (visited[i]) continue;
        int64_t top = 0, size = 0;
        visited[i] = 1;
        stack[top++] = i;
        cluster[size++] = i;
        while (top > 0)
        {
            const int64_t k = stack[--top];
            for (int s = 0; s < nsample; ++s)
            {
                const int64_t nei = neighbours[k * nsample + s];
                if (nei == -1) break;
                if (!visited[nei])
                {
                    visited[nei] = 1;
                    stack[top++] = nei;
                    cluster[size++] = nei;
                }
            }
        }
        if (size >= min_cluster_size)
        {
            for (int64_t j = 0; j < size; ++j) members[written + j] = cluster[j];
            written += size;
            offsets[++nclusters] = written;
        }
    }
    free(visited);
    free(stack);
    free(cluster);
    return nclusters;
}

/* ------------------------------------------------------------------ instance IoU
 *
 * cuda/src/metrics_gpu.cu:9-43: per proposal and ground-truth instance of the proposal's
 * sample, intersection / (float)(|proposal| + |instance| - intersection) + 1e-5, the division
 * in double, stored as float.  out (n_proposals, total_gt) starts from zero.
 */
void orc_instance_iou(int n_proposals, int64_t total_gt, const int64_t* num_gt, const int64_t* proposals_idx,
                      const int64_t* proposals_offset, const int64_t* instance_labels, const int64_t* offset_num_gt,
                      const int64_t* batch, const int64_t* instance_pointnum, float* out)
{
    for (int64_t i = 0; i < (int64_t)n_proposals * total_gt; ++i) out[i] = 0.f;
    for (int p = 0; p < n_proposals; ++p)
    {
        const int start = (int)proposals_offset[p], end = (int)proposals_offset[p + 1];
        const int sample = (int)batch[proposals_idx[start]];
        const int ninst = (int)num_gt[sample];
        const int inst_off = (int)offset_num_gt[sample];
        const int proposal_total = end - start;
        for (int inst = 0; inst < ninst; ++inst)
        {
            const int inst_total = (int)instance_pointnum[inst_off + inst];
            int inter = 0;
            for (int i = start; i < end; ++i)
                if ((int)instance_labels[proposals_idx[i]] == inst + 1) inter += 1;
            out[inst_off + inst + (int64_t)p * total_gt] =
                (float)((float)inter / ((float)(proposal_total + inst_total - inter) + 1e-5));
        }
    }
}

/* ------------------------------------------------------------------ gridding (float32)
 *
 * cuda/src/gridding_gpu.cu:28-161 forward, :199-304 backward.  Vertices outside the grid get
 * index -1 and are left out (the reference writes out of bounds there).  The forward sums are
 * taken in double and rounded once (the kernel adds with atomics in arbitrary order); the
 * backward sums run over the eight vertices in the kernel's order, in float.
 */
static float orc_vertex_weight(float x, int x0) { return 1 - fabsf(x - (float)x0); }

void orc_gridding(int b, int n_pts, float min_x, float max_x, float min_y, float max_y, float min_z, float max_z,
                  const float* ptcloud, float* grid, float* grid_pt_weights, int32_t* grid_pt_indexes)
{
    const int len_x = (int)(max_x - min_x + 1), len_y = (int)(max_y - min_y + 1), len_z = (int)(max_z - min_z + 1);
    const int64_t nv = (int64_t)len_x * len_y * len_z;
    double* acc = (double*)calloc((size_t)nv + 1, sizeof(double));
    for (int bi = 0; bi < b; ++bi)
    {
        for (int64_t i = 0; i < nv; ++i) acc[i] = 0.0;
        for (int j = 0; j < n_pts; ++j)
        {
            const size_t t = (size_t)bi * n_pts + j;
            const float p[3] = {ptcloud[t * 3 + 0], ptcloud[t * 3 + 1], ptcloud[t * 3 + 2]};
            const float mn[3] = {min_x, min_y, min_z};
            int off[2][3];
            float w[2][3];
            for (int a = 0; a < 3; ++a)
            {
                int lower = (int)floorf(p[a]), upper = (int)ceilf(p[a]);
                if (lower == upper) upper += 1;
                off[0][a] = (int)(lower - mn[a]);
                off[1][a] = (int)(upper - mn[a]);
                w[0][a] = orc_vertex_weight(p[a], lower);
                w[1][a] = orc_vertex_weight(p[a], upper);
            }
            for (int v = 0; v < 8; ++v)
            {
                const int ux = (v >> 2) & 1, uy = (v >> 1) & 1, uz = v & 1;
                const int ox = off[ux][0], oy = off[uy][1], oz = off[uz][2];
                const int inside = ox >= 0 && ox < len_x && oy >= 0 && oy < len_y && oz >= 0 && oz < len_z;
                const int index = inside ? (ox * len_y + oy) * len_z + oz : -1;
                grid_pt_indexes[t * 8 + v] = index;
                grid_pt_weights[t * 24 + v * 3 + 0] = w[ux][0];
                grid_pt_weights[t * 24 + v * 3 + 1] = w[uy][1];
                grid_pt_weights[t * 24 + v * 3 + 2] = w[uz][2];
                if (inside)
                {
                    const float prod = (w[ux][0] * w[uy][1]) * w[uz][2];
                    acc[index] += (double)prod;
                }
            }
        }
        for (int64_t i = 0; i < nv; ++i) grid[(size_t)bi * nv + i] = (float)acc[i];
    }
    free(acc);
}

void orc_gridding_grad(int b, int n_pts, int64_t n_grid_vertices, const float* grid_pt_weights,
                       const int32_t* grid_pt_indexes, const float* grad_grid, float* grad_ptcloud)
{
    for (int bi = 0; bi < b; ++bi)
        for (int j = 0; j < n_pts; ++j)
        {
            const size_t t = (size_t)bi * n_pts + j;
            float gx = 0, gy = 0, gz = 0;
            for (int v = 0; v < 8; ++v)
            {
                const int index = grid_pt_indexes[t * 8 + v];
                if (index < 0) continue;
                const float g = grad_grid[(size_t)bi * n_grid_vertices + index];
                const float wx = grid_pt_weights[t * 24 + v * 3 + 0], wy = grid_pt_weights[t * 24 + v * 3 + 1],
                            wz = grid_pt_weights[t * 24 + v * 3 + 2];
                const float sx = ((v >> 2) & 1) ? g : -g, sy = ((v >> 1) & 1) ? g : -g, sz = (v & 1) ? g : -g;
                gx = gx + (sx * wy) * wz;
                gy = gy + (sy * wx) * wz;
                gz = gz + (sz * wx) * wy;
            }
            grad_ptcloud[t * 3 + 0] = gx;
            grad_ptcloud[t * 3 + 1] = gy;
            grad_ptcloud[t * 3 + 2] = gz;
        }
}

/* ------------------------------------------------------------------ cubic feature sampling (float32)
 *
 * cuda/src/cubic_feature_sampling_gpu.cu:22-97 forward (copies, exact), :130-177 backward
 * (scatter-add, summed in double here and rounded once).
 */
void orc_cubic_feature_sampling(int b, int n_pts, int channels, int scale, int neighborhood_size, const float* ptcloud,
                                const float* cubic_features, float* point_features, int32_t* grid_pt_indexes)
{
    const int ns = neighborhood_size - 1, side = 2 * neighborhood_size, nvert = side * side * side;
    const int64_t cub = (int64_t)scale * scale * scale;
    for (int bi = 0; bi < b; ++bi)
        for (int i = 0; i < n_pts; ++i)
        {
            const size_t t = (size_t)bi * n_pts + i;
            int lo[3];
            for (int a = 0; a < 3; ++a) lo[a] = (int)floorf(ptcloud[t * 3 + a]);
            int vertex = 0;
            for (int j = lo[0] - ns; j < lo[0] - ns + side; ++j)
                for (int k = lo[1] - ns; k < lo[1] - ns + side; ++k)
                    for (int m = lo[2] - ns; m < lo[2] - ns + side; ++m)
                    {
                        const int outside = j < 0 || j >= scale || k < 0 || k >= scale || m < 0 || m >= scale;
                        const int index = outside ? -1 : (j * scale + k) * scale + m;
                        grid_pt_indexes[t * nvert + vertex] = index;
                        for (int c = 0; c < channels; ++c)
                            point_features[(t * nvert + vertex) * channels + c] =
                                outside ? 0.f : cubic_features[((size_t)bi * channels + c) * cub + index];
                        ++vertex;
                    }
        }
}

void orc_cubic_feature_sampling_grad(int b, int n_pts, int channels, int scale, int neighborhood_size,
                                     const float* grad_point_features, const int32_t* grid_pt_indexes,
                                     float* grad_cubic_features)
{
    const int side = 2 * neighborhood_size, nvert = side * side * side;
    const int64_t cub = (int64_t)scale * scale * scale;
    double* acc = (double*)calloc((size_t)channels * cub + 1, sizeof(double));
    for (int bi = 0; bi < b; ++bi)
    {
        for (int64_t i = 0; i < channels * cub; ++i) acc[i] = 0.0;
        for (int i = 0; i < n_pts; ++i)
            for (int j = 0; j < nvert; ++j)
            {
                const size_t pv = ((size_t)bi * n_pts + i) * nvert + j;
                const int index = grid_pt_indexes[pv];
                if (index < 0) continue;
                for (int c = 0; c < channels; ++c) acc[c * cub + index] += (double)grad_point_features[pv * channels + c];
            }
        for (int64_t i = 0; i < channels * cub; ++i) grad_cubic_features[(size_t)bi * channels * cub + i] = (float)acc[i];
    }
    free(acc);
}
