// Chamfer distance for sm_100a: nearest neighbour in the other cloud (both directions)
// and its gradient.
//
// Forward is an all-pairs arg-min on the FP32 pipe, query-tiled over shared-memory
// candidate tiles (scan.cuh): with three coordinates per point there is no contraction
// dimension worth a tensor core.  Each direction is one launch whose grid covers all
// (batch, query-tile) pairs, so the B200 is full even for small batches.  The f64
// variant (used by gradient checks) is a plain one-thread-per-point loop.
//
// Backward folds the reference's two launches into one: every point adds its own term
// and scatters the opposite term to its nearest neighbour with red.global.add.
//
// forward  : cuda/src/chamfer_dist_gpu.cu:8-155   (strict '<' => lowest index among equal minima)
// backward : cuda/src/chamfer_dist_gpu.cu:186-245
#include <math_constants.h>

#include "scan.cuh"

namespace tpk
{
// grid_query.cu
size_t grid_three_nn_scratch_bytes(int b, int n, int m);
int grid_nn(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2,
            int32_t* idx, void* scratch, const unsigned char** need_scan_out, cudaStream_t s);
// smem_grid.cu
bool sg_three_nn_fits(int m);
int sg_nn(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
          unsigned char* need, cudaStream_t s);
bool sg_nn_slab_fits(int b, int n, int m);
int sg_nn_slab(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
               unsigned char* need, cudaStream_t s);

namespace
{

template <int Q>
struct ArgMinOp
{
    float qx[Q], qy[Q], qz[Q];
    float best[Q];
    int besti[Q];
    bool act[Q];

    __device__ __forceinline__ float threshold(int q) const { return act[q] ? best[q] : -CUDART_INF_F; }
    __device__ __forceinline__ bool finished() const
    {
        bool done = true;
#pragma unroll
        for (int q = 0; q < Q; ++q) done &= !act[q];
        return done;
    }
    __device__ __forceinline__ bool exact(int q, long long k, float cx, float cy, float cz)
    {
        const float d = sumsq_abc(cx - qx[q], cy - qy[q], cz - qz[q]);
        if (!act[q] || !(d < best[q])) return false;
        best[q] = d;
        besti[q] = static_cast<int>(k);
        return true;
    }
};

template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    chamfer_f32_kernel(int n, int m, int tiles_per_cloud, const float* __restrict__ xyz1,
                       const float* __restrict__ xyz2, float* __restrict__ dist,
                       int32_t* __restrict__ indexes, const unsigned char* __restrict__ need)
{
    __shared__ __align__(16) float smem[2 * kScanTileFloats];
    const int cloud = blockIdx.x / tiles_per_cloud;
    const int qtile = blockIdx.x - cloud * tiles_per_cloud;
    ArgMinOp<Q> op;
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        // `need` (optional): one byte per point, 0 = already answered by the grid path
        op.act[q] = j < n && (need == nullptr || need[static_cast<size_t>(cloud) * n + j] != 0);
        const size_t row = static_cast<size_t>(cloud) * n + (op.act[q] ? j : 0);
        op.qx[q] = op.act[q] ? __ldg(xyz1 + row * 3 + 0) : 0.f;
        op.qy[q] = op.act[q] ? __ldg(xyz1 + row * 3 + 1) : 0.f;
        op.qz[q] = op.act[q] ? __ldg(xyz1 + row * 3 + 2) : 0.f;
        op.best[q] = CUDART_INF_F;
        op.besti[q] = 0;
    }
    if (need != nullptr)
    {
        // nothing left over for this CTA (the usual case behind the grid kernel): leave
        // before staging a single tile
        bool any = false;
#pragma unroll
        for (int q = 0; q < Q; ++q) any |= op.act[q];
        if (!__syncthreads_or(any ? 1 : 0)) return;
    }
    scan_candidates<THREADS, Q>(xyz2 + static_cast<size_t>(cloud) * m * 3, m, smem, op.qx, op.qy, op.qz, op);
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        if (!op.act[q]) continue;
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        const size_t o = static_cast<size_t>(cloud) * n + j;
        dist[o] = op.best[q];
        indexes[o] = op.besti[q];
    }
}

__global__ void __launch_bounds__(128)
    chamfer_f64_kernel(int b, int n, int m, const double* __restrict__ xyz1,
                       const double* __restrict__ xyz2, double* __restrict__ dist,
                       int32_t* __restrict__ indexes)
{
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(b) * n) return;
    const int bi = static_cast<int>(t / n);
    const double x1 = xyz1[t * 3 + 0], y1 = xyz1[t * 3 + 1], z1 = xyz1[t * 3 + 2];
    const double* c2 = xyz2 + static_cast<size_t>(bi) * m * 3;
    double best = 0.0;
    int besti = 0;
    for (int k = 0; k < m; ++k)
    {
        const double d = sumsq_abc(c2[k * 3 + 0] - x1, c2[k * 3 + 1] - y1, c2[k * 3 + 2] - z1);
        if (k == 0 || d < best)
        {
            best = d;
            besti = k;
        }
    }
    dist[t] = best;
    indexes[t] = besti;
}

template <typename T>
__global__ void __launch_bounds__(256)
    chamfer_grad_kernel(int b, int n, int m, const T* __restrict__ xyz1, const T* __restrict__ xyz2,
                        const int32_t* __restrict__ idx1, const int32_t* __restrict__ idx2,
                        const T* __restrict__ gd1, const T* __restrict__ gd2,
                        T* __restrict__ grad1, T* __restrict__ grad2)
{
    const long long per = static_cast<long long>(n) + m;
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= per * b) return;
    const int bi = static_cast<int>(t / per);
    const long long r = t - bi * per;
    const bool first = r < n;
    const int j = static_cast<int>(first ? r : r - n);
    const int na = first ? n : m, nb = first ? m : n;
    const T* pa = (first ? xyz1 : xyz2) + (static_cast<size_t>(bi) * na + j) * 3;
    const int j2 = (first ? idx1 : idx2)[static_cast<size_t>(bi) * na + j];
    const T* pb = (first ? xyz2 : xyz1) + (static_cast<size_t>(bi) * nb + j2) * 3;
    const T g = (first ? gd1 : gd2)[static_cast<size_t>(bi) * na + j] * T(2);
    T* ga = (first ? grad1 : grad2) + (static_cast<size_t>(bi) * na + j) * 3;
    T* gb = (first ? grad2 : grad1) + (static_cast<size_t>(bi) * nb + j2) * 3;
#pragma unroll
    for (int d = 0; d < 3; ++d)
    {
        const T v = g * (pa[d] - pb[d]);
        atomicAdd(ga + d, v);
        atomicAdd(gb + d, -v);
    }
}

int chamfer_dir_f32(int b, int n, const float* xyz1, int m, const float* xyz2, float* dist,
                    int32_t* idx, const unsigned char* need, cudaStream_t s)
{
    if (b == 0 || n == 0) return TPK_OK;
    if (m == 0)
    {
        // the reference leaves its zero-initialised outputs untouched when the other cloud is empty
        cudaError_t e1 = cudaMemsetAsync(dist, 0, sizeof(float) * static_cast<size_t>(b) * n, s);
        cudaError_t e2 = cudaMemsetAsync(idx, 0, sizeof(int32_t) * static_cast<size_t>(b) * n, s);
        if (e1 != cudaSuccess || e2 != cudaSuccess)
        {
            set_error("chamfer_dist: memset failed");
            return TPK_ERR_CUDA;
        }
        return TPK_OK;
    }
    const long long queries = static_cast<long long>(b) * n;
    const int q = queries >= 300000 ? 2 : 1;
    const int threads = queries >= 32768 ? 128 : 64;
    const int tiles = (n + threads * q - 1) / (threads * q);
    const long long grid = static_cast<long long>(b) * tiles;
    TPK_REQUIRE(grid < (1ll << 31), "chamfer_dist: too many points");
    const dim3 g(static_cast<unsigned>(grid));
    if (threads == 128 && q == 2)
    {
        prefer_max_shared(chamfer_f32_kernel<128, 2>);
        count_launches(1), chamfer_f32_kernel<128, 2><<<g, 128, 0, s>>>(n, m, tiles, xyz1, xyz2, dist, idx, need);
    }
    else if (threads == 128)
    {
        prefer_max_shared(chamfer_f32_kernel<128, 1>);
        count_launches(1), chamfer_f32_kernel<128, 1><<<g, 128, 0, s>>>(n, m, tiles, xyz1, xyz2, dist, idx, need);
    }
    else if (q == 2)
    {
        prefer_max_shared(chamfer_f32_kernel<64, 2>);
        count_launches(1), chamfer_f32_kernel<64, 2><<<g, 64, 0, s>>>(n, m, tiles, xyz1, xyz2, dist, idx, need);
    }
    else
    {
        prefer_max_shared(chamfer_f32_kernel<64, 1>);
        count_launches(1), chamfer_f32_kernel<64, 1><<<g, 64, 0, s>>>(n, m, tiles, xyz1, xyz2, dist, idx, need);
    }
    return check_launch("chamfer_dist");
}

int chamfer_dir_f64(int b, int n, const double* xyz1, int m, const double* xyz2, double* dist,
                    int32_t* idx, cudaStream_t s)
{
    if (b == 0 || n == 0) return TPK_OK;
    if (m == 0)
    {
        cudaError_t e1 = cudaMemsetAsync(dist, 0, sizeof(double) * static_cast<size_t>(b) * n, s);
        cudaError_t e2 = cudaMemsetAsync(idx, 0, sizeof(int32_t) * static_cast<size_t>(b) * n, s);
        if (e1 != cudaSuccess || e2 != cudaSuccess)
        {
            set_error("chamfer_dist: memset failed");
            return TPK_ERR_CUDA;
        }
        return TPK_OK;
    }
    const long long total = static_cast<long long>(b) * n;
    const long long grid = (total + 127) / 128;
    TPK_REQUIRE(grid < (1ll << 31), "chamfer_dist: too many points");
    count_launches(1), chamfer_f64_kernel<<<static_cast<unsigned>(grid), 128, 0, s>>>(b, n, m, xyz1, xyz2, dist, idx);
    return check_launch("chamfer_dist_f64");
}

template <typename T>
int chamfer_grad_t(int b, int n, const T* xyz1, int m, const T* xyz2, const int32_t* idx1,
                   const int32_t* idx2, const T* gd1, const T* gd2, T* g1, T* g2, cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "chamfer_dist_grad: negative size");
    if (b == 0) return TPK_OK;
    TPK_REQUIRE((g1 || n == 0) && (g2 || m == 0), "chamfer_dist_grad: NULL pointer");
    cudaError_t e1 = n ? cudaMemsetAsync(g1, 0, sizeof(T) * static_cast<size_t>(b) * n * 3, s) : cudaSuccess;
    cudaError_t e2 = m ? cudaMemsetAsync(g2, 0, sizeof(T) * static_cast<size_t>(b) * m * 3, s) : cudaSuccess;
    if (e1 != cudaSuccess || e2 != cudaSuccess)
    {
        set_error("chamfer_dist_grad: memset failed");
        return TPK_ERR_CUDA;
    }
    // with an empty cloud there is no nearest neighbour to differentiate through
    if (n == 0 || m == 0) return TPK_OK;
    TPK_REQUIRE(xyz1 && xyz2 && idx1 && idx2 && gd1 && gd2, "chamfer_dist_grad: NULL pointer");
    const long long total = (static_cast<long long>(n) + m) * b;
    const long long grid = (total + 255) / 256;
    TPK_REQUIRE(grid < (1ll << 31), "chamfer_dist_grad: too many points");
    count_launches(1), chamfer_grad_kernel<T><<<static_cast<unsigned>(grid), 256, 0, s>>>(b, n, m, xyz1, xyz2, idx1, idx2,
                                                                      gd1, gd2, g1, g2);
    return check_launch("chamfer_dist_grad");
}

}  // namespace
}  // namespace tpk

extern "C" int tpk_chamfer_dist_f32(int b, int n, const float* xyz1, int m, const float* xyz2,
                                    float* dist1, float* dist2, int32_t* idx1, int32_t* idx2,
                                    void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "chamfer_dist: negative size");
    TPK_REQUIRE(b == 0 || ((n == 0 || (xyz1 && dist1 && idx1)) && (m == 0 || (xyz2 && dist2 && idx2))),
                "chamfer_dist: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = chamfer_dir_f32(b, n, xyz1, m, xyz2, dist1, idx1, nullptr, s);
    if (rc != TPK_OK) return rc;
    return chamfer_dir_f32(b, m, xyz2, n, xyz1, dist2, idx2, nullptr, s);
}

// The grid pays from about a thousand candidates per cloud on (the test hook "chamfer_scan" forces the scan).
static bool chamfer_wants_grid(int known) { return known >= 1024 && !tpk::test_path("chamfer_scan"); }

// the test hook "nn_global_grid" keeps clouds above 8192 points on the grid in global memory
// (comparison runs and tests of that path)
static bool chamfer_by_layers(int b, int queries, int known)
{
    return tpk::sg_nn_slab_fits(b, queries, known) && !tpk::test_path("nn_global_grid");
}

// scratch of one direction: one flag per query with the grid in shared memory (whole cloud
// up to 8192 candidates, by layers above), the whole grid where it has to live in global memory
static size_t chamfer_dir_scratch(int b, int queries, int known)
{
    if (!chamfer_wants_grid(known)) return 0;
    if (tpk::sg_three_nn_fits(known) || chamfer_by_layers(b, queries, known))
        return (static_cast<size_t>(b) * queries + 255) / 256 * 256;
    return tpk::grid_three_nn_scratch_bytes(b, queries, known);
}

extern "C" int64_t tpk_chamfer_dist_scratch_bytes(int b, int n, int m)
{
    if (b <= 0 || n <= 0 || m <= 0) return 0;
    // the two directions run one after the other on the same scratch
    const size_t d1 = chamfer_dir_scratch(b, n, m), d2 = chamfer_dir_scratch(b, m, n);
    return static_cast<int64_t>(d1 > d2 ? d1 : d2);
}

// One direction on the grid of the `known` cloud; *need = flags of the points left to the scan.
static int chamfer_dir_grid(int b, int queries, const float* q, int known, const float* c, float* dist,
                            int32_t* idx, void* scratch, const unsigned char** need, cudaStream_t s)
{
    *need = nullptr;
    if (!chamfer_wants_grid(known)) return TPK_OK;
    if (tpk::sg_three_nn_fits(known))
    {
        *need = static_cast<const unsigned char*>(scratch);
        return tpk::sg_nn(1, b, queries, known, q, c, dist, idx, static_cast<unsigned char*>(scratch), s);
    }
    if (chamfer_by_layers(b, queries, known))
    {
        *need = static_cast<const unsigned char*>(scratch);
        return tpk::sg_nn_slab(1, b, queries, known, q, c, dist, idx, static_cast<unsigned char*>(scratch), s);
    }
    return tpk::grid_nn(1, b, queries, known, q, c, dist, idx, scratch, need, s);
}

extern "C" int tpk_chamfer_dist_f32_ws(int b, int n, const float* xyz1, int m, const float* xyz2,
                                       float* dist1, float* dist2, int32_t* idx1, int32_t* idx2,
                                       void* scratch, int64_t scratch_bytes, void* stream)
{
    using namespace tpk;
    const int64_t want = tpk_chamfer_dist_scratch_bytes(b, n, m);
    if (want == 0 || scratch == nullptr)
        return tpk_chamfer_dist_f32(b, n, xyz1, m, xyz2, dist1, dist2, idx1, idx2, stream);
    if (scratch_bytes < want)
    {
        set_error("chamfer_dist: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch_bytes),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE(xyz1 && xyz2 && dist1 && dist2 && idx1 && idx2, "chamfer_dist: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "chamfer_dist: scratch must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // per direction: nearest neighbour on the uniform grid of the other cloud, then the
    // all-pairs scan for the points the grid handed back (non-finite coordinates, degenerate clouds)
    const unsigned char* need = nullptr;
    int rc = chamfer_dir_grid(b, n, xyz1, m, xyz2, dist1, idx1, scratch, &need, s);
    if (rc != TPK_OK) return rc;
    rc = chamfer_dir_f32(b, n, xyz1, m, xyz2, dist1, idx1, need, s);
    if (rc != TPK_OK) return rc;
    rc = chamfer_dir_grid(b, m, xyz2, n, xyz1, dist2, idx2, scratch, &need, s);
    if (rc != TPK_OK) return rc;
    return chamfer_dir_f32(b, m, xyz2, n, xyz1, dist2, idx2, need, s);
}

extern "C" int tpk_chamfer_dist_f64(int b, int n, const double* xyz1, int m, const double* xyz2,
                                    double* dist1, double* dist2, int32_t* idx1, int32_t* idx2,
                                    void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "chamfer_dist: negative size");
    TPK_REQUIRE(b == 0 || ((n == 0 || (xyz1 && dist1 && idx1)) && (m == 0 || (xyz2 && dist2 && idx2))),
                "chamfer_dist: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = chamfer_dir_f64(b, n, xyz1, m, xyz2, dist1, idx1, s);
    if (rc != TPK_OK) return rc;
    return chamfer_dir_f64(b, m, xyz2, n, xyz1, dist2, idx2, s);
}

extern "C" int tpk_chamfer_dist_grad_f32(int b, int n, const float* xyz1, int m, const float* xyz2,
                                         const int32_t* idx1, const int32_t* idx2,
                                         const float* grad_dist1, const float* grad_dist2,
                                         float* grad_xyz1, float* grad_xyz2, void* stream)
{
    return tpk::chamfer_grad_t<float>(b, n, xyz1, m, xyz2, idx1, idx2, grad_dist1, grad_dist2,
                                      grad_xyz1, grad_xyz2, static_cast<cudaStream_t>(stream));
}

extern "C" int tpk_chamfer_dist_grad_f64(int b, int n, const double* xyz1, int m,
                                         const double* xyz2, const int32_t* idx1,
                                         const int32_t* idx2, const double* grad_dist1,
                                         const double* grad_dist2, double* grad_xyz1,
                                         double* grad_xyz2, void* stream)
{
    return tpk::chamfer_grad_t<double>(b, n, xyz1, m, xyz2, idx1, idx2, grad_dist1, grad_dist2,
                                       grad_xyz1, grad_xyz2, static_cast<cudaStream_t>(stream));
}
