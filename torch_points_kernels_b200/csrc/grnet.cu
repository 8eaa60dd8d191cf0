// Gridding and cubic feature sampling (the GRNet ops next to Chamfer distance) for sm_100a.
//
// gridding              : cuda/src/gridding_gpu.cu:28-304 of the reference
// cubic_feature_sampling: cuda/src/cubic_feature_sampling_gpu.cu:22-177
//
// The reference runs one CTA per cloud.  Here a thread owns a point (index and weight
// computation, the gridding gradient) or one output element (the feature gather and its
// scatter), the grid covers every cloud of the batch, and the accumulating stores are
// fire-and-forget global reductions.  Arithmetic follows the reference expression by
// expression (weights 1 - |x - x0|, products left to right, the gridding gradient summed
// over the eight vertices in the reference's order), so everything that does not depend
// on the order of atomic additions is bit-identical.
//
// One deliberate difference: the reference writes outside its tensors when a point lies
// outside the grid (no bounds check on the eight vertex indices).  Here a vertex outside the
// grid gets index -1 and contributes nothing, forward and backward.
#include <type_traits>

#include "tpk_common.cuh"

namespace tpk
{
TPK_DEFINE_STATUS_WORD()

namespace
{

constexpr int kGrThreads = 256;

template <class T>
__device__ __forceinline__ T mul_rn(T a, T b);
template <>
__device__ __forceinline__ float mul_rn<float>(float a, float b)
{
    return __fmul_rn(a, b);
}
template <>
__device__ __forceinline__ double mul_rn<double>(double a, double b)
{
    return __dmul_rn(a, b);
}
template <class T>
__device__ __forceinline__ T add_rn(T a, T b);
template <>
__device__ __forceinline__ float add_rn<float>(float a, float b)
{
    return __fadd_rn(a, b);
}
template <>
__device__ __forceinline__ double add_rn<double>(double a, double b)
{
    return __dadd_rn(a, b);
}

// floor / ceil of a coordinate as the reference takes them: int lower = floor(x), upper = ceil(x),
// upper = lower + 1 on integers (gridding_gpu.cu:48-66)
template <class T>
__device__ __forceinline__ void cell_of(T x, int& lower, int& upper)
{
    lower = static_cast<int>(floor(x));
    upper = static_cast<int>(ceil(x));
    if (lower == upper) upper += 1;
}

// 1 - |x - x0| (gridding_gpu.cu:21-25)
template <class T>
__device__ __forceinline__ T vertex_weight(T x, int x0)
{
    return static_cast<T>(1) - fabs(x - static_cast<T>(x0));
}

template <class T>
__global__ void __launch_bounds__(kGrThreads)
    gridding_kernel(long long total, int n_pts, long long n_grid_vertices, float min_x, float min_y, float min_z, int len_x,
                    int len_y, int len_z, const T* __restrict__ ptcloud, T* __restrict__ grid,
                    T* __restrict__ grid_pt_weights, int* __restrict__ grid_pt_indexes)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGrThreads + threadIdx.x;
    if (t >= total) return;
    const long long cloud = t / n_pts;
    const T px = ptcloud[3 * t + 0], py = ptcloud[3 * t + 1], pz = ptcloud[3 * t + 2];
    int lo[3], up[3];
    cell_of(px, lo[0], up[0]);
    cell_of(py, lo[1], up[1]);
    cell_of(pz, lo[2], up[2]);
    // int - float -> float -> int, as the reference converts (gridding_gpu.cu:68-70)
    const int off[2][3] = {{static_cast<int>(lo[0] - min_x), static_cast<int>(lo[1] - min_y), static_cast<int>(lo[2] - min_z)},
                           {static_cast<int>(up[0] - min_x), static_cast<int>(up[1] - min_y), static_cast<int>(up[2] - min_z)}};
    const T w[2][3] = {{vertex_weight(px, lo[0]), vertex_weight(py, lo[1]), vertex_weight(pz, lo[2])},
                       {vertex_weight(px, up[0]), vertex_weight(py, up[1]), vertex_weight(pz, up[2])}};
    T* g = grid + cloud * n_grid_vertices;
    bool bad = false;
#pragma unroll
    for (int v = 0; v < 8; ++v)
    {
        // vertex v: bit 2 = upper x, bit 1 = upper y, bit 0 = upper z (LLL, LLU, LUL, ... UUU)
        const int ux = (v >> 2) & 1, uy = (v >> 1) & 1, uz = v & 1;
        const int ox = off[ux][0], oy = off[uy][1], oz = off[uz][2];
        const bool inside = ox >= 0 && ox < len_x && oy >= 0 && oy < len_y && oz >= 0 && oz < len_z;
        const int index = inside ? (ox * len_y + oy) * len_z + oz : -1;
        bad |= !inside;
        grid_pt_indexes[8 * t + v] = index;
        grid_pt_weights[24 * t + 3 * v + 0] = w[ux][0];
        grid_pt_weights[24 * t + 3 * v + 1] = w[uy][1];
        grid_pt_weights[24 * t + 3 * v + 2] = w[uz][2];
        if (inside) atomicAdd(g + index, mul_rn(mul_rn(w[ux][0], w[uy][1]), w[uz][2]));
    }
    if (bad) atomicOr(&g_dev_status, kStatusBadIndex);
}

template <class T>
__global__ void __launch_bounds__(kGrThreads)
    gridding_grad_kernel(long long total, int n_pts, long long n_grid_vertices, const T* __restrict__ grid_pt_weights,
                         const int* __restrict__ grid_pt_indexes, const T* __restrict__ grad_grid,
                         T* __restrict__ grad_ptcloud)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGrThreads + threadIdx.x;
    if (t >= total) return;
    const T* gg = grad_grid + (t / n_pts) * n_grid_vertices;
    T gx = 0, gy = 0, gz = 0;
#pragma unroll
    for (int v = 0; v < 8; ++v)
    {
        const int index = grid_pt_indexes[8 * t + v];
        if (index < 0 || index >= n_grid_vertices) continue;
        const T g = gg[index];
        const T wx = grid_pt_weights[24 * t + 3 * v + 0], wy = grid_pt_weights[24 * t + 3 * v + 1],
                wz = grid_pt_weights[24 * t + 3 * v + 2];
        // (+-g * a) * b, minus for the lower vertex of the axis (gridding_gpu.cu:223-301)
        const T sx = ((v >> 2) & 1) ? g : -g, sy = ((v >> 1) & 1) ? g : -g, sz = (v & 1) ? g : -g;
        gx = add_rn(gx, mul_rn(mul_rn(sx, wy), wz));
        gy = add_rn(gy, mul_rn(mul_rn(sy, wx), wz));
        gz = add_rn(gz, mul_rn(mul_rn(sz, wx), wy));
    }
    grad_ptcloud[3 * t + 0] = gx;
    grad_ptcloud[3 * t + 1] = gy;
    grad_ptcloud[3 * t + 2] = gz;
}

// Indices of the (2 * neighborhood_size)^3 vertices around every point, -1 outside the grid
// (cubic_feature_sampling_gpu.cu:44-91).
template <class T>
__global__ void __launch_bounds__(kGrThreads)
    cubic_index_kernel(long long total, int scale, int ns, int n_vertices, const T* __restrict__ ptcloud,
                       int* __restrict__ grid_pt_indexes)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGrThreads + threadIdx.x;
    if (t >= total) return;
    int lo[3], up[3];
    cell_of(ptcloud[3 * t + 0], lo[0], up[0]);
    cell_of(ptcloud[3 * t + 1], lo[1], up[1]);
    cell_of(ptcloud[3 * t + 2], lo[2], up[2]);
    int* out = grid_pt_indexes + t * n_vertices;
    // upper = lower + 1 always, so every axis runs over 2 * neighborhood_size cells; written as
    // fixed-length loops in 64-bit arithmetic so that every slot is written whatever the coordinates
    const int side = 2 * (ns + 1);
    (void)up;
    int vertex = 0;
    for (int a = 0; a < side; ++a)
        for (int b2 = 0; b2 < side; ++b2)
            for (int c = 0; c < side; ++c)
            {
                const long long j = static_cast<long long>(lo[0]) - ns + a, k = static_cast<long long>(lo[1]) - ns + b2,
                                m = static_cast<long long>(lo[2]) - ns + c;
                const bool outside = j < 0 || j >= scale || k < 0 || k >= scale || m < 0 || m >= scale;
                out[vertex++] = outside ? -1 : static_cast<int>((j * scale + k) * scale + m);
            }
}

// point_features[b, i, j, k] = cubic_features[b, k, vertex(i, j)] (0 for a vertex outside the grid);
// one thread per output element, channel fastest: coalesced stores.
template <class T>
__global__ void __launch_bounds__(kGrThreads)
    cubic_gather_kernel(long long total, int n_pts, int n_vertices, int channels, long long cub_scale,
                        const T* __restrict__ cubic_features, const int* __restrict__ grid_pt_indexes,
                        T* __restrict__ point_features)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGrThreads + threadIdx.x;
    if (t >= total) return;
    const int k = static_cast<int>(t % channels);
    const long long pv = t / channels;  // (cloud, point, vertex)
    const long long cloud = pv / (static_cast<long long>(n_pts) * n_vertices);
    const int vertex = grid_pt_indexes[pv];
    point_features[t] = (vertex < 0 || vertex >= cub_scale) ? static_cast<T>(0)
                                                              : cubic_features[(cloud * channels + k) * cub_scale + vertex];
}

template <class T>
__global__ void __launch_bounds__(kGrThreads)
    cubic_scatter_kernel(long long total, int n_pts, int n_vertices, int channels, long long cub_scale,
                         const T* __restrict__ grad_point_features, const int* __restrict__ grid_pt_indexes,
                         T* __restrict__ grad_cubic_features)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGrThreads + threadIdx.x;
    if (t >= total) return;
    const int k = static_cast<int>(t % channels);
    const long long pv = t / channels;
    const long long cloud = pv / (static_cast<long long>(n_pts) * n_vertices);
    const int vertex = grid_pt_indexes[pv];
    if (vertex < 0 || vertex >= cub_scale) return;
    atomicAdd(grad_cubic_features + (cloud * channels + k) * cub_scale + vertex, grad_point_features[t]);
}

int grid_blocks(long long total, unsigned* out, const char* what)
{
    const long long g = (total + kGrThreads - 1) / kGrThreads;
    if (g >= (1ll << 31))
    {
        set_error("%s: problem too large for one launch", what);
        return TPK_ERR_UNSUPPORTED;
    }
    *out = static_cast<unsigned>(g);
    return TPK_OK;
}

template <class T>
int gridding_impl(int b, int n_pts, float min_x, float max_x, float min_y, float max_y, float min_z, float max_z,
                  const T* ptcloud, T* grid, T* grid_pt_weights, int32_t* grid_pt_indexes, cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && n_pts >= 0, "gridding: negative size");
    const int len_x = static_cast<int>(max_x - min_x + 1), len_y = static_cast<int>(max_y - min_y + 1),
              len_z = static_cast<int>(max_z - min_z + 1);
    TPK_REQUIRE(len_x > 0 && len_y > 0 && len_z > 0, "gridding: empty grid");
    const long long nv = static_cast<long long>(len_x) * len_y * len_z;
    TPK_REQUIRE(nv < (1ll << 31), "gridding: grid too large");
    if (b == 0) return TPK_OK;
    TPK_REQUIRE(grid != nullptr, "gridding: NULL pointer");
    cudaError_t err = cudaMemsetAsync(grid, 0, sizeof(T) * static_cast<size_t>(b) * nv, s);
    if (err != cudaSuccess)
    {
        set_error("gridding: memset: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    if (n_pts == 0) return TPK_OK;
    TPK_REQUIRE(ptcloud && grid_pt_weights && grid_pt_indexes, "gridding: NULL pointer");
    const long long total = static_cast<long long>(b) * n_pts;
    unsigned g;
    const int rc = grid_blocks(total, &g, "gridding");
    if (rc != TPK_OK) return rc;
    count_launches(1), gridding_kernel<T><<<g, kGrThreads, 0, s>>>(total, n_pts, nv, min_x, min_y, min_z, len_x, len_y, len_z,
                                                                ptcloud, grid, grid_pt_weights, grid_pt_indexes);
    return check_launch("gridding");
}

template <class T>
int gridding_grad_impl(int b, int n_pts, int64_t n_grid_vertices, const T* grid_pt_weights, const int32_t* grid_pt_indexes,
                       const T* grad_grid, T* grad_ptcloud, cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && n_pts >= 0 && n_grid_vertices >= 0, "gridding_grad: negative size");
    if (b == 0 || n_pts == 0) return TPK_OK;
    TPK_REQUIRE(grid_pt_weights && grid_pt_indexes && grad_grid && grad_ptcloud, "gridding_grad: NULL pointer");
    const long long total = static_cast<long long>(b) * n_pts;
    unsigned g;
    const int rc = grid_blocks(total, &g, "gridding_grad");
    if (rc != TPK_OK) return rc;
    count_launches(1), gridding_grad_kernel<T><<<g, kGrThreads, 0, s>>>(total, n_pts, n_grid_vertices, grid_pt_weights,
                                                                     grid_pt_indexes, grad_grid, grad_ptcloud);
    return check_launch("gridding_grad");
}

template <class T>
int cubic_impl(int b, int n_pts, int channels, int scale, int neighborhood_size, const T* ptcloud, const T* cubic_features,
               T* point_features, int32_t* grid_pt_indexes, cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && n_pts >= 0 && channels >= 0 && scale > 0 && neighborhood_size >= 1 && neighborhood_size <= 8,
                "cubic_feature_sampling: size out of range");
    if (b == 0 || n_pts == 0) return TPK_OK;
    TPK_REQUIRE(ptcloud && grid_pt_indexes && (channels == 0 || (cubic_features && point_features)),
                "cubic_feature_sampling: NULL pointer");
    const int nvert = 8 * neighborhood_size * neighborhood_size * neighborhood_size;
    const long long pts = static_cast<long long>(b) * n_pts;
    unsigned g;
    int rc = grid_blocks(pts, &g, "cubic_feature_sampling");
    if (rc != TPK_OK) return rc;
    count_launches(1), cubic_index_kernel<T><<<g, kGrThreads, 0, s>>>(pts, scale, neighborhood_size - 1, nvert, ptcloud, grid_pt_indexes);
    if (channels > 0)
    {
        const long long total = pts * nvert * channels;
        rc = grid_blocks(total, &g, "cubic_feature_sampling");
        if (rc != TPK_OK) return rc;
        count_launches(1), cubic_gather_kernel<T><<<g, kGrThreads, 0, s>>>(total, n_pts, nvert, channels,
                                                                        static_cast<long long>(scale) * scale * scale,
                                                                        cubic_features, grid_pt_indexes, point_features);
    }
    return check_launch("cubic_feature_sampling");
}

template <class T>
int cubic_grad_impl(int b, int n_pts, int channels, int scale, int neighborhood_size, const T* grad_point_features,
                    const int32_t* grid_pt_indexes, T* grad_ptcloud, T* grad_cubic_features, cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && n_pts >= 0 && channels >= 0 && scale > 0 && neighborhood_size >= 1 && neighborhood_size <= 8,
                "cubic_feature_sampling_grad: size out of range");
    if (b == 0) return TPK_OK;
    const long long cub = static_cast<long long>(scale) * scale * scale;
    cudaError_t err = cudaSuccess;
    // the coordinates get no gradient: floor and ceil are flat (cubic_feature_sampling_gpu.cu:139-144)
    if (grad_ptcloud && n_pts > 0) err = cudaMemsetAsync(grad_ptcloud, 0, sizeof(T) * static_cast<size_t>(b) * n_pts * 3, s);
    if (err == cudaSuccess && grad_cubic_features && channels > 0)
        err = cudaMemsetAsync(grad_cubic_features, 0, sizeof(T) * static_cast<size_t>(b) * channels * cub, s);
    if (err != cudaSuccess)
    {
        set_error("cubic_feature_sampling_grad: memset: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    if (n_pts == 0 || channels == 0) return TPK_OK;
    TPK_REQUIRE(grad_point_features && grid_pt_indexes && grad_cubic_features, "cubic_feature_sampling_grad: NULL pointer");
    const int nvert = 8 * neighborhood_size * neighborhood_size * neighborhood_size;
    const long long total = static_cast<long long>(b) * n_pts * nvert * channels;
    unsigned g;
    const int rc = grid_blocks(total, &g, "cubic_feature_sampling_grad");
    if (rc != TPK_OK) return rc;
    count_launches(1), cubic_scatter_kernel<T><<<g, kGrThreads, 0, s>>>(total, n_pts, nvert, channels, cub, grad_point_features,
                                                                     grid_pt_indexes, grad_cubic_features);
    return check_launch("cubic_feature_sampling_grad");
}

}  // namespace
}  // namespace tpk

#define TPK_GRNET_ENTRY(SUFFIX, T)                                                                                      \
    extern "C" int tpk_gridding_##SUFFIX(int b, int n_pts, float min_x, float max_x, float min_y, float max_y, float min_z, \
                                         float max_z, const T* ptcloud, T* grid, T* grid_pt_weights,                  \
                                         int32_t* grid_pt_indexes, void* stream)                                       \
    {                                                                                                                   \
        return tpk::gridding_impl<T>(b, n_pts, min_x, max_x, min_y, max_y, min_z, max_z, ptcloud, grid, grid_pt_weights, \
                                     grid_pt_indexes, static_cast<cudaStream_t>(stream));                              \
    }                                                                                                                   \
    extern "C" int tpk_gridding_grad_##SUFFIX(int b, int n_pts, int64_t n_grid_vertices, const T* grid_pt_weights,      \
                                              const int32_t* grid_pt_indexes, const T* grad_grid, T* grad_ptcloud,     \
                                              void* stream)                                                             \
    {                                                                                                                   \
        return tpk::gridding_grad_impl<T>(b, n_pts, n_grid_vertices, grid_pt_weights, grid_pt_indexes, grad_grid,      \
                                          grad_ptcloud, static_cast<cudaStream_t>(stream));                            \
    }                                                                                                                   \
    extern "C" int tpk_cubic_feature_sampling_##SUFFIX(int b, int n_pts, int channels, int scale, int neighborhood_size, \
                                                       const T* ptcloud, const T* cubic_features, T* point_features,   \
                                                       int32_t* grid_pt_indexes, void* stream)                         \
    {                                                                                                                   \
        return tpk::cubic_impl<T>(b, n_pts, channels, scale, neighborhood_size, ptcloud, cubic_features, point_features, \
                                  grid_pt_indexes, static_cast<cudaStream_t>(stream));                                 \
    }                                                                                                                   \
    extern "C" int tpk_cubic_feature_sampling_grad_##SUFFIX(int b, int n_pts, int channels, int scale,                  \
                                                            int neighborhood_size, const T* grad_point_features,       \
                                                            const int32_t* grid_pt_indexes, T* grad_ptcloud,           \
                                                            T* grad_cubic_features, void* stream)                      \
    {                                                                                                                   \
        return tpk::cubic_grad_impl<T>(b, n_pts, channels, scale, neighborhood_size, grad_point_features,              \
                                       grid_pt_indexes, grad_ptcloud, grad_cubic_features,                             \
                                       static_cast<cudaStream_t>(stream));                                             \
    }

TPK_GRNET_ENTRY(f32, float)
TPK_GRNET_ENTRY(f64, double)
#undef TPK_GRNET_ENTRY
