// Nearest-neighbour searches for sm_100a: three_nn (fixed k = 3, int32 indices, the
// feature-propagation search) and kNN (1 <= k <= 64, int64 indices, dense and packed).
//
// Both are brute force over shared-memory candidate tiles (scan.cuh).  A thread keeps
// the running k-th best distance of each of its queries in a register and touches its
// sorted result list only when a candidate beats it, which on real clouds happens
// O(k log(n/k)) times per query out of n candidates.
//
// three_nn : cuda/src/interpolate_gpu.cu:9-65 (strict '<' cascade: ascending distance,
//            lowest index first among equals; missing neighbours are +inf / index 0)
// kNN      : cpu/src/knn.cpp:40-59 -> nanoflann knnSearch; unfused distance arithmetic,
//            ascending distance, index order among equals
#include <math_constants.h>

#include "scan.cuh"

namespace tpk
{
namespace
{

template <int Q>
struct ThreeNnOp
{
    float qx[Q], qy[Q], qz[Q];
    float b1[Q], b2[Q], b3[Q];
    int i1[Q], i2[Q], i3[Q];
    bool act[Q];

    __device__ __forceinline__ float threshold(int q) const { return act[q] ? b3[q] : -CUDART_INF_F; }
    __device__ __forceinline__ bool finished() const
    {
        bool done = true;
#pragma unroll
        for (int q = 0; q < Q; ++q) done &= !act[q];
        return done;
    }
    __device__ __forceinline__ bool exact(int q, long long k, float cx, float cy, float cz)
    {
        const float v = sumsq_abc(qx[q] - cx, qy[q] - cy, qz[q] - cz);
        if (!act[q] || !(v < b3[q])) return false;
        const int kk = static_cast<int>(k);
        if (v < b1[q])
        {
            b3[q] = b2[q]; i3[q] = i2[q];
            b2[q] = b1[q]; i2[q] = i1[q];
            b1[q] = v;     i1[q] = kk;
        }
        else if (v < b2[q])
        {
            b3[q] = b2[q]; i3[q] = i2[q];
            b2[q] = v;     i2[q] = kk;
        }
        else
        {
            b3[q] = v; i3[q] = kk;
        }
        return true;
    }
};

template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    three_nn_kernel(int n, int m, int tiles_per_cloud, const float* __restrict__ unknown,
                    const float* __restrict__ known, float* __restrict__ dist2,
                    int32_t* __restrict__ idx, const unsigned char* __restrict__ need)
{
    __shared__ __align__(16) float smem[2 * kScanTileFloats];
    const int cloud = blockIdx.x / tiles_per_cloud;
    const int qtile = blockIdx.x - cloud * tiles_per_cloud;

    ThreeNnOp<Q> op;
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        // `need` (optional): one byte per query, 0 = already answered by the grid path
        op.act[q] = j < n && (need == nullptr || need[static_cast<size_t>(cloud) * n + j] != 0);
        const size_t row = static_cast<size_t>(cloud) * n + (op.act[q] ? j : 0);
        op.qx[q] = op.act[q] ? __ldg(unknown + row * 3 + 0) : 0.f;
        op.qy[q] = op.act[q] ? __ldg(unknown + row * 3 + 1) : 0.f;
        op.qz[q] = op.act[q] ? __ldg(unknown + row * 3 + 2) : 0.f;
        op.b1[q] = op.b2[q] = op.b3[q] = CUDART_INF_F;
        op.i1[q] = op.i2[q] = op.i3[q] = 0;
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
    scan_candidates<THREADS, Q>(known + static_cast<size_t>(cloud) * m * 3, m, smem, op.qx, op.qy, op.qz, op);
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        if (!op.act[q]) continue;
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        const size_t o = (static_cast<size_t>(cloud) * n + j) * 3;
        dist2[o + 0] = op.b1[q];
        dist2[o + 1] = op.b2[q];
        dist2[o + 2] = op.b3[q];
        idx[o + 0] = op.i1[q];
        idx[o + 1] = op.i2[q];
        idx[o + 2] = op.i3[q];
    }
}

// Sorted lists live in shared memory, slot s of list l at [s * LISTS + l]: consecutive
// threads hit consecutive banks.
template <int Q, int LISTS>
struct KnnOp
{
    float qx[Q], qy[Q], qz[Q];
    float thr[Q];  // current k-th best (the admission threshold), +inf until the list is full
    int cnt[Q];
    bool act[Q];
    float* ldist;  // list of q = 0 of this thread; the q-th list is at + q * (LISTS / Q)
    int* lidx;
    int k;

    __device__ __forceinline__ float threshold(int q) const { return act[q] ? thr[q] : -CUDART_INF_F; }
    __device__ __forceinline__ bool finished() const
    {
        bool done = true;
#pragma unroll
        for (int q = 0; q < Q; ++q) done &= !act[q];
        return done;
    }
    __device__ __forceinline__ bool exact(int q, long long cand, float cx, float cy, float cz)
    {
        const float v = sumsq_unfused(qx[q] - cx, qy[q] - cy, qz[q] - cz);
        if (!act[q] || !(v < thr[q])) return false;
        float* dl = ldist + q * (LISTS / Q);
        int* il = lidx + q * (LISTS / Q);
        int i = cnt[q] < k ? cnt[q] : k - 1;
        for (; i > 0 && dl[(i - 1) * LISTS] > v; --i)
        {
            dl[i * LISTS] = dl[(i - 1) * LISTS];
            il[i * LISTS] = il[(i - 1) * LISTS];
        }
        dl[i * LISTS] = v;
        il[i * LISTS] = static_cast<int>(cand);
        if (cnt[q] < k) ++cnt[q];
        if (cnt[q] == k) thr[q] = dl[(k - 1) * LISTS];
        return true;
    }
};

template <int THREADS, int Q>
__device__ __forceinline__ void knn_write(const KnnOp<Q, THREADS * Q>& op, int q, int k,
                                          long long idx_base, int64_t* orow, float* drow)
{
    const float* dl = op.ldist + q * THREADS;
    const int* il = op.lidx + q * THREADS;
    for (int s = 0; s < k; ++s)
    {
        const bool have = s < op.cnt[q];
        orow[s] = have ? il[s * THREADS * Q] + idx_base : -1;
        drow[s] = have ? dl[s * THREADS * Q] : -1.0f;
    }
}

template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    knn_dense_kernel(int n, int m, int k, int tiles_per_cloud, const float* __restrict__ support,
                     const float* __restrict__ query, int64_t* __restrict__ idx,
                     float* __restrict__ dist2, const unsigned char* __restrict__ need)
{
    extern __shared__ __align__(16) float dyn_smem[];
    float* tile = dyn_smem;
    float* ldist = dyn_smem + 2 * kScanTileFloats;
    int* lidx = reinterpret_cast<int*>(ldist + static_cast<size_t>(k) * THREADS * Q);
    const int cloud = blockIdx.x / tiles_per_cloud;
    const int qtile = blockIdx.x - cloud * tiles_per_cloud;

    KnnOp<Q, THREADS * Q> op;
    op.k = k;
    op.ldist = ldist + threadIdx.x;
    op.lidx = lidx + threadIdx.x;
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        // `need` (optional): one byte per query, 0 = already answered by the grid path
        op.act[q] = j < m && (need == nullptr || need[static_cast<size_t>(cloud) * m + j] != 0);
        const size_t row = static_cast<size_t>(cloud) * m + (op.act[q] ? j : 0);
        op.qx[q] = op.act[q] ? __ldg(query + row * 3 + 0) : 0.f;
        op.qy[q] = op.act[q] ? __ldg(query + row * 3 + 1) : 0.f;
        op.qz[q] = op.act[q] ? __ldg(query + row * 3 + 2) : 0.f;
        op.thr[q] = CUDART_INF_F;
        op.cnt[q] = 0;
    }
    if (need != nullptr)
    {
        // nothing left over for this CTA (the usual case behind the grid kernel)
        bool any = false;
#pragma unroll
        for (int q = 0; q < Q; ++q) any |= op.act[q];
        if (!__syncthreads_or(any ? 1 : 0)) return;
    }
    scan_candidates<THREADS, Q>(support + static_cast<size_t>(cloud) * n * 3, n, tile, op.qx, op.qy, op.qz, op);
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        if (!op.act[q]) continue;
        const int j = qtile * (THREADS * Q) + q * THREADS + threadIdx.x;
        const size_t row = static_cast<size_t>(cloud) * m + j;
        knn_write<THREADS, Q>(op, q, k, 0, idx + row * k, dist2 + row * k);
    }
}

template <int THREADS, int Q>
__global__ void __launch_bounds__(THREADS)
    knn_partial_kernel(long long size_s, long long size_q, int k,
                       const float* __restrict__ support, const float* __restrict__ query,
                       const int64_t* __restrict__ batch_s, const int64_t* __restrict__ batch_q,
                       int64_t* __restrict__ idx, float* __restrict__ dist2, const unsigned char* __restrict__ need)
{
    extern __shared__ __align__(16) float dyn_smem[];
    __shared__ long long s_range[2];
    __shared__ unsigned long long s_next;
    float* tile = dyn_smem;
    float* ldist = dyn_smem + 2 * kScanTileFloats;
    int* lidx = reinterpret_cast<int*>(ldist + static_cast<size_t>(k) * THREADS * Q);

    KnnOp<Q, THREADS * Q> op;
    op.k = k;
    op.ldist = ldist + threadIdx.x;
    op.lidx = lidx + threadIdx.x;
    int64_t seg[Q];
    bool valid[Q];
    long long base[Q];
    const long long j0 = static_cast<long long>(blockIdx.x) * (THREADS * Q);
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        const long long j = j0 + q * THREADS + threadIdx.x;
        // `need` (optional): one byte per query, 0 = already answered by the grid path
        valid[q] = j < size_q && (need == nullptr || need[j] != 0);
        const long long row = valid[q] ? j : 0;
        seg[q] = valid[q] ? __ldg(batch_q + row) : 0;
        op.qx[q] = valid[q] ? __ldg(query + row * 3 + 0) : 0.f;
        op.qy[q] = valid[q] ? __ldg(query + row * 3 + 1) : 0.f;
        op.qz[q] = valid[q] ? __ldg(query + row * 3 + 2) : 0.f;
        op.thr[q] = CUDART_INF_F;
        op.cnt[q] = 0;
        base[q] = 0;
    }
    const unsigned long long kNone = ~0ull;
    // the first segment any query of this CTA still needs (segment ids are non-negative)
    if (threadIdx.x == 0) s_next = kNone;
    __syncthreads();
#pragma unroll
    for (int q = 0; q < Q; ++q)
        if (valid[q]) atomicMin(&s_next, static_cast<unsigned long long>(seg[q]));
    __syncthreads();
    if (s_next == kNone) return;  // nothing left over for this CTA
    int64_t cur = static_cast<int64_t>(s_next);
    __syncthreads();
    while (true)
    {
        if (threadIdx.x == 0)
        {
            s_range[0] = segment_bound(batch_s, size_s, cur, false);
            s_range[1] = segment_bound(batch_s, size_s, cur, true);
            s_next = kNone;
        }
        __syncthreads();
        const long long lo = s_range[0], hi = s_range[1];
#pragma unroll
        for (int q = 0; q < Q; ++q)
        {
            op.act[q] = valid[q] && seg[q] == cur;
            if (op.act[q]) base[q] = lo;
            if (valid[q] && seg[q] > cur)
                atomicMin(&s_next, static_cast<unsigned long long>(seg[q]));
        }
        scan_candidates<THREADS, Q>(support + lo * 3, hi - lo, tile, op.qx, op.qy, op.qz, op);
        const unsigned long long nxt = s_next;
        __syncthreads();
        if (nxt == kNone) break;
        cur = static_cast<int64_t>(nxt);
    }
#pragma unroll
    for (int q = 0; q < Q; ++q)
    {
        if (!valid[q]) continue;
        const long long row = j0 + q * THREADS + threadIdx.x;
        knn_write<THREADS, Q>(op, q, k, base[q], idx + row * k, dist2 + row * k);
    }
}

void pick_shape_nn(long long queries, int* threads, int* q)
{
    *q = queries >= 300000 ? 2 : 1;
    *threads = queries >= 32768 ? 128 : 64;
}

size_t knn_smem_bytes(int threads, int q, int k)
{
    return sizeof(float) * 2 * kScanTileFloats + static_cast<size_t>(k) * threads * q * 8;
}

template <class K>
int set_smem(K kernel, size_t bytes, const char* what)
{
    if (bytes > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(bytes));
        if (err != cudaSuccess)
        {
            set_error("%s: shared memory attribute: %s", what, cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    return TPK_OK;
}

}  // namespace
}  // namespace tpk

namespace tpk
{
// grid_query.cu
size_t grid_three_nn_scratch_bytes(int b, int n, int m);
int grid_three_nn(int b, int n, int m, const float* unknown, const float* known, float* dist2,
                  int32_t* idx, void* scratch, const unsigned char** need_scan_out, cudaStream_t s);

// smem_grid.cu
bool sg_three_nn_fits(int m);
int sg_three_nn(int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
                unsigned char* need, cudaStream_t s);
bool sg_nn_slab_fits(int b, int n, int m);
int sg_nn_slab(int k, int b, int n, int m, const float* unknown, const float* known, float* dist2, int32_t* idx,
               unsigned char* need, cudaStream_t s);

static int launch_three_nn_scan(int b, int n, int m, const float* unknown, const float* known,
                                float* dist2, int32_t* idx, const unsigned char* need, cudaStream_t s)
{
    int threads, q;
    pick_shape_nn(static_cast<long long>(b) * n, &threads, &q);
    const int tiles = (n + threads * q - 1) / (threads * q);
    const long long grid = static_cast<long long>(b) * tiles;
    TPK_REQUIRE(grid < (1ll << 31), "three_nn: too many queries");
    const dim3 g(static_cast<unsigned>(grid));
    if (threads == 128 && q == 2)
    {
        prefer_max_shared(three_nn_kernel<128, 2>);
        count_launches(1), three_nn_kernel<128, 2><<<g, 128, 0, s>>>(n, m, tiles, unknown, known, dist2, idx, need);
    }
    else if (threads == 128)
    {
        prefer_max_shared(three_nn_kernel<128, 1>);
        count_launches(1), three_nn_kernel<128, 1><<<g, 128, 0, s>>>(n, m, tiles, unknown, known, dist2, idx, need);
    }
    else if (q == 2)
    {
        prefer_max_shared(three_nn_kernel<64, 2>);
        count_launches(1), three_nn_kernel<64, 2><<<g, 64, 0, s>>>(n, m, tiles, unknown, known, dist2, idx, need);
    }
    else
    {
        prefer_max_shared(three_nn_kernel<64, 1>);
        count_launches(1), three_nn_kernel<64, 1><<<g, 64, 0, s>>>(n, m, tiles, unknown, known, dist2, idx, need);
    }
    return check_launch("three_nn");
}
}  // namespace tpk

extern "C" int tpk_three_nn(int b, int n, int m, const float* unknown, const float* known,
                            float* dist2, int32_t* idx, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "three_nn: negative size (b=%d n=%d m=%d)", b, n, m);
    if (b == 0 || n == 0) return TPK_OK;
    TPK_REQUIRE(unknown && dist2 && idx && (known || m == 0), "three_nn: NULL pointer");
    return launch_three_nn_scan(b, n, m, unknown, known, dist2, idx, nullptr, static_cast<cudaStream_t>(stream));
}

// the test hook "three_nn_global_grid" selects the grid in global memory where the
// shared-memory grid would be used
static bool three_nn_smem_grid(int m)
{
    return tpk::sg_three_nn_fits(m) && !tpk::test_path("three_nn_global_grid");
}

// above 8192 known points: the shared-memory grid by layers
static bool three_nn_by_layers(int b, int n, int m)
{
    return tpk::sg_nn_slab_fits(b, n, m) && !tpk::test_path("three_nn_global_grid");
}

extern "C" int64_t tpk_three_nn_scratch_bytes(int b, int n, int m)
{
    if (b <= 0 || n <= 0) return 0;
    if (tpk::test_path("three_nn_scan")) return 0;  // test hook: the scan alone
    // shared-memory grid: one flag per unknown point
    if (three_nn_smem_grid(m) || three_nn_by_layers(b, n, m)) return (static_cast<int64_t>(b) * n + 255) / 256 * 256;
    if (m < 4096) return 0;
    return static_cast<int64_t>(tpk::grid_three_nn_scratch_bytes(b, n, m));
}

extern "C" int tpk_three_nn_ws(int b, int n, int m, const float* unknown, const float* known,
                               float* dist2, int32_t* idx, void* scratch, int64_t scratch_bytes,
                               void* stream)
{
    using namespace tpk;
    const int64_t want = tpk_three_nn_scratch_bytes(b, n, m);
    if (want == 0 || scratch == nullptr) return tpk_three_nn(b, n, m, unknown, known, dist2, idx, stream);
    if (scratch_bytes < want)
    {
        set_error("three_nn: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch_bytes),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE(unknown && known && dist2 && idx, "three_nn: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "three_nn: scratch must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned char* need = nullptr;
    int rc;
    if (three_nn_smem_grid(m))
    {
        need = static_cast<const unsigned char*>(scratch);
        rc = sg_three_nn(b, n, m, unknown, known, dist2, idx, static_cast<unsigned char*>(scratch), s);
    }
    else if (three_nn_by_layers(b, n, m))
    {
        need = static_cast<const unsigned char*>(scratch);
        rc = sg_nn_slab(3, b, n, m, unknown, known, dist2, idx, static_cast<unsigned char*>(scratch), s);
    }
    else
    {
        rc = grid_three_nn(b, n, m, unknown, known, dist2, idx, scratch, &need, s);
    }
    if (rc != TPK_OK) return rc;
    return launch_three_nn_scan(b, n, m, unknown, known, dist2, idx, need, s);
}

#define TPK_KNN_DISPATCH(KERNEL, ...)                                                              \
    do                                                                                             \
    {                                                                                              \
        int rc_;                                                                                   \
        if (threads == 128 && q == 2)                                                              \
        {                                                                                          \
            if ((rc_ = set_smem(KERNEL<128, 2>, smem, "knn")) != TPK_OK) return rc_;               \
            count_launches(1), KERNEL<128, 2><<<g, 128, smem, s>>>(__VA_ARGS__);                                      \
        }                                                                                          \
        else if (threads == 128)                                                                   \
        {                                                                                          \
            if ((rc_ = set_smem(KERNEL<128, 1>, smem, "knn")) != TPK_OK) return rc_;               \
            count_launches(1), KERNEL<128, 1><<<g, 128, smem, s>>>(__VA_ARGS__);                                      \
        }                                                                                          \
        else if (q == 2)                                                                           \
        {                                                                                          \
            if ((rc_ = set_smem(KERNEL<64, 2>, smem, "knn")) != TPK_OK) return rc_;                \
            count_launches(1), KERNEL<64, 2><<<g, 64, smem, s>>>(__VA_ARGS__);                                        \
        }                                                                                          \
        else                                                                                       \
        {                                                                                          \
            if ((rc_ = set_smem(KERNEL<64, 1>, smem, "knn")) != TPK_OK) return rc_;                \
            count_launches(1), KERNEL<64, 1><<<g, 64, smem, s>>>(__VA_ARGS__);                                        \
        }                                                                                          \
    } while (0)

namespace tpk
{
// hash_grid.cu
bool hash_grid_fits(long long size_x, long long size_y);
size_t hash_grid_knn_scratch_bytes(long long size_s, long long size_q);
int hash_grid_knn(long long size_s, long long size_q, long long per_cloud_s, long long per_cloud_q, int k,
                  const float* support, const float* query, const int64_t* batch_s, const int64_t* batch_q, int64_t* idx,
                  float* dist2, void* scratch, const unsigned char** need_out, cudaStream_t s);
}  // namespace tpk

// `need` (optional, device): one byte per query, 0 = already answered, skip it
static int knn_dense_scan(int b, int n, int m, int k, const float* support, const float* query, int64_t* idx,
                          float* dist2, const unsigned char* need, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "knn: negative size (b=%d n=%d m=%d)", b, n, m);
    TPK_REQUIRE(k >= 1 && k <= TPK_KNN_MAX_K, "knn: k=%d outside 1..%d", k, TPK_KNN_MAX_K);
    TPK_REQUIRE(k <= n, "Not enough points in support to find %d neighboors", k);
    if (b == 0 || m == 0) return TPK_OK;
    TPK_REQUIRE(support && query && idx && dist2, "knn: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int threads, q;
    pick_shape_nn(static_cast<long long>(b) * m, &threads, &q);
    if (k > 16) q = 1;
    if (k > 32 && threads > 64) threads = 64;
    const size_t smem = knn_smem_bytes(threads, q, k);
    const int tiles = (m + threads * q - 1) / (threads * q);
    const long long grid = static_cast<long long>(b) * tiles;
    TPK_REQUIRE(grid < (1ll << 31), "knn: too many queries");
    const dim3 g(static_cast<unsigned>(grid));
    TPK_KNN_DISPATCH(knn_dense_kernel, n, m, k, tiles, support, query, idx, dist2, need);
    return check_launch("knn_dense");
}

extern "C" int tpk_knn_dense(int b, int n, int m, int k, const float* support, const float* query,
                             int64_t* idx, float* dist2, void* stream)
{
    return knn_dense_scan(b, n, m, k, support, query, idx, dist2, nullptr, stream);
}

// The hashed grid pays from a few thousand support points per cloud on; the test hook
// "knn_scan" keeps every query on the scan.
static bool knn_dense_wants_grid(int b, int n, int m)
{
    return n >= 2048 && tpk::hash_grid_fits(static_cast<long long>(b) * n, static_cast<long long>(b) * m) &&
           !tpk::test_path("knn_scan");
}

extern "C" int64_t tpk_knn_dense_scratch_bytes(int b, int n, int m, int k)
{
    if (b <= 0 || n <= 0 || m <= 0 || k <= 0 || !knn_dense_wants_grid(b, n, m)) return 0;
    return static_cast<int64_t>(tpk::hash_grid_knn_scratch_bytes(static_cast<long long>(b) * n, static_cast<long long>(b) * m));
}

extern "C" int tpk_knn_dense_ws(int b, int n, int m, int k, const float* support, const float* query, int64_t* idx,
                                float* dist2, void* scratch, int64_t scratch_bytes, void* stream)
{
    using namespace tpk;
    const int64_t want = tpk_knn_dense_scratch_bytes(b, n, m, k);
    if (want == 0 || scratch == nullptr) return tpk_knn_dense(b, n, m, k, support, query, idx, dist2, stream);
    if (scratch_bytes < want)
    {
        set_error("knn: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch_bytes),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE(k >= 1 && k <= TPK_KNN_MAX_K, "knn: k=%d outside 1..%d", k, TPK_KNN_MAX_K);
    TPK_REQUIRE(k <= n, "Not enough points in support to find %d neighboors", k);
    TPK_REQUIRE(support && query && idx && dist2, "knn: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "knn: scratch must be 256-byte aligned");
    const unsigned char* need = nullptr;
    const int rc = hash_grid_knn(static_cast<long long>(b) * n, static_cast<long long>(b) * m, n, m, k, support, query,
                                 nullptr, nullptr, idx, dist2, scratch, &need, static_cast<cudaStream_t>(stream));
    if (rc != TPK_OK) return rc;
    return knn_dense_scan(b, n, m, k, support, query, idx, dist2, need, stream);
}

static int knn_partial_scan(int64_t size_s, int64_t size_q, int k, const float* support, const float* query,
                            const int64_t* batch_s, const int64_t* batch_q, int64_t* idx, float* dist2,
                            const unsigned char* need, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(size_s >= 0 && size_q >= 0, "knn_partial_dense: negative size");
    TPK_REQUIRE(k >= 1 && k <= TPK_KNN_MAX_K, "knn: k=%d outside 1..%d", k, TPK_KNN_MAX_K);
    if (size_q == 0) return TPK_OK;
    TPK_REQUIRE(query && batch_q && idx && dist2 && ((support && batch_s) || size_s == 0),
                "knn_partial_dense: NULL pointer");
    TPK_REQUIRE(size_s < (1ll << 31), "knn_partial_dense: support too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int threads, q;
    pick_shape_nn(size_q, &threads, &q);
    if (k > 16) q = 1;
    if (k > 32 && threads > 64) threads = 64;
    const size_t smem = knn_smem_bytes(threads, q, k);
    const long long grid = (size_q + threads * q - 1) / (threads * q);
    TPK_REQUIRE(grid < (1ll << 31), "knn_partial_dense: too many queries");
    const dim3 g(static_cast<unsigned>(grid));
    TPK_KNN_DISPATCH(knn_partial_kernel, size_s, size_q, k, support, query, batch_s, batch_q, idx, dist2, need);
    return check_launch("knn_partial_dense");
}

extern "C" int tpk_knn_partial_dense(int64_t size_s, int64_t size_q, int k, const float* support,
                                     const float* query, const int64_t* batch_s,
                                     const int64_t* batch_q, int64_t* idx, float* dist2,
                                     void* stream)
{
    return knn_partial_scan(size_s, size_q, k, support, query, batch_s, batch_q, idx, dist2, nullptr, stream);
}

static bool knn_partial_wants_grid(int64_t size_s, int64_t size_q)
{
    return tpk::hash_grid_fits(size_s, size_q) && !tpk::test_path("knn_scan");
}

extern "C" int64_t tpk_knn_partial_dense_scratch_bytes(int64_t size_s, int64_t size_q, int k)
{
    if (k <= 0 || !knn_partial_wants_grid(size_s, size_q)) return 0;
    return static_cast<int64_t>(tpk::hash_grid_knn_scratch_bytes(size_s, size_q));
}

extern "C" int tpk_knn_partial_dense_ws(int64_t size_s, int64_t size_q, int k, const float* support,
                                        const float* query, const int64_t* batch_s, const int64_t* batch_q,
                                        int64_t* idx, float* dist2, void* scratch, int64_t scratch_bytes,
                                        void* stream)
{
    using namespace tpk;
    const int64_t want = tpk_knn_partial_dense_scratch_bytes(size_s, size_q, k);
    if (want == 0 || scratch == nullptr)
        return tpk_knn_partial_dense(size_s, size_q, k, support, query, batch_s, batch_q, idx, dist2, stream);
    if (scratch_bytes < want)
    {
        set_error("knn_partial_dense: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch_bytes),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE(k >= 1 && k <= TPK_KNN_MAX_K, "knn: k=%d outside 1..%d", k, TPK_KNN_MAX_K);
    TPK_REQUIRE(query && batch_q && idx && dist2 && support && batch_s, "knn_partial_dense: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "knn_partial_dense: scratch must be 256-byte aligned");
    const unsigned char* need = nullptr;
    const int rc = hash_grid_knn(size_s, size_q, 1, 1, k, support, query, batch_s, batch_q, idx, dist2, scratch, &need,
                                 static_cast<cudaStream_t>(stream));
    if (rc != TPK_OK) return rc;
    return knn_partial_scan(size_s, size_q, k, support, query, batch_s, batch_q, idx, dist2, need, stream);
}
