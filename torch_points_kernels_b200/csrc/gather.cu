// Gather / scatter-add kernels for sm_100a: grouping_operation and three_interpolate,
// forward and backward.  All four are bandwidth problems: the forward passes write a
// large output from a small, cache-resident feature tensor, the backward passes read a
// large gradient and reduce it into a small one.
//
// Forward: a thread owns four consecutive output positions, loads their indices (and
// weights) once, then walks a chunk of channels; per channel it gathers from the
// (L1/L2-resident) feature row and issues one 16-byte streaming store, so a warp
// writes 512 contiguous bytes per channel.
//
// Backward: a CTA owns a few (batch, channel) rows of the small gradient tensor and
// keeps them in shared memory; it streams the matching rows of the incoming gradient
// with 16-byte loads, accumulates with shared-memory atomics (no global atomics, no
// zero-fill pass over the output) and writes each finished row once.  Rows too long
// for shared memory fall back to global red.add on a zeroed output.
//
// grouping          : torch_points_kernels/torchpoints.py:129-146 (torch.gather + autograd)
// three_interpolate : cuda/src/interpolate_gpu.cu:78-107, :122-152
#include "tpk_common.cuh"

namespace tpk
{
TPK_DEFINE_STATUS_WORD()

namespace
{

constexpr int kGatherThreads = 256;
constexpr int kScatterThreads = 512;
constexpr int kChanChunk = 16;
constexpr size_t kRowSmemBudget = 200 * 1024;

// p1*w1 + p2*w2 + p3*w3 as nvcc contracts the reference expression (interpolate_gpu.cu:105)
__device__ __forceinline__ float interp3(float p1, float w1, float p2, float w2, float p3, float w3)
{
    return __fmaf_rn(p3, w3, __fmaf_rn(p1, w1, __fmul_rn(p2, w2)));
}

// An index as the kernels use it: the value itself when it addresses an element of a row of
// `len` elements, -1 otherwise.  An index out of range never reaches a load, a store or an
// atomic: gathers return 0 for it, scatters drop the contribution, and the sticky status
// word of the device records it (the reference's torch.gather raises a device assert there).
// `bad` collects the finding in a register; the kernel reports it once, on its way out
// (report_bad), so that no atomic sits between the loads of the streaming loops.
__device__ __forceinline__ int checked_index(long long v, int len, bool& bad)
{
    const bool ok = static_cast<unsigned long long>(v) < static_cast<unsigned long long>(len);
    bad |= !ok;
    return ok ? static_cast<int>(v) : -1;
}
__device__ __forceinline__ void report_bad(bool bad)
{
    if (bad) atomicOr(&g_dev_status, kStatusBadIndex);
}
__device__ __forceinline__ float gather_or_zero(const float* row, int i) { return i >= 0 ? row[i] : 0.f; }
__device__ __forceinline__ float ldg_or_zero(const float* row, int i) { return i >= 0 ? __ldg(row + i) : 0.f; }

// ------------------------------------------------------------------ grouping forward

template <bool VEC>
__global__ void __launch_bounds__(kGatherThreads)
    grouping_fwd_kernel(int c, int n, long long ps, int out_c, int out_off, const float* __restrict__ features,
                        const int64_t* __restrict__ idx, float* __restrict__ out)
{
    const int bi = blockIdx.z;
    const int c0 = blockIdx.y * kChanChunk;
    const int c1 = min(c, c0 + kChanChunk);
    const long long pos = (static_cast<long long>(blockIdx.x) * kGatherThreads + threadIdx.x) * 4;
    if (pos >= ps) return;
    const int64_t* ip = idx + static_cast<size_t>(bi) * ps + pos;
    bool bad = false;
    int i0, i1 = 0, i2 = 0, i3 = 0;
    const bool full = VEC || pos + 3 < ps;
    if (VEC)
    {
        const longlong2 a = __ldg(reinterpret_cast<const longlong2*>(ip));
        const longlong2 b2 = __ldg(reinterpret_cast<const longlong2*>(ip) + 1);
        i0 = checked_index(a.x, n, bad);
        i1 = checked_index(a.y, n, bad);
        i2 = checked_index(b2.x, n, bad);
        i3 = checked_index(b2.y, n, bad);
    }
    else
    {
        i0 = checked_index(__ldg(ip), n, bad);
        if (pos + 1 < ps) i1 = checked_index(__ldg(ip + 1), n, bad);
        if (pos + 2 < ps) i2 = checked_index(__ldg(ip + 2), n, bad);
        if (pos + 3 < ps) i3 = checked_index(__ldg(ip + 3), n, bad);
    }
    const float* f = features + (static_cast<size_t>(bi) * c + c0) * n;
    // row (bi, ch) of the result is row out_off + ch of out_c rows per batch element (the fused
    // set-abstraction op writes its features behind three coordinate rows)
    float* o = out + (static_cast<size_t>(bi) * out_c + out_off + c0) * ps + pos;
#pragma unroll 4
    for (int ch = c0; ch < c1; ++ch, f += n, o += ps)
    {
        float4 v;
        v.x = ldg_or_zero(f, i0);
        v.y = ldg_or_zero(f, i1);
        v.z = ldg_or_zero(f, i2);
        v.w = ldg_or_zero(f, i3);
        if (VEC)
            __stcs(reinterpret_cast<float4*>(o), v);
        else if (full)
        {
            o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
        }
        else
        {
            o[0] = v.x;
            if (pos + 1 < ps) o[1] = v.y;
            if (pos + 2 < ps) o[2] = v.z;
        }
    }
    report_bad(bad);
}

// ------------------------------------------------- grouping forward, rows in shared memory

// Bounded wait for a TMA bulk copy into this CTA's shared memory (parity 0 of a fresh
// mbarrier).  Gives up after one second; the caller then records it in the device status
// word and stages the rows with plain loads instead.
__device__ __forceinline__ bool wait_bulk_copy(uint32_t mbar)
{
    unsigned long long t0 = 0;
    for (unsigned it = 1;; ++it)
    {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(mbar)
                     : "memory");
        if (ok) return true;
        if ((it & 255u) == 0u)
        {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > 1000000000ull)
                return false;
        }
    }
}

// A CTA stages ROWS consecutive (batch, channel) feature rows in shared memory - one TMA
// bulk copy per row when the rows are 16-byte aligned, coalesced loads otherwise - and
// then walks a chunk of output positions: per thread four consecutive positions, their
// indices loaded once (two 16-byte loads), ROWS x 4 shared-memory gathers, ROWS 16-byte
// streaming stores.  Gathering from shared memory instead of L1/L2 removes the
// sector-per-lane traffic that bounds the direct-gather kernel.
// Four consecutive indices of a position run: int64 as the callers pass them, or the 16-bit
// copy the fused set-abstraction op makes (0xFFFF = out of range).
constexpr uint16_t kBadIdx16 = 0xFFFFu;
__device__ __forceinline__ void load_four(const int64_t* p, int n, bool& bad, int& i0, int& i1, int& i2, int& i3)
{
    const longlong2 a = __ldg(reinterpret_cast<const longlong2*>(p));
    const longlong2 b2 = __ldg(reinterpret_cast<const longlong2*>(p) + 1);
    i0 = checked_index(a.x, n, bad);
    i1 = checked_index(a.y, n, bad);
    i2 = checked_index(b2.x, n, bad);
    i3 = checked_index(b2.y, n, bad);
}
__device__ __forceinline__ void load_four(const uint16_t* p, int, bool&, int& i0, int& i1, int& i2, int& i3)
{
    const ushort4 a = __ldg(reinterpret_cast<const ushort4*>(p));
    i0 = a.x == kBadIdx16 ? -1 : a.x;
    i1 = a.y == kBadIdx16 ? -1 : a.y;
    i2 = a.z == kBadIdx16 ? -1 : a.z;
    i3 = a.w == kBadIdx16 ? -1 : a.w;
}

template <int ROWS, class IdxT>
__global__ void __launch_bounds__(kScatterThreads)
    grouping_fwd_rows_kernel(int c, int n, long long ps, long long chunk, int use_tma, int out_c, int out_off,
                             const float* __restrict__ features, const IdxT* __restrict__ idx,
                             float* __restrict__ out)
{
    extern __shared__ __align__(128) float rows[];
    __shared__ __align__(8) uint64_t mbar;
    const int groups_per_batch = (c + ROWS - 1) / ROWS;
    const int bi = blockIdx.y / groups_per_batch;
    const int c0 = (blockIdx.y - bi * groups_per_batch) * ROWS;
    const int nrows = min(ROWS, c - c0);
    const float* src = features + (static_cast<size_t>(bi) * c + c0) * n;

    if (use_tma)
    {
        const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(&mbar));
        if (threadIdx.x == 0)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        if (threadIdx.x == 0)
        {
            const uint32_t bytes = static_cast<uint32_t>(nrows) * n * 4u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
            for (int r = 0; r < nrows; ++r)
            {
                const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(rows + static_cast<size_t>(r) * n));
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                    "l"(src + static_cast<size_t>(r) * n), "r"(static_cast<uint32_t>(n) * 4u), "r"(bar)
                    : "memory");
            }
        }
        // a copy that did not arrive in time is recorded and the rows are staged with plain loads
        use_tma = __syncthreads_or(wait_bulk_copy(bar) ? 0 : 1) == 0;
        if (!use_tma && threadIdx.x == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
    }
    if (!use_tma)
    {
        for (int i = threadIdx.x; i < nrows * n; i += kScatterThreads) rows[i] = __ldg(src + i);
        __syncthreads();
    }

    const long long p0 = static_cast<long long>(blockIdx.x) * chunk;
    const long long p1 = min(ps, p0 + chunk);
    const IdxT* ib = idx + static_cast<size_t>(bi) * ps;
    float* ob = out + (static_cast<size_t>(bi) * out_c + out_off + c0) * ps;
    bool bad = false;
    for (long long p = p0 + static_cast<long long>(threadIdx.x) * 4; p < p1; p += kScatterThreads * 4)
    {
        int i0, i1, i2, i3;
        load_four(ib + p, n, bad, i0, i1, i2, i3);
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
        {
            if (r < nrows)
            {
                const float* row = rows + static_cast<size_t>(r) * n;
                __stcs(reinterpret_cast<float4*>(ob + r * ps + p),
                       make_float4(gather_or_zero(row, i0), gather_or_zero(row, i1), gather_or_zero(row, i2),
                                   gather_or_zero(row, i3)));
            }
        }
    }
    report_bad(bad);
}

template <int ROWS, class IdxT>
int launch_grouping_fwd_rows(int b, int c, int n, long long ps, int out_c, int out_off, const float* features,
                             const IdxT* idx, float* out, cudaStream_t s)
{
    auto kernel = grouping_fwd_rows_kernel<ROWS, IdxT>;
    prefer_max_shared(kernel);
    const size_t smem = static_cast<size_t>(ROWS) * n * sizeof(float);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("grouping: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long groups = static_cast<long long>(b) * ((c + ROWS - 1) / ROWS);
    // split the positions so that every SM gets a few CTAs, in multiples of the 2048
    // positions one sweep of the CTA covers
    long long nchunks = (4ll * num_sms() + groups - 1) / groups;
    const long long max_chunks = (ps + 8191) / 8192;
    if (nchunks > max_chunks) nchunks = max_chunks;
    if (nchunks < 1) nchunks = 1;
    long long chunk = (ps + nchunks - 1) / nchunks;
    chunk = (chunk + 2047) / 2048 * 2048;
    nchunks = (ps + chunk - 1) / chunk;
    TPK_REQUIRE(groups <= 65535 && nchunks < (1ll << 31), "grouping: grid too large");
    const int use_tma = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(features) & 15u) == 0);
    const dim3 g(static_cast<unsigned>(nchunks), static_cast<unsigned>(groups));
    count_launches(1), kernel<<<g, kScatterThreads, smem, s>>>(c, n, ps, chunk, use_tma, out_c, out_off, features, idx, out);
    return check_launch("grouping");
}

// ---------------------------------------------------------- three_interpolate forward

template <bool VEC>
__global__ void __launch_bounds__(kGatherThreads)
    interp_fwd_kernel(int c, int m, int n, const float* __restrict__ points,
                      const int32_t* __restrict__ idx, const float* __restrict__ weight,
                      float* __restrict__ out)
{
    const int bi = blockIdx.z;
    const int c0 = blockIdx.y * kChanChunk;
    const int c1 = min(c, c0 + kChanChunk);
    const int j0 = (blockIdx.x * kGatherThreads + threadIdx.x) * 4;
    if (j0 >= n) return;
    bool bad = false;
    int id[4][3];
    float w[4][3];
#pragma unroll
    for (int t = 0; t < 4; ++t)
    {
        const bool ok = j0 + t < n;
        const size_t o = (static_cast<size_t>(bi) * n + (ok ? j0 + t : j0)) * 3;
#pragma unroll
        for (int k = 0; k < 3; ++k)
        {
            id[t][k] = checked_index(__ldg(idx + o + k), m, bad);
            w[t][k] = __ldg(weight + o + k);
        }
    }
    const float* f = points + (static_cast<size_t>(bi) * c + c0) * m;
    float* o = out + (static_cast<size_t>(bi) * c + c0) * n + j0;
#pragma unroll 2
    for (int ch = c0; ch < c1; ++ch, f += m, o += n)
    {
        float r[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
            r[t] = interp3(ldg_or_zero(f, id[t][0]), w[t][0], ldg_or_zero(f, id[t][1]), w[t][1],
                           ldg_or_zero(f, id[t][2]), w[t][2]);
        if (VEC)
            __stcs(reinterpret_cast<float4*>(o), make_float4(r[0], r[1], r[2], r[3]));
        else
        {
#pragma unroll
            for (int t = 0; t < 4; ++t)
                if (j0 + t < n) o[t] = r[t];
        }
    }
    report_bad(bad);
}

// --------------------------------------- three_interpolate forward, rows in shared memory

// Same residency scheme as grouping_fwd_rows_kernel: ROWS feature rows (length m) staged
// with TMA bulk copies, then every thread produces four consecutive outputs per row
// from 12 shared-memory gathers; the 12 indices and weights of its four points are
// loaded once (six 16-byte loads) for all rows.
template <int ROWS>
__global__ void __launch_bounds__(kGatherThreads)
    interp_fwd_rows_kernel(int c, int m, int n, int chunk, int use_tma,
                           const float* __restrict__ points, const int32_t* __restrict__ idx,
                           const float* __restrict__ weight, float* __restrict__ out)
{
    extern __shared__ __align__(128) float rows[];
    __shared__ __align__(8) uint64_t mbar;
    const int groups_per_batch = (c + ROWS - 1) / ROWS;
    const int bi = blockIdx.y / groups_per_batch;
    const int c0 = (blockIdx.y - bi * groups_per_batch) * ROWS;
    const int nrows = min(ROWS, c - c0);
    const float* src = points + (static_cast<size_t>(bi) * c + c0) * m;
    if (use_tma)
    {
        const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(&mbar));
        if (threadIdx.x == 0)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        if (threadIdx.x == 0)
        {
            // consecutive rows are contiguous in memory: one copy for all of them
            const uint32_t bytes = static_cast<uint32_t>(nrows) * m * 4u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
            const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(rows));
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                "l"(src), "r"(bytes), "r"(bar)
                : "memory");
        }
        use_tma = __syncthreads_or(wait_bulk_copy(bar) ? 0 : 1) == 0;
        if (!use_tma && threadIdx.x == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
    }
    if (!use_tma)
    {
        for (int i = threadIdx.x; i < nrows * m; i += kGatherThreads) rows[i] = __ldg(src + i);
        __syncthreads();
    }

    const int j_begin = blockIdx.x * chunk;
    const int j_end = min(n, j_begin + chunk);
    bool bad = false;
    for (int j0 = j_begin + threadIdx.x * 4; j0 < j_end; j0 += kGatherThreads * 4)
    {
        const size_t o = (static_cast<size_t>(bi) * n + j0) * 3;  // multiple of 12: 16-byte aligned
        int id[12];
        float w[12];
#pragma unroll
        for (int t = 0; t < 3; ++t)
        {
            const int4 a = __ldg(reinterpret_cast<const int4*>(idx + o) + t);
            const float4 b4 = __ldg(reinterpret_cast<const float4*>(weight + o) + t);
            id[4 * t + 0] = checked_index(a.x, m, bad); id[4 * t + 1] = checked_index(a.y, m, bad);
            id[4 * t + 2] = checked_index(a.z, m, bad); id[4 * t + 3] = checked_index(a.w, m, bad);
            w[4 * t + 0] = b4.x; w[4 * t + 1] = b4.y; w[4 * t + 2] = b4.z; w[4 * t + 3] = b4.w;
        }
        float* op = out + (static_cast<size_t>(bi) * c + c0) * n + j0;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
        {
            if (r < nrows)
            {
                const float* row = rows + r * m;
                float v[4];
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    v[t] = interp3(gather_or_zero(row, id[3 * t + 0]), w[3 * t + 0], gather_or_zero(row, id[3 * t + 1]),
                                   w[3 * t + 1], gather_or_zero(row, id[3 * t + 2]), w[3 * t + 2]);
                __stcs(reinterpret_cast<float4*>(op + static_cast<size_t>(r) * n), make_float4(v[0], v[1], v[2], v[3]));
            }
        }
    }
    report_bad(bad);
}

template <int ROWS>
int launch_interp_fwd_rows(int b, int c, int m, int n, const float* points, const int32_t* idx,
                           const float* weight, float* out, cudaStream_t s)
{
    auto kernel = interp_fwd_rows_kernel<ROWS>;
    prefer_max_shared(kernel);
    const size_t smem = static_cast<size_t>(ROWS) * m * sizeof(float);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("three_interpolate: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long groups = static_cast<long long>(b) * ((c + ROWS - 1) / ROWS);
    long long nchunks = (4ll * num_sms() + groups - 1) / groups;
    const long long max_chunks = (n + 4095) / 4096;
    if (nchunks > max_chunks) nchunks = max_chunks;
    if (nchunks < 1) nchunks = 1;
    int chunk = static_cast<int>((n + nchunks - 1) / nchunks);
    chunk = (chunk + 1023) / 1024 * 1024;
    nchunks = (n + chunk - 1) / chunk;
    TPK_REQUIRE(groups <= 65535, "three_interpolate: grid too large");
    const int use_tma = (m % 4 == 0) && ((reinterpret_cast<uintptr_t>(points) & 15u) == 0) &&
                        static_cast<size_t>(ROWS) * m * 4 < (1u << 20);
    const dim3 g(static_cast<unsigned>(nchunks), static_cast<unsigned>(groups));
    count_launches(1), kernel<<<g, kGatherThreads, smem, s>>>(c, m, n, chunk, use_tma, points, idx, weight, out);
    return check_launch("three_interpolate");
}

// ------------------------------------------------------------------ backward, shared rows

// Rows of the small gradient (length row_len) for `rows` consecutive (batch, channel)
// pairs live in shared memory.  INTERP == false: grouping (src positions ps, one int64
// index each).  INTERP == true: three_interpolate (src positions n, three int32
// indices and weights each).
template <bool INTERP>
__global__ void __launch_bounds__(kScatterThreads)
    scatter_rows_kernel(int c, int row_len, long long src_len, long long gbs, int rows, int vec_ok,
                        const float* __restrict__ grad_out, const void* __restrict__ idx_v,
                        const float* __restrict__ weight, float* __restrict__ grad_small)
{
    extern __shared__ __align__(16) float acc[];
    const int groups_per_batch = (c + rows - 1) / rows;
    const int bi = blockIdx.x / groups_per_batch;
    const int c0 = (blockIdx.x - bi * groups_per_batch) * rows;
    const int nrows = min(rows, c - c0);
    for (int i = threadIdx.x; i < nrows * row_len; i += kScatterThreads) acc[i] = 0.f;
    __syncthreads();

    const float* g = grad_out + static_cast<size_t>(bi) * gbs + static_cast<size_t>(c0) * src_len;
    bool bad = false;
    const bool vec = (src_len % 4 == 0) && vec_ok != 0;  // 16-byte loads need aligned inputs
    if (vec)
    {
        for (long long p = static_cast<long long>(threadIdx.x) * 4; p < src_len;
             p += kScatterThreads * 4)
        {
            if (!INTERP)
            {
                const int64_t* ip = static_cast<const int64_t*>(idx_v) + static_cast<size_t>(bi) * src_len + p;
                const longlong2 a = __ldg(reinterpret_cast<const longlong2*>(ip));
                const longlong2 b2 = __ldg(reinterpret_cast<const longlong2*>(ip) + 1);
                const int i0 = checked_index(a.x, row_len, bad), i1 = checked_index(a.y, row_len, bad);
                const int i2 = checked_index(b2.x, row_len, bad), i3 = checked_index(b2.y, row_len, bad);
                for (int r = 0; r < nrows; ++r)
                {
                    const float4 v = __ldcs(reinterpret_cast<const float4*>(g + r * src_len + p));
                    float* a_r = acc + r * row_len;
                    if (i0 >= 0) atomicAdd(a_r + i0, v.x);
                    if (i1 >= 0) atomicAdd(a_r + i1, v.y);
                    if (i2 >= 0) atomicAdd(a_r + i2, v.z);
                    if (i3 >= 0) atomicAdd(a_r + i3, v.w);
                }
            }
            else
            {
                const size_t o = (static_cast<size_t>(bi) * src_len + p) * 3;
                const int32_t* ip = static_cast<const int32_t*>(idx_v) + o;
                const float* wp = weight + o;
                int id[12];
                float w[12];
                // 12 consecutive values, 16-byte aligned because p is a multiple of 4
#pragma unroll
                for (int t = 0; t < 3; ++t)
                {
                    const int4 a = __ldg(reinterpret_cast<const int4*>(ip) + t);
                    const float4 b4 = __ldg(reinterpret_cast<const float4*>(wp) + t);
                    id[4 * t + 0] = checked_index(a.x, row_len, bad); id[4 * t + 1] = checked_index(a.y, row_len, bad);
                    id[4 * t + 2] = checked_index(a.z, row_len, bad); id[4 * t + 3] = checked_index(a.w, row_len, bad);
                    w[4 * t + 0] = b4.x; w[4 * t + 1] = b4.y; w[4 * t + 2] = b4.z; w[4 * t + 3] = b4.w;
                }
                for (int r = 0; r < nrows; ++r)
                {
                    const float4 v = __ldcs(reinterpret_cast<const float4*>(g + r * src_len + p));
                    const float gv[4] = {v.x, v.y, v.z, v.w};
                    float* a_r = acc + r * row_len;
#pragma unroll
                    for (int t = 0; t < 4; ++t)
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            if (id[3 * t + k] >= 0) atomicAdd(a_r + id[3 * t + k], __fmul_rn(gv[t], w[3 * t + k]));
                }
            }
        }
    }
    else
    {
        for (long long p = threadIdx.x; p < src_len; p += kScatterThreads)
        {
            if (!INTERP)
            {
                const int i0 = checked_index(
                    __ldg(static_cast<const int64_t*>(idx_v) + static_cast<size_t>(bi) * src_len + p), row_len, bad);
                if (i0 >= 0)
                    for (int r = 0; r < nrows; ++r) atomicAdd(acc + r * row_len + i0, g[r * src_len + p]);
            }
            else
            {
                const size_t o = (static_cast<size_t>(bi) * src_len + p) * 3;
                const int32_t* ip = static_cast<const int32_t*>(idx_v) + o;
                for (int r = 0; r < nrows; ++r)
                {
                    const float gv = g[r * src_len + p];
#pragma unroll
                    for (int k = 0; k < 3; ++k)
                    {
                        const int ik = checked_index(__ldg(ip + k), row_len, bad);
                        if (ik >= 0) atomicAdd(acc + r * row_len + ik, __fmul_rn(gv, __ldg(weight + o + k)));
                    }
                }
            }
        }
    }
    __syncthreads();
    float* dst = grad_small + (static_cast<size_t>(bi) * c + c0) * row_len;
    for (int i = threadIdx.x; i < nrows * row_len; i += kScatterThreads) dst[i] = acc[i];
    report_bad(bad);
}

// ------------------------------------------------------ grouping backward, shared rows

// A warp takes 32 consecutive positions at a time (one 128-byte line of every gradient
// row; with nsample = 32 exactly one neighbourhood).  Ball-query neighbourhoods repeat
// their first index in every unused slot, so many lanes of a warp often target the same
// feature column, and shared-memory float atomics serialise badly on one address.
// Lanes whose index equals that of the first lane of their neighbourhood segment are
// therefore summed with a shuffle butterfly and only the segment's first lane issues
// the atomic for them.  Any other repetition in idx is still correct: those lanes just
// use their own atomics.  `seg` = lanes per segment (a power of two <= 32; 1 = no
// pre-reduction, used when nsample is not a power of two).
template <int ROWS, int SEG>
__global__ void __launch_bounds__(kScatterThreads)
    grouping_bwd_rows_kernel(int c, int row_len, long long src_len, long long gbs,
                             const float* __restrict__ grad_out, const int64_t* __restrict__ idx,
                             float* __restrict__ grad_small)
{
    constexpr int UNROLL = 4;
    constexpr int NWARPS = kScatterThreads / 32;
    extern __shared__ __align__(16) float acc[];
    const int groups_per_batch = (c + ROWS - 1) / ROWS;
    const int bi = blockIdx.x / groups_per_batch;
    const int c0 = (blockIdx.x - bi * groups_per_batch) * ROWS;
    const int nrows = min(ROWS, c - c0);
    for (int i = threadIdx.x; i < nrows * row_len; i += kScatterThreads) acc[i] = 0.f;
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool bad = false;
    const int seg_first = lane & ~(SEG - 1);
    const long long nfull = src_len / 32;  // whole 32-position sets
    // this lane's element of set `warp`; sets advance by NWARPS per step
    const int64_t* ip = idx + static_cast<size_t>(bi) * src_len + warp * 32 + lane;
    const float* gp[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
        gp[r] = grad_out + static_cast<size_t>(bi) * gbs + static_cast<size_t>(c0 + (r < nrows ? r : 0)) * src_len + warp * 32 + lane;

    for (long long set = warp; set < nfull; set += NWARPS * UNROLL)
    {
        int id[UNROLL];
        float v[UNROLL][ROWS];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
        {
            if (set + u * NWARPS < nfull)  // warp-uniform
            {
                id[u] = checked_index(__ldg(ip + u * (NWARPS * 32)), row_len, bad);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) v[u][r] = __ldcs(gp[r] + u * (NWARPS * 32));
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
        {
            if (set + u * NWARPS >= nfull) break;  // warp-uniform
            bool mine = true;  // this lane issues its own atomic
            if (SEG > 1)
            {
                const int first_id = __shfl_sync(kFullMask, id[u], seg_first);
                const bool same = id[u] == first_id;  // true for the segment's first lane too
                mine = !same || lane == seg_first;
                if (__ballot_sync(kFullMask, !mine) != 0u)
                {
#pragma unroll
                    for (int r = 0; r < ROWS; ++r)
                    {
                        float sum = same ? v[u][r] : 0.f;
#pragma unroll
                        for (int o = SEG / 2; o >= 1; o >>= 1) sum += __shfl_xor_sync(kFullMask, sum, o);
                        if (lane == seg_first) v[u][r] = sum;
                    }
                }
            }
            if (mine && id[u] >= 0)  // an index out of range (-1) is dropped, with everything folded into it
            {
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r < nrows) atomicAdd(acc + r * row_len + id[u], v[u][r]);
            }
        }
        ip += NWARPS * UNROLL * 32;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) gp[r] += NWARPS * UNROLL * 32;
    }
    // the last src_len % 32 positions
    if (warp == 0)
    {
        const long long p = nfull * 32 + lane;
        if (p < src_len)
        {
            const int i0 = checked_index(__ldg(idx + static_cast<size_t>(bi) * src_len + p), row_len, bad);
            if (i0 >= 0)
                for (int r = 0; r < nrows; ++r)
                    atomicAdd(acc + r * row_len + i0,
                              grad_out[static_cast<size_t>(bi) * gbs + static_cast<size_t>(c0 + r) * src_len + p]);
        }
    }
    __syncthreads();
    float* dst = grad_small + (static_cast<size_t>(bi) * c + c0) * row_len;
    for (int i = threadIdx.x; i < nrows * row_len; i += kScatterThreads) dst[i] = acc[i];
    report_bad(bad);
}

template <int ROWS, int SEG>
int launch_grouping_bwd_rows_seg(int b, int c, int row_len, long long src_len, long long gbs, const float* grad_out,
                                 const int64_t* idx, float* grad_small, cudaStream_t s)
{
    auto kernel = grouping_bwd_rows_kernel<ROWS, SEG>;
    prefer_max_shared(kernel);
    const size_t smem = static_cast<size_t>(ROWS) * row_len * sizeof(float);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("grouping_grad: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long grid = static_cast<long long>(b) * ((c + ROWS - 1) / ROWS);
    TPK_REQUIRE(grid < (1ll << 31), "grouping_grad: too many rows");
    count_launches(1), kernel<<<static_cast<unsigned>(grid), kScatterThreads, smem, s>>>(c, row_len, src_len, gbs, grad_out, idx,
                                                                    grad_small);
    return check_launch("grouping_grad");
}

template <int ROWS>
int launch_grouping_bwd_rows(int b, int c, int row_len, long long src_len, long long gbs, int nsample,
                             const float* grad_out, const int64_t* idx, float* grad_small,
                             cudaStream_t s)
{
    // neighbourhood segments line up with warps when nsample is a power of two
    int seg = 1;
    if (nsample > 1 && (nsample & (nsample - 1)) == 0) seg = nsample < 32 ? nsample : 32;
    switch (seg)
    {
    case 32: return launch_grouping_bwd_rows_seg<ROWS, 32>(b, c, row_len, src_len, gbs, grad_out, idx, grad_small, s);
    case 16: return launch_grouping_bwd_rows_seg<ROWS, 16>(b, c, row_len, src_len, gbs, grad_out, idx, grad_small, s);
    case 8: return launch_grouping_bwd_rows_seg<ROWS, 8>(b, c, row_len, src_len, gbs, grad_out, idx, grad_small, s);
    default: return launch_grouping_bwd_rows_seg<ROWS, 1>(b, c, row_len, src_len, gbs, grad_out, idx, grad_small, s);
    }
}

// ------------------------------------------- three_interpolate backward, shared rows

// ROWS rows of the small gradient (length m) in shared memory; every warp streams sets of
// 32 consecutive points: their three indices and weights are loaded once, then per row
// one coalesced load of the incoming gradient and three shared-memory atomics.
template <int ROWS, int THREADS>
__global__ void __launch_bounds__(THREADS)
    interp_bwd_rows_kernel(int c, int m, int n, const float* __restrict__ grad_out,
                           const int32_t* __restrict__ idx, const float* __restrict__ weight,
                           float* __restrict__ grad_points)
{
    constexpr int NWARPS = THREADS / 32;
    extern __shared__ __align__(16) float acc[];
    const int groups_per_batch = (c + ROWS - 1) / ROWS;
    const int bi = blockIdx.x / groups_per_batch;
    const int c0 = (blockIdx.x - bi * groups_per_batch) * ROWS;
    const int nrows = min(ROWS, c - c0);
    for (int i = threadIdx.x; i < nrows * m; i += THREADS) acc[i] = 0.f;
    __syncthreads();

    const float* g = grad_out + (static_cast<size_t>(bi) * c + c0) * n;
    bool bad = false;
    for (int j = threadIdx.x; j < n; j += THREADS)
    {
        const size_t o = (static_cast<size_t>(bi) * n + j) * 3;
        const int i0 = checked_index(__ldg(idx + o), m, bad), i1 = checked_index(__ldg(idx + o + 1), m, bad),
                  i2 = checked_index(__ldg(idx + o + 2), m, bad);
        const float w0 = __ldg(weight + o), w1 = __ldg(weight + o + 1), w2 = __ldg(weight + o + 2);
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
        {
            if (r < nrows)
            {
                const float gv = __ldcs(g + static_cast<size_t>(r) * n + j);
                float* a = acc + r * m;
                if (i0 >= 0) atomicAdd(a + i0, __fmul_rn(gv, w0));
                if (i1 >= 0) atomicAdd(a + i1, __fmul_rn(gv, w1));
                if (i2 >= 0) atomicAdd(a + i2, __fmul_rn(gv, w2));
            }
        }
    }
    (void)NWARPS;
    __syncthreads();
    float* dst = grad_points + (static_cast<size_t>(bi) * c + c0) * m;
    for (int i = threadIdx.x; i < nrows * m; i += THREADS) dst[i] = acc[i];
    report_bad(bad);
}

template <int ROWS, int THREADS>
int launch_interp_bwd_rows(int b, int c, int m, int n, const float* grad_out, const int32_t* idx,
                           const float* weight, float* grad_points, cudaStream_t s)
{
    auto kernel = interp_bwd_rows_kernel<ROWS, THREADS>;
    prefer_max_shared(kernel);
    const size_t smem = static_cast<size_t>(ROWS) * m * sizeof(float);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("three_interpolate_grad: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long grid = static_cast<long long>(b) * ((c + ROWS - 1) / ROWS);
    TPK_REQUIRE(grid < (1ll << 31), "three_interpolate_grad: too many rows");
    count_launches(1), kernel<<<static_cast<unsigned>(grid), THREADS, smem, s>>>(c, m, n, grad_out, idx, weight, grad_points);
    return check_launch("three_interpolate_grad");
}

// ------------------------------------------------------------------ backward, global atomics

template <bool INTERP>
__global__ void __launch_bounds__(kGatherThreads)
    scatter_global_kernel(int c, int row_len, long long src_len, long long gbs, const float* __restrict__ grad_out,
                          const void* __restrict__ idx_v, const float* __restrict__ weight,
                          float* __restrict__ grad_small)
{
    const int bi = blockIdx.z;
    const int c0 = blockIdx.y * kChanChunk;
    const int c1 = min(c, c0 + kChanChunk);
    const long long p = static_cast<long long>(blockIdx.x) * kGatherThreads + threadIdx.x;
    if (p >= src_len) return;
    bool bad = false;
    int id[3];
    float w[3] = {1.f, 1.f, 1.f};
    if (!INTERP)
        id[0] = checked_index(__ldg(static_cast<const int64_t*>(idx_v) + static_cast<size_t>(bi) * src_len + p), row_len, bad);
    else
    {
        const size_t o = (static_cast<size_t>(bi) * src_len + p) * 3;
#pragma unroll
        for (int k = 0; k < 3; ++k)
        {
            id[k] = checked_index(__ldg(static_cast<const int32_t*>(idx_v) + o + k), row_len, bad);
            w[k] = __ldg(weight + o + k);
        }
    }
    for (int ch = c0; ch < c1; ++ch)
    {
        const float gv = __ldg(grad_out + static_cast<size_t>(bi) * gbs + static_cast<size_t>(ch) * src_len + p);
        float* dst = grad_small + (static_cast<size_t>(bi) * c + ch) * row_len;
        if (!INTERP)
        {
            if (id[0] >= 0) atomicAdd(dst + id[0], gv);
        }
        else
        {
#pragma unroll
            for (int k = 0; k < 3; ++k)
                if (id[k] >= 0) atomicAdd(dst + id[k], __fmul_rn(gv, w[k]));
        }
    }
    report_bad(bad);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <bool INTERP>
int launch_scatter(int b, int c, int row_len, long long src_len, long long gbs, const float* grad_out,
                   const void* idx, const float* weight, float* grad_small, cudaStream_t s,
                   const char* what)
{
    const size_t row_bytes = static_cast<size_t>(row_len) * sizeof(float);
    const bool force_global = test_path("scatter_global");
    if (row_bytes <= kRowSmemBudget && !force_global)
    {
        int rows = static_cast<int>(kRowSmemBudget / row_bytes);
        if (rows > 4) rows = 4;
        if (rows > c) rows = c;
        // keep at least ~2 CTAs per SM when the problem allows it
        while (rows > 1 && static_cast<long long>(b) * ((c + rows - 1) / rows) < 2ll * num_sms()) --rows;
        const size_t smem = static_cast<size_t>(rows) * row_bytes;
        auto kernel = scatter_rows_kernel<INTERP>;
        prefer_max_shared(kernel);
        if (smem > kDynSmemOptIn)
        {
            cudaError_t err = cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (err != cudaSuccess)
            {
                set_error("%s: shared memory attribute: %s", what, cudaGetErrorString(err));
                return TPK_ERR_CUDA;
            }
        }
        const long long grid = static_cast<long long>(b) * ((c + rows - 1) / rows);
        TPK_REQUIRE(grid < (1ll << 31), "%s: too many rows", what);
        const int vec_ok = aligned16(grad_out) && gbs % 4 == 0 && aligned16(idx) && (weight == nullptr || aligned16(weight));
        count_launches(1), kernel<<<static_cast<unsigned>(grid), kScatterThreads, smem, s>>>(
            c, row_len, src_len, gbs, rows, vec_ok, grad_out, idx, weight, grad_small);
        return check_launch(what);
    }
    cudaError_t err = cudaMemsetAsync(grad_small, 0, static_cast<size_t>(b) * c * row_bytes, s);
    if (err != cudaSuccess)
    {
        set_error("%s: memset: %s", what, cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    const long long gx = (src_len + kGatherThreads - 1) / kGatherThreads;
    TPK_REQUIRE(gx < (1ll << 31) && b <= 65535 && (c + kChanChunk - 1) / kChanChunk <= 65535,
                "%s: grid too large", what);
    const dim3 g(static_cast<unsigned>(gx), (c + kChanChunk - 1) / kChanChunk, b);
    count_launches(1), scatter_global_kernel<INTERP><<<g, kGatherThreads, 0, s>>>(c, row_len, src_len, gbs, grad_out, idx,
                                                              weight, grad_small);
    return check_launch(what);
}

}  // namespace
}  // namespace tpk

namespace tpk
{
namespace
{
// out[b, out_off + ch, p] = features[b, ch, idx[b, p]] for ch < c, rows of out_c per batch element.
// idx16 (optional): a 16-bit copy of idx, read instead of it by the row-resident kernel.
int grouping_forward(int b, int c, int n, long long ps, int out_c, int out_off, const float* features, const int64_t* idx,
                     const uint16_t* idx16, float* out, cudaStream_t s)
{
    const size_t row_bytes = static_cast<size_t>(n) * sizeof(float);
    if (ps % 4 == 0 && aligned16(idx) && aligned16(out) && row_bytes <= kRowSmemBudget && ps >= 4096 &&
        static_cast<long long>(b) * c <= 65535 && !test_path("gather_direct"))
    {
        // rows per CTA: as many as fit the shared memory of one SM, at most 4 (the indices
        // of a position are loaded once for all rows of the CTA)
        int rows = static_cast<int>(kRowSmemBudget / row_bytes);
        if (rows < 1) rows = 1;
        if (rows > 4) rows = 4;
        if (rows > c) rows = c;
#define TPK_GF(R)                                                                                                      \
    return idx16 ? launch_grouping_fwd_rows<R, uint16_t>(b, c, n, ps, out_c, out_off, features, idx16, out, s)         \
                 : launch_grouping_fwd_rows<R, int64_t>(b, c, n, ps, out_c, out_off, features, idx, out, s)
        switch (rows)
        {
        case 1: TPK_GF(1);
        case 2: TPK_GF(2);
        case 3: TPK_GF(3);
        default: TPK_GF(4);
        }
#undef TPK_GF
    }
    const long long gx = (ps + kGatherThreads * 4 - 1) / (kGatherThreads * 4);
    const int gy = (c + kChanChunk - 1) / kChanChunk;
    TPK_REQUIRE(gx < (1ll << 31) && gy <= 65535 && b <= 65535, "grouping: grid too large");
    const dim3 g(static_cast<unsigned>(gx), gy, b);
    if (ps % 4 == 0 && aligned16(idx) && aligned16(out))
        count_launches(1), grouping_fwd_kernel<true><<<g, kGatherThreads, 0, s>>>(c, n, ps, out_c, out_off, features, idx, out);
    else
        count_launches(1), grouping_fwd_kernel<false><<<g, kGatherThreads, 0, s>>>(c, n, ps, out_c, out_off, features, idx, out);
    return check_launch("grouping");
}

// ------------------------------------------------------- fused set-abstraction grouping
//
// The three coordinate rows of the fused op: out[b, a, p, s] = xyz[b, idx[b, p, s], a] - new_xyz[b, p, a]
// (what callers compute as grouping_operation(xyz^T, idx) - new_xyz^T[..., None]); also writes the
// 16-bit copy of idx the feature kernel reads.
__global__ void __launch_bounds__(kGatherThreads)
    sa_group_xyz_kernel(long long total, int n, int m, int nsample, int out_c, const float* __restrict__ xyz,
                        const float* __restrict__ new_xyz, const int64_t* __restrict__ idx, float* __restrict__ out,
                        uint16_t* __restrict__ idx16)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGatherThreads + threadIdx.x;
    if (t >= total) return;
    const long long ps = static_cast<long long>(m) * nsample;
    const long long bi = t / ps, pos = t - bi * ps;
    const long long centre = bi * m + pos / nsample;
    bool bad = false;
    const int i = checked_index(__ldg(idx + t), n, bad);
    if (idx16) idx16[t] = i < 0 ? kBadIdx16 : static_cast<uint16_t>(i);
    float* o = out + bi * out_c * ps + pos;
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
        const float v = i < 0 ? 0.f : __ldg(xyz + (bi * n + i) * 3 + a);
        o[a * ps] = __fsub_rn(v, __ldg(new_xyz + centre * 3 + a));
    }
    report_bad(bad);
}

__global__ void __launch_bounds__(kGatherThreads)
    gather_centres_kernel(long long total, int n, int m, const float* __restrict__ xyz, const int32_t* __restrict__ fps_idx,
                          float* __restrict__ new_xyz)
{
    const long long t = static_cast<long long>(blockIdx.x) * kGatherThreads + threadIdx.x;
    if (t >= total) return;
    bool bad = false;
    const int i = checked_index(__ldg(fps_idx + t), n, bad);
    const float* src = xyz + ((t / m) * n + (i < 0 ? 0 : i)) * 3;
    new_xyz[3 * t + 0] = __ldg(src + 0);
    new_xyz[3 * t + 1] = __ldg(src + 1);
    new_xyz[3 * t + 2] = __ldg(src + 2);
    report_bad(bad);
}
}  // namespace
}  // namespace tpk

extern "C" int tpk_grouping(int b, int c, int n, int npoint, int nsample, const float* features,
                            const int64_t* idx, float* out, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && c >= 0 && n >= 0 && npoint >= 0 && nsample >= 0, "grouping: negative size");
    const long long ps = static_cast<long long>(npoint) * nsample;
    if (b == 0 || c == 0 || ps == 0) return TPK_OK;
    TPK_REQUIRE(features && idx && out && n > 0, "grouping: NULL pointer or empty feature row");
    return grouping_forward(b, c, n, ps, c, 0, features, idx, nullptr, out, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t tpk_sa_group_scratch_bytes(int b, int n, int m, int nsample)
{
    if (b <= 0 || n <= 0 || m <= 0 || nsample <= 0) return 0;
    const int64_t per = static_cast<int64_t>(b) * m * nsample;
    // ball-query scratch, its distances (the fused op does not return them), the 16-bit indices
    return (tpk_ball_query_dense_scratch_bytes(b, n, m, nsample) + 255) / 256 * 256 + (per * 4 + 255) / 256 * 256 +
           (per * 2 + 255) / 256 * 256;
}

extern "C" int tpk_sa_group(int b, int n, int m, int c, float radius, int nsample, const float* xyz, const float* features,
                            const int32_t* fps_idx, float* new_xyz, int64_t* idx, float* out, void* scratch,
                            int64_t scratch_bytes, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0 && c >= 0 && nsample >= 0, "sa_group: negative size");
    if (b == 0 || m == 0 || nsample == 0) return TPK_OK;
    TPK_REQUIRE(n > 0, "sa_group: empty cloud");
    TPK_REQUIRE(xyz && fps_idx && new_xyz && idx && out && (features || c == 0), "sa_group: NULL pointer");
    const int64_t want = tpk_sa_group_scratch_bytes(b, n, m, nsample);
    if (scratch == nullptr || scratch_bytes < want)
    {
        set_error("sa_group: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch ? scratch_bytes : 0),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "sa_group: scratch must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t per = static_cast<int64_t>(b) * m * nsample;
    const int64_t bq_bytes = (tpk_ball_query_dense_scratch_bytes(b, n, m, nsample) + 255) / 256 * 256;
    unsigned char* p = static_cast<unsigned char*>(scratch);
    void* bq_scratch = bq_bytes ? p : nullptr;
    float* dist = reinterpret_cast<float*>(p + bq_bytes);
    uint16_t* idx16 = n < 65535 ? reinterpret_cast<uint16_t*>(p + bq_bytes + (per * 4 + 255) / 256 * 256) : nullptr;

    // 1. the centres
    const long long centres = static_cast<long long>(b) * m;
    TPK_REQUIRE((centres + kGatherThreads - 1) / kGatherThreads < (1ll << 31) && (per + kGatherThreads - 1) / kGatherThreads < (1ll << 31),
                "sa_group: problem too large for one launch");
    count_launches(1), gather_centres_kernel<<<static_cast<unsigned>((centres + kGatherThreads - 1) / kGatherThreads), kGatherThreads, 0, s>>>(
        centres, n, m, xyz, fps_idx, new_xyz);
    // 2. their neighbourhoods (grid search where the cloud is large enough, the scan otherwise)
    int rc = tpk_ball_query_dense_ws(b, n, m, radius, nsample, new_xyz, xyz, idx, dist, bq_scratch, bq_bytes, stream);
    if (rc != TPK_OK) return rc;
    // 3. relative coordinates (rows 0..2) and the 16-bit indices, then the features (rows 3..)
    const int out_c = 3 + c;
    count_launches(1), sa_group_xyz_kernel<<<static_cast<unsigned>((per + kGatherThreads - 1) / kGatherThreads), kGatherThreads, 0, s>>>(
        per, n, m, nsample, out_c, xyz, new_xyz, idx, out, idx16);
    rc = check_launch("sa_group");
    if (rc != TPK_OK || c == 0) return rc;
    return grouping_forward(b, c, n, static_cast<long long>(m) * nsample, out_c, 3, features, idx, idx16, out, s);
}

namespace tpk
{
// Gradient of grouping with shared-memory (or, for long rows, global) atomics.  Row (bi, ch) of
// the incoming gradient starts at grad_out + bi * gbs + ch * npoint * nsample: gbs is the batch
// stride in floats (c * npoint * nsample for a plain (b,c,npoint,nsample) tensor; the fused
// set-abstraction op passes the feature rows of its (b,3+c,npoint,nsample) gradient).
int grouping_grad_atomic(int b, int c, int n, int npoint, int nsample, const float* grad_out, long long gbs,
                         const int64_t* idx, float* grad_features, cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && c >= 0 && n >= 0 && npoint >= 0 && nsample >= 0,
                "grouping_grad: negative size");
    if (b == 0 || c == 0 || n == 0) return TPK_OK;
    TPK_REQUIRE(grad_features, "grouping_grad: NULL pointer");
    const long long ps = static_cast<long long>(npoint) * nsample;
    if (ps == 0)
    {
        cudaError_t err = cudaMemsetAsync(grad_features, 0, sizeof(float) * static_cast<size_t>(b) * c * n, s);
        if (err != cudaSuccess)
        {
            set_error("grouping_grad: memset: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
        return TPK_OK;
    }
    TPK_REQUIRE(grad_out && idx, "grouping_grad: NULL pointer");
    const size_t row_bytes = static_cast<size_t>(n) * sizeof(float);
    // (no alignment beyond the elements' own is needed: a view at an odd offset is fine)
    if (row_bytes <= kRowSmemBudget && !test_path("scatter_global"))
    {
        // rows per CTA: as many as fit 32 KB, at least one, at most 4, fewer when that would
        // leave SMs without a CTA (measured on the pipeline's shapes: the atomics want many
        // resident warps more than they want the indices shared between rows)
        int rows = static_cast<int>(32 * 1024 / row_bytes);
        if (rows < 1) rows = 1;
        if (rows > 4) rows = 4;
        if (rows > c) rows = c;
        while (rows > 1 && static_cast<long long>(b) * ((c + rows - 1) / rows) < 2ll * num_sms()) --rows;
        switch (rows)
        {
        case 1: return launch_grouping_bwd_rows<1>(b, c, n, ps, gbs, nsample, grad_out, idx, grad_features, s);
        case 2: return launch_grouping_bwd_rows<2>(b, c, n, ps, gbs, nsample, grad_out, idx, grad_features, s);
        case 3: return launch_grouping_bwd_rows<3>(b, c, n, ps, gbs, nsample, grad_out, idx, grad_features, s);
        default: return launch_grouping_bwd_rows<4>(b, c, n, ps, gbs, nsample, grad_out, idx, grad_features, s);
        }
    }
    return launch_scatter<false>(b, c, n, ps, gbs, grad_out, idx, nullptr, grad_features, s, "grouping_grad");
}
}  // namespace tpk

extern "C" int tpk_grouping_grad(int b, int c, int n, int npoint, int nsample,
                                 const float* grad_out, const int64_t* idx, float* grad_features,
                                 void* stream)
{
    return tpk::grouping_grad_atomic(b, c, n, npoint, nsample, grad_out,
                                     static_cast<long long>(c) * npoint * nsample, idx, grad_features,
                                     static_cast<cudaStream_t>(stream));
}

extern "C" int tpk_three_interpolate(int b, int c, int m, int n, const float* points,
                                     const int32_t* idx, const float* weight, float* out,
                                     void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && c >= 0 && m >= 0 && n >= 0, "three_interpolate: negative size");
    if (b == 0 || c == 0 || n == 0) return TPK_OK;
    TPK_REQUIRE(points && idx && weight && out && m > 0,
                "three_interpolate: NULL pointer or empty feature row");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n % 4 == 0 && aligned16(out) && aligned16(idx) && aligned16(weight) && n >= 1024 &&
        static_cast<size_t>(m) * 4 * 4 <= kRowSmemBudget && static_cast<long long>(b) * c <= 65535 &&
        !test_path("gather_direct"))
    {
        if (c >= 8 && static_cast<size_t>(m) * 4 * 8 <= 128 * 1024)
            return launch_interp_fwd_rows<8>(b, c, m, n, points, idx, weight, out, s);
        return launch_interp_fwd_rows<4>(b, c, m, n, points, idx, weight, out, s);
    }
    const int gx = (n + kGatherThreads * 4 - 1) / (kGatherThreads * 4);
    const int gy = (c + kChanChunk - 1) / kChanChunk;
    TPK_REQUIRE(gy <= 65535 && b <= 65535, "three_interpolate: grid too large");
    const dim3 g(gx, gy, b);
    if (n % 4 == 0 && aligned16(out))
        count_launches(1), interp_fwd_kernel<true><<<g, kGatherThreads, 0, s>>>(c, m, n, points, idx, weight, out);
    else
        count_launches(1), interp_fwd_kernel<false><<<g, kGatherThreads, 0, s>>>(c, m, n, points, idx, weight, out);
    return check_launch("three_interpolate");
}

extern "C" int tpk_three_interpolate_grad(int b, int c, int n, int m, const float* grad_out,
                                          const int32_t* idx, const float* weight,
                                          float* grad_points, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && c >= 0 && m >= 0 && n >= 0, "three_interpolate_grad: negative size");
    if (b == 0 || c == 0 || m == 0) return TPK_OK;
    TPK_REQUIRE(grad_points, "three_interpolate_grad: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n == 0)
    {
        cudaError_t err = cudaMemsetAsync(grad_points, 0, sizeof(float) * static_cast<size_t>(b) * c * m, s);
        if (err != cudaSuccess)
        {
            set_error("three_interpolate_grad: memset: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
        return TPK_OK;
    }
    TPK_REQUIRE(grad_out && idx && weight, "three_interpolate_grad: NULL pointer");
    if (static_cast<size_t>(m) * 4 * 4 <= 64 * 1024 && !test_path("scatter_global"))
    {
        // measured on the four pipeline shapes: few rows per CTA and small blocks win (many
        // resident CTAs hide the latency of the index/weight loads and of the atomics)
        if (n >= 8192) return launch_interp_bwd_rows<1, 256>(b, c, m, n, grad_out, idx, weight, grad_points, s);
        if (n >= 2048) return launch_interp_bwd_rows<2, 128>(b, c, m, n, grad_out, idx, weight, grad_points, s);
        return launch_interp_bwd_rows<4, 128>(b, c, m, n, grad_out, idx, weight, grad_points, s);
    }
    return launch_scatter<true>(b, c, m, n, static_cast<long long>(c) * n, grad_out, idx, weight, grad_points, s,
                                "three_interpolate_grad");
}
