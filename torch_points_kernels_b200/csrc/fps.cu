// Furthest point sampling for sm_100a.
//
// One thread-block cluster per cloud.  Every thread keeps its points' coordinates and
// running min-distance in registers for the whole call; a round costs one distance
// update per point, a two-instruction warp arg-max (redux.sync), and one exchange of
// 20-byte messages between the warps of the cluster through distributed shared
// memory.  Nothing is re-read from global memory after the initial load and the only
// global store per round is the selected index.
//
// Behaviour follows cuda/src/sampling_gpu.cu:16-144 of the reference bit for bit:
// first sample is index 0; squared distance contracted as in tpk::sumsq_abc; points
// with |p|^2 <= 1e-3 (compared in double) are never updated nor selected; a point's
// running minimum starts at 1e10; among equal maxima the winner is the one the
// reference's strided scan plus shared-memory tree would keep.  That tie rule is
// encoded as a rank: with bs = largest power of two <= n (at most 512) the reference
// prefers the smallest bit-reversed (k mod bs), then the smallest (k div bs).
#include <cooperative_groups.h>

#include "tpk_common.cuh"

namespace cg = cooperative_groups;

namespace tpk
{
namespace
{

__device__ int g_dev_status = 0;

constexpr int kFpsMaxThreads = 512;
constexpr int kFpsMaxRanks = 16;
constexpr int kFpsMaxPpt = 16;
constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // give up a wait after one second
constexpr int kMsgBytes = 20;  // {key_hi, key_lo, x, y} + {z}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_msg(uint32_t addr_a, uint32_t addr_z, uint32_t hi,
                                               uint32_t lo, float x, float y, float z)
{
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr_a), "r"(hi),
                 "r"(lo), "r"(__float_as_uint(x)), "r"(__float_as_uint(y))
                 : "memory");
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr_z), "r"(__float_as_uint(z))
                 : "memory");
}
// Remote store that signals the destination CTA's mbarrier with the bytes written.
__device__ __forceinline__ void st_async_msg(uint32_t addr_a, uint32_t addr_z, uint32_t mbar,
                                             uint32_t hi, uint32_t lo, float x, float y, float z)
{
    asm volatile(
        "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::
            "r"(addr_a), "r"(hi), "r"(lo), "r"(__float_as_uint(x)), "r"(__float_as_uint(y)), "r"(mbar)
        : "memory");
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::
                     "r"(addr_z), "r"(__float_as_uint(z)), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t mbar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(mbar), "r"(parity)
                 : "memory");
    return ok != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for the phase with the given parity; false if it has not completed within
// kWaitLimitNs (the clock is read only every 256 unsuccessful polls).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity)
{
    unsigned long long t0 = 0;
    for (unsigned it = 1;; ++it)
    {
        if (mbar_try_wait(mbar, parity)) return true;
        if ((it & 255u) == 0u)
        {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > kWaitLimitNs)
                return false;
        }
    }
}

__device__ __forceinline__ uint32_t bitrev_low(uint32_t v, int bits)
{
    return bits == 0 ? 0u : (__brev(v) >> (32 - bits));
}

// SYNC == 0: messages are plain distributed-shared-memory stores followed by a cluster
//            barrier (or __syncthreads for a one-CTA cluster).
// SYNC == 1: messages are st.async stores that complete a transaction count on the
//            receiver's mbarrier; receivers wait (bounded) on their own barrier and no
//            CTA-wide or cluster-wide barrier is executed inside the round loop.
template <int PPT, int SYNC>
__global__ void __launch_bounds__(kFpsMaxThreads, 1)
    fps_onchip_kernel(int n, int m, int log2bs, const float* __restrict__ xyz_all,
                      int32_t* __restrict__ idxs_all)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int nranks = static_cast<int>(cluster_nctarank());
    const int rank = static_cast<int>(cluster_ctarank());
    const int cloud = blockIdx.x / nranks;
    const int total = nranks * nthreads;
    const int gtid = rank * nthreads + tid;
    const int nslots = nranks * nwarps;

    // shared memory: msg_a[2][nslots] (16 B), msg_z[2][nslots] (4 B), 2 mbarriers, xyz copy
    uint4* msg_a = reinterpret_cast<uint4*>(smem_raw);
    float* msg_z = reinterpret_cast<float*>(msg_a + 2 * nslots);
    uint64_t* mbar = reinterpret_cast<uint64_t*>(smem_raw + 2 * nslots * kMsgBytes +
                                                 ((2 * nslots * kMsgBytes) & 8));
    float* sxyz = reinterpret_cast<float*>(mbar + 2);

    const float* xyz = xyz_all + static_cast<size_t>(cloud) * n * 3;
    int32_t* idxs = idxs_all + static_cast<size_t>(cloud) * m;

    float px[PPT], py[PPT], pz[PPT], md[PPT];
#pragma unroll
    for (int p = 0; p < PPT; ++p)
    {
        const int k = p * total + gtid;
        float x = 0.f, y = 0.f, z = 0.f;
        bool valid = false;
        if (k < n)
        {
            x = __ldg(xyz + 3 * static_cast<size_t>(k) + 0);
            y = __ldg(xyz + 3 * static_cast<size_t>(k) + 1);
            z = __ldg(xyz + 3 * static_cast<size_t>(k) + 2);
            const float mag = sumsq_abc(x, y, z);
            valid = !(static_cast<double>(mag) <= 1e-3);
        }
        px[p] = x;
        py[p] = y;
        pz[p] = z;
        // a negative running minimum marks "never a candidate": fminf keeps it negative
        md[p] = valid ? 1e10f : -1.0f;
        float* s = sxyz + (static_cast<size_t>(p) * nthreads + tid) * 3;
        s[0] = x;
        s[1] = y;
        s[2] = z;
    }

    // tie-break rank of point k = p*total + gtid (total is a multiple of bs)
    const uint32_t bs_mask = (1u << log2bs) - 1u;
    const uint32_t rbase = (bitrev_low(static_cast<uint32_t>(gtid) & bs_mask, log2bs) << 22) |
                           (static_cast<uint32_t>(gtid) >> log2bs);
    const uint32_t rstep = static_cast<uint32_t>(total) >> log2bs;

    float cx = 0.f, cy = 0.f, cz = 0.f;
    if (n > 0)
    {
        cx = __ldg(xyz + 0);
        cy = __ldg(xyz + 1);
        cz = __ldg(xyz + 2);
    }
    if (gtid == 0 && m > 0) idxs[0] = 0;

    if (SYNC == 1)
    {
        if (tid == 0)
        {
            mbar_init(smem_u32(mbar + 0), 1);
            mbar_init(smem_u32(mbar + 1), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    if (nranks > 1)
        cluster_sync_all();
    else
        __syncthreads();

    const uint32_t my_slot = static_cast<uint32_t>(rank * nwarps + warp);
    bool failed = false;

    for (int j = 1; j < m; ++j)
    {
        const int par = j & 1;
        if (SYNC == 1 && nranks > 1 && tid == 0)
            mbar_arrive_expect_tx(smem_u32(mbar + par), static_cast<uint32_t>(nslots * kMsgBytes));

        float best = -1.0f;
#pragma unroll
        for (int p = 0; p < PPT; ++p)
        {
            const float d = sumsq_abc(px[p] - cx, py[p] - cy, pz[p] - cz);
            md[p] = fminf(d, md[p]);
            best = fmaxf(best, md[p]);
        }
        // 64-bit key (hi, lo): hi orders by distance (0 = no candidate), lo by tie rank
        const uint32_t hi = best >= 0.0f ? __float_as_uint(best) + 1u : 0u;
        const uint32_t whi = __reduce_max_sync(kFullMask, hi);
        uint32_t lo = 0;
        int bp = 0;
        if (hi == whi && hi != 0u)
        {
#pragma unroll
            for (int p = PPT - 1; p >= 0; --p) bp = (md[p] == best) ? p : bp;
            lo = ~(rbase + static_cast<uint32_t>(bp) * rstep);
        }
        const uint32_t wlo = __reduce_max_sync(kFullMask, lo);
        const int src = __ffs(__ballot_sync(kFullMask, hi == whi && lo == wlo)) - 1;
        float wx = 0.f, wy = 0.f, wz = 0.f;
        if (lane == src)
        {
            const float* s = sxyz + (static_cast<size_t>(bp) * nthreads + tid) * 3;
            wx = s[0];
            wy = s[1];
            wz = s[2];
        }
        wx = __shfl_sync(kFullMask, wx, src);
        wy = __shfl_sync(kFullMask, wy, src);
        wz = __shfl_sync(kFullMask, wz, src);

        // lane r delivers this warp's message to CTA r of the cluster
        if (lane < nranks)
        {
            const uint32_t a_local = smem_u32(msg_a + par * nslots + my_slot);
            const uint32_t z_local = smem_u32(msg_z + par * nslots + my_slot);
            if (nranks == 1)
            {
                msg_a[par * nslots + my_slot] =
                    make_uint4(whi, wlo, __float_as_uint(wx), __float_as_uint(wy));
                msg_z[par * nslots + my_slot] = wz;
            }
            else if (SYNC == 0)
            {
                st_cluster_msg(mapa_cluster(a_local, lane), mapa_cluster(z_local, lane), whi, wlo,
                               wx, wy, wz);
            }
            else
            {
                st_async_msg(mapa_cluster(a_local, lane), mapa_cluster(z_local, lane),
                             mapa_cluster(smem_u32(mbar + par), lane), whi, wlo, wx, wy, wz);
            }
        }

        if (SYNC == 1 && nranks > 1)
        {
            const uint32_t parity = static_cast<uint32_t>((j - 1) >> 1) & 1u;
            const uint32_t bar = smem_u32(mbar + par);
            if (!mbar_wait_bounded(bar, parity))
            {
                if (lane == 0) atomicExch(&g_dev_status, 1);
                failed = true;
                break;
            }
        }
        else if (nranks > 1)
        {
            cluster_sync_all();
        }
        else
        {
            __syncthreads();
        }

        // every warp reduces all messages of the round to the same winner
        uint32_t bhi = 0, blo = 0;
        float bx = 0.f, by = 0.f, bz = 0.f;
        for (int s = lane; s < nslots; s += 32)
        {
            const uint4 a = msg_a[par * nslots + s];
            const float z = msg_z[par * nslots + s];
            if (a.x > bhi || (a.x == bhi && a.y > blo))
            {
                bhi = a.x;
                blo = a.y;
                bx = __uint_as_float(a.z);
                by = __uint_as_float(a.w);
                bz = z;
            }
        }
        const uint32_t ghi = __reduce_max_sync(kFullMask, bhi);
        const uint32_t glo = __reduce_max_sync(kFullMask, bhi == ghi ? blo : 0u);
        const int gsrc = __ffs(__ballot_sync(kFullMask, bhi == ghi && blo == glo)) - 1;
        cx = __shfl_sync(kFullMask, bx, gsrc);
        cy = __shfl_sync(kFullMask, by, gsrc);
        cz = __shfl_sync(kFullMask, bz, gsrc);
        if (gtid == 0)
        {
            int k = 0;
            if (ghi != 0u)
            {
                const uint32_t r = ~glo;
                k = static_cast<int>(((r & 0x3FFFFFu) << log2bs) | bitrev_low(r >> 22, log2bs));
            }
            idxs[j] = k;
        }
    }
    (void)failed;
    // no CTA may leave while a peer can still write into its shared memory
    if (nranks > 1) cluster_sync_all();
}

struct FpsConfig
{
    int nranks, nthreads, ppt, sync;
};

size_t fps_smem_bytes(const FpsConfig& c)
{
    const size_t nslots = static_cast<size_t>(c.nranks) * (c.nthreads / 32);
    size_t off = 2 * nslots * kMsgBytes;
    off += off & 8;
    off += 16;
    off += static_cast<size_t>(c.ppt) * c.nthreads * 3 * sizeof(float);
    return off;
}

int floor_log2(int v)
{
    int l = 0;
    while ((2 << l) <= v) ++l;
    return l;
}

int round_up_pow2(int v)
{
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

// Picks cluster size, block size and points per thread for n points per cloud.
bool fps_pick_config(int n, FpsConfig* out)
{
    FpsConfig c;
    c.sync = 1;
    if (n <= 4096)
        c.nranks = 1;
    else if (n <= 8192)
        c.nranks = 4;
    else if (n <= 65536)
        c.nranks = 8;
    else
        c.nranks = 16;
    c.nthreads = 512;
    const int per_thread = (n + c.nranks * c.nthreads - 1) / (c.nranks * c.nthreads);
    c.ppt = round_up_pow2(per_thread < 1 ? 1 : per_thread);
    if (c.ppt > kFpsMaxPpt) return false;
    // override for tuning runs: "nranks,nthreads,ppt,sync"
    if (const char* env = getenv("TPK_FPS_CONFIG"))
    {
        FpsConfig e = c;
        if (sscanf(env, "%d,%d,%d,%d", &e.nranks, &e.nthreads, &e.ppt, &e.sync) == 4)
        {
            const bool ok = (e.nranks == 1 || e.nranks == 2 || e.nranks == 4 || e.nranks == 8 ||
                             e.nranks == 16) &&
                            (e.nthreads == 128 || e.nthreads == 256 || e.nthreads == 512) &&
                            (e.ppt == 1 || e.ppt == 2 || e.ppt == 4 || e.ppt == 8 || e.ppt == 16) &&
                            (e.sync == 0 || e.sync == 1) &&
                            static_cast<long long>(e.nranks) * e.nthreads * e.ppt >= n &&
                            e.nranks * e.nthreads >= 512;
            if (ok) c = e;
        }
    }
    *out = c;
    return true;
}

template <int PPT, int SYNC>
int fps_launch_t(const FpsConfig& c, int b, int n, int m, int log2bs, const float* xyz,
                 int32_t* idxs, cudaStream_t stream)
{
    auto kernel = fps_onchip_kernel<PPT, SYNC>;
    const size_t smem = fps_smem_bytes(c);
    cudaError_t err;
    if (smem > 48 * 1024)
    {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("fps: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    if (c.nranks > 8)
    {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (err != cudaSuccess)
        {
            set_error("fps: cluster size attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(b) * c.nranks, 1, 1);
    cfg.blockDim = dim3(c.nthreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = c.nranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    err = cudaLaunchKernelEx(&cfg, kernel, n, m, log2bs, xyz, idxs);
    if (err != cudaSuccess)
    {
        set_error("fps launch (cluster %d x %d threads x %d points): %s", c.nranks, c.nthreads,
                  c.ppt, cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    return TPK_OK;
}

template <int SYNC>
int fps_launch_s(const FpsConfig& c, int b, int n, int m, int log2bs, const float* xyz,
                 int32_t* idxs, cudaStream_t stream)
{
    switch (c.ppt)
    {
    case 1: return fps_launch_t<1, SYNC>(c, b, n, m, log2bs, xyz, idxs, stream);
    case 2: return fps_launch_t<2, SYNC>(c, b, n, m, log2bs, xyz, idxs, stream);
    case 4: return fps_launch_t<4, SYNC>(c, b, n, m, log2bs, xyz, idxs, stream);
    case 8: return fps_launch_t<8, SYNC>(c, b, n, m, log2bs, xyz, idxs, stream);
    case 16: return fps_launch_t<16, SYNC>(c, b, n, m, log2bs, xyz, idxs, stream);
    default: break;
    }
    set_error("fps: unsupported points per thread %d", c.ppt);
    return TPK_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace tpk

extern "C" int64_t tpk_fps_scratch_bytes(int b, int n, int m)
{
    (void)b;
    (void)m;
    tpk::FpsConfig c;
    if (n <= 0 || tpk::fps_pick_config(n, &c)) return 0;
    return -1;  // larger clouds: not supported by this build
}

extern "C" int tpk_furthest_point_sampling(int b, int n, int m, const float* xyz, void* scratch,
                                           int32_t* idxs, void* stream)
{
    using namespace tpk;
    (void)scratch;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "fps: negative size (b=%d n=%d m=%d)", b, n, m);
    if (b == 0 || m == 0) return TPK_OK;
    TPK_REQUIRE(n > 0, "fps: cannot sample %d points from an empty cloud", m);
    TPK_REQUIRE(xyz != nullptr && idxs != nullptr, "fps: NULL pointer");
    FpsConfig c;
    if (!fps_pick_config(n, &c))
    {
        set_error("fps: n=%d exceeds the on-chip capacity of %d points per cloud", n,
                  kFpsMaxRanks * kFpsMaxThreads * kFpsMaxPpt);
        return TPK_ERR_UNSUPPORTED;
    }
    // block size of the reference launch (largest power of two <= n, capped at 512,
    // cuda/include/cuda_utils.h:16-21); it fixes the tie order
    int log2bs = floor_log2(n);
    if (log2bs > 9) log2bs = 9;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return c.sync ? fps_launch_s<1>(c, b, n, m, log2bs, xyz, idxs, s)
                  : fps_launch_s<0>(c, b, n, m, log2bs, xyz, idxs, s);
}

extern "C" int tpk_device_status(int* status_out, int reset)
{
    int v = 0;
    cudaError_t err = cudaMemcpyFromSymbol(&v, tpk::g_dev_status, sizeof(int));
    if (err == cudaSuccess && reset && v != 0)
    {
        const int zero = 0;
        err = cudaMemcpyToSymbol(tpk::g_dev_status, &zero, sizeof(int));
    }
    if (err != cudaSuccess)
    {
        tpk::set_error("device status: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    if (status_out) *status_out = v;
    return TPK_OK;
}
