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
#include <atomic>
#include <climits>
#include <math_constants.h>
#include <type_traits>

#include <cooperative_groups.h>

#include "tpk_common.cuh"

namespace cg = cooperative_groups;

namespace tpk
{
TPK_DEFINE_STATUS_WORD()

namespace
{

constexpr int kFpsMaxThreads = 512;
constexpr int kFpsMaxRanks = 16;
constexpr int kFpsMaxPpt = 32;
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

// Winner of one arg-max stage: key = bits of the running minimum (negative: no
// candidate), k = index of the point in its cloud, (x, y, z) = its coordinates.
struct Msg
{
    int key, k;
    float x, y, z;
};

constexpr int fps_max_threads(int ppt) { return ppt <= 16 ? 512 : 128; }

// Tie rank of point k: the reference's strided scan + tree keeps, among equal maxima,
// the smallest bit-reversed (k mod bs), then the smallest (k div bs).
__device__ __forceinline__ uint32_t fps_rank(int k, int log2bs)
{
    const uint32_t u = static_cast<uint32_t>(k);
    return (bitrev_low(u & ((1u << log2bs) - 1u), log2bs) << 22) | (u >> log2bs);
}

// Lane holding the largest key among the lanes of the warp.  One redux and one ballot
// when that key is unique (the usual case); ranks are only computed and reduced when
// two lanes carry exactly the same distance.
__device__ __forceinline__ int warp_argmax(int key, int k, int log2bs)
{
    const int wkey = __reduce_max_sync(kFullMask, key);
    uint32_t ball = __ballot_sync(kFullMask, key == wkey);
    if (__popc(ball) > 1 && wkey >= 0)
    {
        const uint32_t r = key == wkey ? fps_rank(k, log2bs) : 0xFFFFFFFFu;
        const uint32_t wr = __reduce_min_sync(kFullMask, r);
        ball = __ballot_sync(kFullMask, key == wkey && r == wr);
    }
    return __ffs(ball) - 1;
}

// One round = three arg-max stages, each a redux over at most 32 lanes:
//   1. inside every warp, over its lanes' best points;
//   2. inside the CTA, over its warps' winners (shared memory + one __syncthreads);
//   3. (CLUSTERED) inside the cluster, over its CTAs' winners: warp 0 delivers the CTA's
//      winner to every CTA of the cluster with st.async stores into distributed shared
//      memory that complete a transaction count on the receiver's mbarrier; every warp
//      then polls its own CTA's barrier (with a time limit) and reduces the messages.
// The round loop is unrolled by two so that the double-buffered message slots and
// barriers have compile-time addresses.  A CTA has at least two warps.
// packed pairs of floats for the two-wide FP32 instructions of sm_100
__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b)
{
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b)
{
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

//
// SORTED: the points come from a spatially sorted copy (x, y, z, original index) and a
// warp owns a contiguous run of it, i.e. a compact region of space.  A warp whose
// bounding box is farther from the newest sample than its largest running minimum
// cannot change any of its minima, so it skips the update and sends last round's winner
// again.  In the late rounds, which are most of them, a sample only reaches a few warps.
// The result does not depend on the order of the copy: ties are decided by the rank of
// the original index at every level.
template <int PPT, bool CLUSTERED, bool SORTED>
__global__ void __launch_bounds__(fps_max_threads(PPT), 1)
    fps_onchip_kernel(int n, int m, int log2bs, int flat, const float* __restrict__ xyz_all,
                      const float4* __restrict__ sorted_all, int32_t* __restrict__ idxs_all)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int nranks = CLUSTERED ? static_cast<int>(cluster_nctarank()) : 1;
    const int rank = CLUSTERED ? static_cast<int>(cluster_ctarank()) : 0;
    const int cloud = blockIdx.x / nranks;
    const int total = nranks * nthreads;
    const int gtid = rank * nthreads + tid;

    // shared memory: 2 x 32 warp messages, 2 x 32 CTA messages (16 B + 4 B each),
    // 2 mbarriers, then this CTA's coordinates as float4
    uint4* wmsg_a = reinterpret_cast<uint4*>(smem_raw);
    uint4* cmsg_a = wmsg_a + 64;
    float* wmsg_z = reinterpret_cast<float*>(cmsg_a + 64);
    float* cmsg_z = wmsg_z + 64;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(cmsg_z + 64);
    float4* sxyz = reinterpret_cast<float4*>(mbar + 2);

    const float* xyz = xyz_all + static_cast<size_t>(cloud) * n * 3;
    int32_t* idxs = idxs_all + static_cast<size_t>(cloud) * m;

    // Point p of this thread.  The layout makes "lowest p" the winner of the tie rule
    // among one thread's points: with at least bs threads in the cluster all of a
    // thread's points share (k mod bs) and ascend in (k div bs); with fewer, a thread
    // owns bs/total residues, visited in bit-reversed order, each with ascending k div bs.
    const int bs = 1 << log2bs;
    const bool wide = total >= bs;
    const int log2_per_residue = wide ? 0 : (31 - __clz(PPT)) + (31 - __clz(total)) - log2bs;
    const int residue_bits = wide ? 0 : log2bs - (31 - __clz(total));
    auto point_index = [&](int p) -> int {
        if (wide) return p * total + gtid;
        const int q = p >> log2_per_residue, i = p & ((1 << log2_per_residue) - 1);
        return (i << log2bs) + static_cast<int>(bitrev_low(static_cast<uint32_t>(q), residue_bits)) * total + gtid;
    };

    float px[PPT], py[PPT], pz[PPT], md[PPT];
    // bounding box of the warp's points (SORTED only)
    float bminx = CUDART_INF_F, bminy = CUDART_INF_F, bminz = CUDART_INF_F;
    float bmaxx = -CUDART_INF_F, bmaxy = -CUDART_INF_F, bmaxz = -CUDART_INF_F;
#pragma unroll
    for (int p = 0; p < PPT; ++p)
    {
        int k = point_index(p);
        float x = 0.f, y = 0.f, z = 0.f;
        bool valid = false;
        if (SORTED)
        {
            // slot of the sorted copy: warp-contiguous, lanes interleaved
            const int slot = ((rank * nwarps + warp) * PPT + p) * 32 + lane;
            k = n;
            if (slot < n)
            {
                const float4 v = __ldg(sorted_all + static_cast<size_t>(cloud) * n + slot);
                x = v.x;
                y = v.y;
                z = v.z;
                k = __float_as_int(v.w);
                const float mag = sumsq_abc(x, y, z);
                valid = !(static_cast<double>(mag) <= 1e-3);
                // fminf/fmaxf drop NaN: such a point never changes its minimum anyway
                bminx = fminf(bminx, x);
                bminy = fminf(bminy, y);
                bminz = fminf(bminz, z);
                bmaxx = fmaxf(bmaxx, x);
                bmaxy = fmaxf(bmaxy, y);
                bmaxz = fmaxf(bmaxz, z);
            }
        }
        else if (k < n)
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
        // w carries the point's index so that the winner's message needs no index arithmetic
        sxyz[p * nthreads + tid] = make_float4(x, y, z, __int_as_float(k));
    }

    if (SORTED)
    {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
        {
            bminx = fminf(bminx, __shfl_xor_sync(kFullMask, bminx, o));
            bminy = fminf(bminy, __shfl_xor_sync(kFullMask, bminy, o));
            bminz = fminf(bminz, __shfl_xor_sync(kFullMask, bminz, o));
            bmaxx = fmaxf(bmaxx, __shfl_xor_sync(kFullMask, bmaxx, o));
            bmaxy = fmaxf(bmaxy, __shfl_xor_sync(kFullMask, bmaxy, o));
            bmaxz = fmaxf(bmaxz, __shfl_xor_sync(kFullMask, bmaxz, o));
        }
    }
    // SORTED: the warp's winner of the last round it updated in, and the bound a sample's
    // squared distance to the box must exceed for the warp to skip (infinite: never skip)
    Msg wm = {INT_MIN, 0, 0.f, 0.f, 0.f};
    float skip_above = CUDART_INF_F;

    float cx = 0.f, cy = 0.f, cz = 0.f;
    if (n > 0)
    {
        cx = __ldg(xyz + 0);
        cy = __ldg(xyz + 1);
        cz = __ldg(xyz + 2);
    }
    if (gtid == 0 && m > 0) idxs[0] = 0;

    if (CLUSTERED)
    {
        if (tid == 0)
        {
            mbar_init(smem_u32(mbar + 0), 1);
            mbar_init(smem_u32(mbar + 1), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        cluster_sync_all();
    }
    else
    {
        __syncthreads();
    }

    // remote addresses of this CTA's slot in CTA `lane` of the cluster, both parities
    uint32_t rem_a[2] = {0, 0}, rem_z[2] = {0, 0}, rem_bar[2] = {0, 0};
    // flat exchange (flat != 0, at most 32 warps in the cluster): every warp sends its own
    // winner to all CTAs and stage 2 is skipped
    const int my_slot = flat ? rank * nwarps + warp : rank;
    const int nslots = flat ? nranks * nwarps : nranks;
    if (CLUSTERED && (warp == 0 || flat) && lane < nranks)
    {
#pragma unroll
        for (int par = 0; par < 2; ++par)
        {
            rem_a[par] = mapa_cluster(smem_u32(cmsg_a + par * 32 + my_slot), lane);
            rem_z[par] = mapa_cluster(smem_u32(cmsg_z + par * 32 + my_slot), lane);
            rem_bar[par] = mapa_cluster(smem_u32(mbar + par), lane);
        }
    }
    const float4* my_xyz = sxyz + tid;
    bool failed = false;

    auto round = [&](int j, auto par_tag) {
        constexpr int PAR = decltype(par_tag)::value;
        if (CLUSTERED && tid == 0)
            mbar_arrive_expect_tx(smem_u32(mbar + PAR), static_cast<uint32_t>(nslots * kMsgBytes));

        bool active = true;
        if (SORTED)
        {
            // squared distance from the sample to the warp's box; a computed distance is at
            // least this bound less a few ulp, far inside the margin taken here
            const float ex = fmaxf(fmaxf(bminx - cx, cx - bmaxx), 0.f);
            const float ey = fmaxf(fmaxf(bminy - cy, cy - bmaxy), 0.f);
            const float ez = fmaxf(fmaxf(bminz - cz, cz - bmaxz), 0.f);
            const float lb = __fmaf_rn(ez, ez, __fmaf_rn(ex, ex, __fmul_rn(ey, ey)));
            // the operands are the same in every lane; the vote makes the branch provably
            // uniform for the warp-wide instructions inside it
            active = __any_sync(kFullMask, !(__fmul_rn(lb, 0.9999f) > skip_above)) != 0;
        }
        Msg msg;
        if (active)
        {
        // ---- every point: distance to the newest sample, running minimum, thread maximum
        if constexpr (PPT >= 2)
        {
            // two points per packed instruction; x + (-c) rounds like x - c, and
            // mul, fma, fma is the operation order of sumsq_abc
            const unsigned long long ncx = pack2(-cx, -cx), ncy = pack2(-cy, -cy), ncz = pack2(-cz, -cz);
#pragma unroll
            for (int p = 0; p < PPT; p += 2)
            {
                const unsigned long long dx = add2(pack2(px[p], px[p + 1]), ncx);
                const unsigned long long dy = add2(pack2(py[p], py[p + 1]), ncy);
                const unsigned long long dz = add2(pack2(pz[p], pz[p + 1]), ncz);
                const unsigned long long d = fma2(dz, dz, fma2(dx, dx, mul2(dy, dy)));
                float d0, d1;
                unpack2(d, d0, d1);
                md[p] = fminf(d0, md[p]);
                md[p + 1] = fminf(d1, md[p + 1]);
            }
        }
        else
        {
#pragma unroll
            for (int p = 0; p < PPT; ++p)
                md[p] = fminf(sumsq_abc(px[p] - cx, py[p] - cy, pz[p] - cz), md[p]);
        }
        float red[PPT];
#pragma unroll
        for (int p = 0; p < PPT; ++p) red[p] = md[p];
#pragma unroll
        for (int w = PPT / 2; w >= 1; w >>= 1)
#pragma unroll
            for (int p = 0; p < w; ++p) red[p] = fmaxf(red[p], red[p + w]);
        const float best = red[0];

        // ---- stage 1: the warp's best point.  Non-negative floats order like their bits;
        // a negative key means "no candidate".  While the redux is in flight every lane
        // looks up its own best point (lowest p among equal minima), so that the winning
        // lane only has to store.
        const int key = __float_as_int(best);
        const int wkey = __reduce_max_sync(kFullMask, key);
        uint32_t eq = 0;
#pragma unroll
        for (int p = 0; p < PPT; ++p) eq |= (md[p] == best) ? (1u << p) : 0u;
        int bp = __ffs(eq) - 1;
        if (SORTED && key == wkey && wkey >= 0 && (eq & (eq - 1u)) != 0u)
        {
            // several of this lane's points tie: the original index decides (no layout rule
            // in a sorted copy).  Plain per-lane code, no warp-wide instruction.
            uint32_t best_rank = 0xFFFFFFFFu;
            for (uint32_t e = eq; e != 0u; e &= e - 1u)
            {
                const int p = __ffs(e) - 1;
                const uint32_t r = fps_rank(__float_as_int(my_xyz[p * nthreads].w), log2bs);
                if (r < best_rank)
                {
                    best_rank = r;
                    bp = p;
                }
            }
        }
        const float4 mine = my_xyz[bp * nthreads];
        uint32_t ball = __ballot_sync(kFullMask, key == wkey);
        if (__popc(ball) > 1 && wkey >= 0)
        {
            const uint32_t r = key == wkey ? fps_rank(__float_as_int(mine.w), log2bs) : 0xFFFFFFFFu;
            const uint32_t wr = __reduce_min_sync(kFullMask, r);
            ball = __ballot_sync(kFullMask, key == wkey && r == wr);
        }
        const int src1 = __ffs(ball) - 1;
        if (SORTED || (CLUSTERED && flat))
        {
            msg.key = wkey;
            msg.k = __shfl_sync(kFullMask, __float_as_int(mine.w), src1);
            msg.x = __shfl_sync(kFullMask, mine.x, src1);
            msg.y = __shfl_sync(kFullMask, mine.y, src1);
            msg.z = __shfl_sync(kFullMask, mine.z, src1);
            if (SORTED)
            {
                wm = msg;
                // no skipping on tiny bounds, where a computed distance may have lost precision
                skip_above = fmaxf(__int_as_float(wkey), 1.0e-30f);
            }
        }
        else if (lane == src1)
        {
            wmsg_a[PAR * 32 + warp] = make_uint4(static_cast<uint32_t>(key), __float_as_uint(mine.w),
                                                 __float_as_uint(mine.x), __float_as_uint(mine.y));
            wmsg_z[PAR * 32 + warp] = mine.z;
        }
        }  // active
        else
        {
            msg = wm;
        }
        if (SORTED && !(CLUSTERED && flat) && lane == 0)
        {
            wmsg_a[PAR * 32 + warp] = make_uint4(static_cast<uint32_t>(msg.key), static_cast<uint32_t>(msg.k),
                                                 __float_as_uint(msg.x), __float_as_uint(msg.y));
            wmsg_z[PAR * 32 + warp] = msg.z;
        }

        // ---- stage 2: the CTA's best point
        if (!(CLUSTERED && flat))
        {
            __syncthreads();
            int key2 = INT_MIN, k2 = 0;  // below every real key, including "no candidate"
            float x2 = 0.f, y2 = 0.f, z2 = 0.f;
            if (lane < nwarps)
            {
                const uint4 a = wmsg_a[PAR * 32 + lane];
                key2 = static_cast<int>(a.x);
                k2 = static_cast<int>(a.y);
                x2 = __uint_as_float(a.z);
                y2 = __uint_as_float(a.w);
                z2 = wmsg_z[PAR * 32 + lane];
            }
            const int src = warp_argmax(key2, k2, log2bs);
            msg.key = __shfl_sync(kFullMask, key2, src);
            msg.k = __shfl_sync(kFullMask, k2, src);
            msg.x = __shfl_sync(kFullMask, x2, src);
            msg.y = __shfl_sync(kFullMask, y2, src);
            msg.z = __shfl_sync(kFullMask, z2, src);
        }

        // ---- stage 3: the cluster's best point
        if (CLUSTERED)
        {
            if ((warp == 0 || flat) && lane < nranks)
                st_async_msg(rem_a[PAR], rem_z[PAR], rem_bar[PAR], static_cast<uint32_t>(msg.key),
                             static_cast<uint32_t>(msg.k), msg.x, msg.y, msg.z);
            // a warp whose wait ran out records it and stops waiting, but keeps taking part
            // in every barrier and exchange so that no other warp or CTA is left behind at
            // one; the results are then meaningless and the status word says so
            const uint32_t parity = static_cast<uint32_t>((j - 1) >> 1) & 1u;
            if (!failed && !mbar_wait_bounded(smem_u32(mbar + PAR), parity))
            {
                if (lane == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
                failed = true;
            }
            int key3 = INT_MIN, k3 = 0;
            if (lane < nslots)
            {
                const uint2 a = *reinterpret_cast<const uint2*>(cmsg_a + PAR * 32 + lane);
                key3 = static_cast<int>(a.x);
                k3 = static_cast<int>(a.y);
            }
            // every lane reads the winning slot itself (two broadcast loads instead of five
            // shuffles); the slot is not rewritten before all warps of the cluster have
            // sent their messages of the next round, i.e. after this read
            const int src = warp_argmax(key3, k3, log2bs);
            const uint4 win = cmsg_a[PAR * 32 + src];
            msg.key = static_cast<int>(win.x);
            msg.k = static_cast<int>(win.y);
            msg.x = __uint_as_float(win.z);
            msg.y = __uint_as_float(win.w);
            msg.z = cmsg_z[PAR * 32 + src];
        }

        cx = msg.x;
        cy = msg.y;
        cz = msg.z;
        if (gtid == 0) idxs[j] = msg.key >= 0 ? msg.k : 0;
    };

    int j = 1;
    for (; j + 1 < m; j += 2)
    {
        round(j, std::integral_constant<int, 1>{});
        round(j + 1, std::integral_constant<int, 0>{});
    }
    if (j < m) round(j, std::integral_constant<int, 1>{});

    // no CTA may leave while a peer can still write into its shared memory
    if (CLUSTERED) cluster_sync_all();
}

// ---------------------------------------------------------------- several samples per exchange
//
// The sorted kernel above pays one arg-max exchange per sample.  This kernel takes up to eight
// samples out of one exchange, exactly:
//
//   Every warp publishes its best point e1 = {key, index, x, y, z} and the KEY of its second
//   best point (key2).  Every warp then sorts the warps' best points (key, then tie rank of the
//   index) and accepts the longest prefix t0, t1, ... in which every t_i
//     (a) is untouched by the samples accepted before it: !(dist(t_i, t_j) < md(t_i)) for all
//         j < i, evaluated with the update's own arithmetic, so its running minimum - its key -
//         is what the sequential algorithm would see after applying t_0..t_{i-1};
//     (b) beats everything a warp that already gave a sample still holds: key(t_i) > key2 of
//         those warps (running minima only shrink, so key2 bounds the warp's leftovers);
//     (c) has a positive key (the list is sorted by key, then by the tie rank of the index, so
//         equal keys come in the reference's order);
//     (d) follows only samples with finite coordinates: a sample's own minimum must drop to
//         zero when it is applied, or the reference would pick it again (a warp publishes such
//         a point with the largest key2 there is, so test (b) covers it).
//   Points of warps that gave no sample are bounded by that warp's e1, which sorts after t_i.
//   So t_i is the largest running minimum that remains after t_0..t_{i-1} were applied: the
//   sample the reference picks next.  Cutting the prefix early is always allowed, which is
//   what makes the conservative tests (b) and (c) safe.
//
// Late in a run the largest running minima sit in different holes of the cloud, so almost
// every candidate passes: about five samples per exchange at 16384 points, with the update,
// the warp arg-max and the cluster exchange paid once for all of them.  Applying several
// samples is one pass over the warp's points with a minimum per sample in reach; the order
// of the minima does not matter.  With 16 or more points per lane a warp's points are four groups
// with a bounding box each, and a sample only updates the groups it can reach (under half the
// groups of the warps it reaches at all): 12 % faster at 32768 points per cloud and with 64
// clouds resident, no change at 16 clouds of 16384, where the update is not what the exchange
// waits for.  Requires the sorted copy and at most 32 warps per cloud.
constexpr int kFpsBatchMax = 8;       // samples per exchange
constexpr int kBatchMsgBytes = 24;    // {x, y, z, key2} + key + index

// One warp's entry into a peer's tables: coordinates and key2 (what the acceptance test reads
// with one load), the key into a compact table of its own (the ranking reads 32 keys with eight
// loads), and the point's index.
__device__ __forceinline__ void st_async_batch(uint32_t addr_c, uint32_t addr_key, uint32_t addr_k, uint32_t mbar,
                                               const uint4& c, uint32_t key, uint32_t k)
{
    asm volatile(
        "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::
            "r"(addr_c), "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w), "r"(mbar)
        : "memory");
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::
                     "r"(addr_key), "r"(key), "r"(mbar)
                 : "memory");
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::
                     "r"(addr_k), "r"(k), "r"(mbar)
                 : "memory");
}

template <int PPT, int MAXT, bool CLUSTERED>
__global__ void __launch_bounds__(MAXT, 1)
    fps_batched_kernel(int n, int m, int log2bs, const float* __restrict__ xyz_all,
                       const float4* __restrict__ sorted_all, int32_t* __restrict__ idxs_all)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int nranks = CLUSTERED ? static_cast<int>(cluster_nctarank()) : 1;
    const int rank = CLUSTERED ? static_cast<int>(cluster_ctarank()) : 0;
    const int cloud = blockIdx.x / nranks;
    const int gtid = rank * nthreads + tid;
    const int nslots = nranks * nwarps;  // at most 32: one slot per warp of the cluster
    const int my_slot = rank * nwarps + warp;

    // shared memory: slot tables of both parities (32 x {16, 4, 4} B each), 2 mbarriers, per warp
    // the sorted candidates of an exchange (8 x 24 B) and the warp's own entry, then the CTA's points
    uint4* tab_c = reinterpret_cast<uint4*>(smem_raw);        // [2][32] {x, y, z, key2}
    int* tab_key = reinterpret_cast<int*>(tab_c + 64);        // [2][32] key
    int* tab_k = tab_key + 64;                                // [2][32] index of the point
    uint64_t* mbar = reinterpret_cast<uint64_t*>(tab_k + 64);
    uint4* sort_c = reinterpret_cast<uint4*>(mbar + 2);       // [16 warps][8] {x, y, z, key2}
    uint2* sort_k = reinterpret_cast<uint2*>(sort_c + 16 * kFpsBatchMax);  // [16 warps][8] {key, index}
    uint4* own_c = reinterpret_cast<uint4*>(sort_k + 16 * kFpsBatchMax);   // [16 warps]
    uint2* own_k = reinterpret_cast<uint2*>(own_c + 16);                   // [16 warps] {key, index}
    float4* sxyz = reinterpret_cast<float4*>(own_k + 16);
    uint4* my_sort_c = sort_c + warp * kFpsBatchMax;
    uint2* my_sort_k = sort_k + warp * kFpsBatchMax;

    const float* xyz = xyz_all + static_cast<size_t>(cloud) * n * 3;
    int32_t* idxs = idxs_all + static_cast<size_t>(cloud) * m;

    float px[PPT], py[PPT], pz[PPT], md[PPT];
    // The warp's points in NG groups of GP * 32 consecutive points of the sorted copy (compact in
    // space), each with its bounding box: a sample only updates the groups it can reach.
    constexpr int NG = PPT >= 16 ? 4 : 1;  // measured: no gain below 16 points per lane
    constexpr int GP = PPT / NG;
    float gmin[NG][3], gmax[NG][3];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            gmin[g][a] = CUDART_INF_F;
            gmax[g][a] = -CUDART_INF_F;
        }
#pragma unroll
    for (int p = 0; p < PPT; ++p)
    {
        // slot of the sorted copy: warp-contiguous, lanes interleaved
        const int slot = ((rank * nwarps + warp) * PPT + p) * 32 + lane;
        float x = 0.f, y = 0.f, z = 0.f;
        int k = n;
        bool valid = false;
        if (slot < n)
        {
            const float4 v = __ldg(sorted_all + static_cast<size_t>(cloud) * n + slot);
            x = v.x;
            y = v.y;
            z = v.z;
            k = __float_as_int(v.w);
            const float mag = sumsq_abc(x, y, z);
            valid = !(static_cast<double>(mag) <= 1e-3);
            gmin[p / GP][0] = fminf(gmin[p / GP][0], x);
            gmin[p / GP][1] = fminf(gmin[p / GP][1], y);
            gmin[p / GP][2] = fminf(gmin[p / GP][2], z);
            gmax[p / GP][0] = fmaxf(gmax[p / GP][0], x);
            gmax[p / GP][1] = fmaxf(gmax[p / GP][1], y);
            gmax[p / GP][2] = fmaxf(gmax[p / GP][2], z);
        }
        px[p] = x;
        py[p] = y;
        pz[p] = z;
        md[p] = valid ? 1e10f : -1.0f;  // negative: never a candidate (fminf keeps it negative)
        sxyz[p * nthreads + tid] = make_float4(x, y, z, __int_as_float(k));
    }
    // lane l keeps the box of group l % NG: in the reach test below it answers for that group
    // and for sample l / NG of the list
    float bminx = CUDART_INF_F, bminy = CUDART_INF_F, bminz = CUDART_INF_F;
    float bmaxx = -CUDART_INF_F, bmaxy = -CUDART_INF_F, bmaxz = -CUDART_INF_F;
#pragma unroll
    for (int g = 0; g < NG; ++g)
    {
#pragma unroll
        for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1)
            {
                gmin[g][a] = fminf(gmin[g][a], __shfl_xor_sync(kFullMask, gmin[g][a], o));
                gmax[g][a] = fmaxf(gmax[g][a], __shfl_xor_sync(kFullMask, gmax[g][a], o));
            }
        if (lane % NG == g)
        {
            bminx = gmin[g][0];
            bminy = gmin[g][1];
            bminz = gmin[g][2];
            bmaxx = gmax[g][0];
            bmaxy = gmax[g][1];
            bmaxz = gmax[g][2];
        }
    }
    if (gtid == 0 && m > 0) idxs[0] = 0;
    // the list of samples to apply next (the same in every warp), in the warp's sort scratch:
    // at first the cloud's point 0
    if (lane == 0)
    {
        float cx = 0.f, cy = 0.f, cz = 0.f;
        if (n > 0)
        {
            cx = __ldg(xyz + 0);
            cy = __ldg(xyz + 1);
            cz = __ldg(xyz + 2);
        }
        my_sort_c[0] = make_uint4(__float_as_uint(cx), __float_as_uint(cy), __float_as_uint(cz), 0u);
        my_sort_k[0] = make_uint2(0u, 0u);
        own_c[warp] = make_uint4(0u, 0u, 0u, 0x80000000u);
        own_k[warp] = make_uint2(0x80000000u, 0u);
    }
    // slots no warp owns sort behind every real entry (key INT_MIN), in both tables
    if (tid < 64 && (tid & 31) >= nslots)
    {
        tab_c[tid] = make_uint4(0u, 0u, 0u, 0x80000000u);
        tab_key[tid] = static_cast<int>(0x80000000u);
        tab_k[tid] = 0;
    }
    if (CLUSTERED)
    {
        if (tid == 0)
        {
            mbar_init(smem_u32(mbar + 0), 1);
            mbar_init(smem_u32(mbar + 1), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        cluster_sync_all();
    }
    else
    {
        __syncthreads();
    }
    // remote addresses of this warp's slot in CTA `lane` of the cluster, parity 0; parity 1 lies
    // 32 entries (one barrier) further in the same shared window
    uint32_t rem_c = 0, rem_key = 0, rem_k = 0, rem_bar = 0;
    if (CLUSTERED && lane < nranks)
    {
        rem_c = mapa_cluster(smem_u32(tab_c + my_slot), lane);
        rem_key = mapa_cluster(smem_u32(tab_key + my_slot), lane);
        rem_k = mapa_cluster(smem_u32(tab_k + my_slot), lane);
        rem_bar = mapa_cluster(smem_u32(mbar), lane);
    }
    const float4* my_xyz = sxyz + tid;
    // the warp's entry of the last exchange it recomputed lives in own_c / own_k; infinite bound:
    // the first pass never skips
    float skip_above = CUDART_INF_F;
    bool failed = false;
    int nb = 1;   // samples to apply
    int j = 1;    // next output position

    for (int exch = 0; j < m; ++exch)
    {
        const int par = exch & 1;
        // (the CTA's last warp arms the barrier: in the middle CTA of a cluster warp 0 holds the
        // middle of the Morton order, the warp almost every sample reaches and every exchange waits for)
        if (CLUSTERED && tid == nthreads - 32)
            mbar_arrive_expect_tx(smem_u32(mbar + par), static_cast<uint32_t>(nslots * kBatchMsgBytes));

        // ---- 1. apply the samples to the groups of points they can reach
        // lane l tests sample l / NG against the box of group l % NG: one vote for all samples and
        // groups.  Every lane holds all candidates of the list (loads in flight together; entries
        // beyond nb are stale and unused).
        uint4 sc[kFpsBatchMax];
#pragma unroll
        for (int i = 0; i < kFpsBatchMax; ++i) sc[i] = my_sort_c[i];
        bool in_reach = false;
        {
            const int ts = lane / NG;
            const uint4 sl = my_sort_c[ts < kFpsBatchMax ? ts : 0];
            const float cx = __uint_as_float(sl.x), cy = __uint_as_float(sl.y), cz = __uint_as_float(sl.z);
            const float ex = fmaxf(fmaxf(bminx - cx, cx - bmaxx), 0.f);
            const float ey = fmaxf(fmaxf(bminy - cy, cy - bmaxy), 0.f);
            const float ez = fmaxf(fmaxf(bminz - cz, cz - bmaxz), 0.f);
            const float lb = __fmaf_rn(ez, ez, __fmaf_rn(ex, ex, __fmul_rn(ey, ey)));
            // out of reach: farther from the group's box than the largest running minimum of the
            // whole warp (a bound for the group's own)
            in_reach = ts < nb && !(__fmul_rn(lb, 0.9999f) > skip_above);
        }
        const uint32_t todo = __ballot_sync(kFullMask, in_reach);
        const bool touched = todo != 0u;
#pragma unroll
        for (int i = 0; i < kFpsBatchMax; ++i)
        {
            const uint32_t groups = (todo >> (i * NG)) & ((1u << NG) - 1u);  // warp-uniform
            if (groups != 0u)
            {
                const float cx = __uint_as_float(sc[i].x), cy = __uint_as_float(sc[i].y), cz = __uint_as_float(sc[i].z);
                if constexpr (PPT >= 2)
                {
                    const unsigned long long ncx = pack2(-cx, -cx), ncy = pack2(-cy, -cy), ncz = pack2(-cz, -cz);
#pragma unroll
                    for (int g = 0; g < NG; ++g)
                    {
                        if ((groups >> g) & 1u)
                        {
#pragma unroll
                            for (int p = g * GP; p < (g + 1) * GP; p += 2)
                            {
                                const unsigned long long dx = add2(pack2(px[p], px[p + 1]), ncx);
                                const unsigned long long dy = add2(pack2(py[p], py[p + 1]), ncy);
                                const unsigned long long dz = add2(pack2(pz[p], pz[p + 1]), ncz);
                                float d0, d1;
                                unpack2(fma2(dz, dz, fma2(dx, dx, mul2(dy, dy))), d0, d1);
                                md[p] = fminf(d0, md[p]);
                                md[p + 1] = fminf(d1, md[p + 1]);
                            }
                        }
                    }
                }
                else
                {
                    md[0] = fminf(sumsq_abc(px[0] - cx, py[0] - cy, pz[0] - cz), md[0]);
                }
            }
        }
        if (touched)
        {
            // ---- the warp's best point (ties: rank of the original index) and the key of its second best
            float red[PPT];
#pragma unroll
            for (int p = 0; p < PPT; ++p) red[p] = md[p];
#pragma unroll
            for (int w = PPT / 2; w >= 1; w >>= 1)
#pragma unroll
                for (int p = 0; p < w; ++p) red[p] = fmaxf(red[p], red[p + w]);
            const float best = red[0];
            const int key = __float_as_int(best);
            const int wkey = __reduce_max_sync(kFullMask, key);
            uint32_t eq = 0;
#pragma unroll
            for (int p = 0; p < PPT; ++p) eq |= (md[p] == best) ? (1u << p) : 0u;
            int bp = __ffs(eq) - 1;
            if (key == wkey && wkey >= 0 && (eq & (eq - 1u)) != 0u)
            {
                uint32_t best_rank = 0xFFFFFFFFu;
                for (uint32_t e = eq; e != 0u; e &= e - 1u)
                {
                    const int p = __ffs(e) - 1;
                    const uint32_t r = fps_rank(__float_as_int(my_xyz[p * nthreads].w), log2bs);
                    if (r < best_rank)
                    {
                        best_rank = r;
                        bp = p;
                    }
                }
            }
            if (bp < 0) bp = 0;
            const float4 mine = my_xyz[bp * nthreads];
            const bool mine_finite = sumsq_abc(mine.x - mine.x, mine.y - mine.y, mine.z - mine.z) == 0.f;
            // second best of the warp: a lane that holds the best counts the best of its other
            // points (the vote below does not wait for this reduction, nor it for the vote)
            float alt = -2.0f;
#pragma unroll
            for (int p = 0; p < PPT; ++p) alt = fmaxf(alt, p == bp ? -2.0f : md[p]);
            int key2 = __reduce_max_sync(kFullMask, __float_as_int(key == wkey ? alt : best));
            uint32_t ball = __ballot_sync(kFullMask, key == wkey);
            if (__popc(ball) > 1 && wkey >= 0)
            {
                key2 = wkey;  // another lane holds an equal minimum
                const uint32_t r = key == wkey ? fps_rank(__float_as_int(mine.w), log2bs) : 0xFFFFFFFFu;
                const uint32_t wr = __reduce_min_sync(kFullMask, r);
                ball = __ballot_sync(kFullMask, key == wkey && r == wr);
            }
            const int h1 = __ffs(ball) - 1;
            // the holder publishes through shared memory: every warp-wide instruction on this path
            // costs about a hundred cycles, a store and a load do not
            if (lane == h1)
            {
                // (d): a point with a non-finite coordinate does not drop to zero when it becomes a
                // sample (inf - inf and NaN leave its minimum where it is) and the reference then
                // picks it again; the largest key2 there is stops every later candidate
                if (!mine_finite) key2 = 0x7fffffff;
                own_c[warp] = make_uint4(__float_as_uint(mine.x), __float_as_uint(mine.y), __float_as_uint(mine.z),
                                         static_cast<uint32_t>(key2));
                own_k[warp] = make_uint2(static_cast<uint32_t>(wkey), __float_as_uint(mine.w));
            }
            __syncwarp();
            // no skipping on tiny bounds, where a computed distance may have lost precision
            skip_above = fmaxf(__int_as_float(wkey), 1.0e-30f);
        }
        // ---- 2. publish the warp's entry to every CTA of the cluster
        if (CLUSTERED)
        {
            if (lane < nranks)
            {
                const uint4 oc = own_c[warp];
                const uint2 ok2 = own_k[warp];
                st_async_batch(rem_c + par * 32 * 16, rem_key + par * 32 * 4, rem_k + par * 32 * 4, rem_bar + par * 8, oc,
                               ok2.x, ok2.y);
            }
            const uint32_t parity = static_cast<uint32_t>(exch >> 1) & 1u;
            if (!failed && !mbar_wait_bounded(smem_u32(mbar + par), parity))
            {
                if (lane == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
                failed = true;
            }
        }
        else
        {
            if (lane == 0)
            {
                const uint2 ok2 = own_k[warp];
                tab_c[par * 32 + my_slot] = own_c[warp];
                tab_key[par * 32 + my_slot] = static_cast<int>(ok2.x);
                tab_k[par * 32 + my_slot] = static_cast<int>(ok2.y);
            }
            __syncthreads();
        }
        // ---- 3. the samples this exchange yields (every warp computes the same list)
        // Position of every slot's entry in the exact order of the picks: key descending, then the
        // tie rank of the point's index, then the slot.  Every lane walks the 32 keys of the table
        // (broadcast loads, no warp-wide instruction; unowned slots hold INT_MIN).
        const uint4 ec = tab_c[par * 32 + lane];
        const int key_l = tab_key[par * 32 + lane];
        const int k_l = tab_k[par * 32 + lane];
        int4 kq[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) kq[q] = reinterpret_cast<const int4*>(tab_key + par * 32)[q];
        // integer arithmetic on the comparison results, no short-circuit operators: the compiler
        // turns those into a branch per step, which costs more than the step
        int pos = 0, same = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q)
        {
            const int ks[4] = {kq[q].x, kq[q].y, kq[q].z, kq[q].w};
#pragma unroll
            for (int c = 0; c < 4; ++c)
            {
                pos += ks[c] > key_l ? 1 : 0;
                same += ks[c] == key_l ? 1 : 0;
            }
        }
        const bool tie = same > 1;  // the lane's own slot is the one match; without ties pos is exact
        if (tie && key_l >= 0)  // rare: equal keys of real entries, the ranks of the indices decide
        {
            const uint32_t rl = fps_rank(k_l, log2bs);
            pos = 0;
            for (int s = 0; s < 32; ++s)
            {
                const int ks = tab_key[par * 32 + s];
                bool before = ks > key_l;
                if (ks == key_l && s != lane)
                {
                    const uint32_t rs = fps_rank(tab_k[par * 32 + s], log2bs);
                    before = rs < rl || (rs == rl && s < lane);
                }
                pos += before ? 1 : 0;
            }
        }
        __syncwarp();  // the list of the previous exchange has been read by every lane
        if (lane < nslots && pos < kFpsBatchMax)
        {
            my_sort_c[pos] = ec;
            my_sort_k[pos] = make_uint2(static_cast<uint32_t>(key_l), static_cast<uint32_t>(k_l));
        }
        __syncwarp();
        const int ncand = nslots < kFpsBatchMax ? nslots : kFpsBatchMax;
        // every lane runs the test (lanes without a candidate on entry 0): no branch, and the
        // loads do not wait for one another
        bool ok;
        {
            const int tl = lane < ncand ? lane : 0;
            const uint4 tc = my_sort_c[tl];
            const float tx = __uint_as_float(tc.x), ty = __uint_as_float(tc.y), tz = __uint_as_float(tc.z);
            const int tkey = static_cast<int>(my_sort_k[tl].x);
            const float tmd = __int_as_float(tkey);
            uint4 ss[kFpsBatchMax - 1];
#pragma unroll
            for (int s = 0; s < kFpsBatchMax - 1; ++s) ss[s] = my_sort_c[s < ncand ? s : 0];
            // (c) a positive key: at zero every remaining point coincides with a sample, samples of
            // this exchange included, and only the first pick of an exchange knows their order
            int okw = (tkey > 0 ? 1 : 0) & (lane < ncand ? 1 : 0);
#pragma unroll
            for (int s = 0; s < kFpsBatchMax - 1; ++s)
            {
                const float sx = __uint_as_float(ss[s].x), sy = __uint_as_float(ss[s].y), sz = __uint_as_float(ss[s].z);
                // (a) untouched by sample s, with the update's arithmetic (x + (-c) rounds like x - c)
                const float d = sumsq_abc(tx - sx, ty - sy, tz - sz);
                // (b) above whatever the warp that gave sample s still holds; (d) is folded into key2
                const int pass = (d < tmd ? 0 : 1) & (tkey > static_cast<int>(ss[s].w) ? 1 : 0);
                okw &= (s >= lane ? 1 : 0) | pass;
            }
            ok = okw != 0 || lane == 0;  // the first pick of an exchange is exact by construction
        }
        const uint32_t okmask = __ballot_sync(kFullMask, ok);
        nb = __ffs(~okmask) - 1;  // length of the accepted prefix (lane 0 always accepts)
        if (nb > m - j) nb = m - j;
        if (gtid == 0)
        {
            for (int i = 0; i < nb; ++i)
            {
                const uint2 sk = my_sort_k[i];
                idxs[j + i] = static_cast<int>(sk.x) >= 0 ? static_cast<int>(sk.y) : 0;
            }
        }
        j += nb;
    }
    // no CTA may leave while a peer can still write into its shared memory
    if (CLUSTERED) cluster_sync_all();
}

// ---------------------------------------------------------------- spatial sort
//
// Copy of every cloud in Morton order of a 2^bits-per-axis grid over its bounding box,
// as (x, y, z, original index): one CTA per cloud, counting sort with the cell counters
// in shared memory.  The order inside a cell is whatever the atomics give; the sampling
// kernel's result does not depend on it.
constexpr int kSortThreads = 1024;

__device__ __forceinline__ uint32_t spread3(uint32_t v)
{
    v = (v | (v << 16)) & 0x030000FFu;
    v = (v | (v << 8)) & 0x0300F00Fu;
    v = (v | (v << 4)) & 0x030C30C3u;
    v = (v | (v << 2)) & 0x09249249u;
    return v;
}

__global__ void __launch_bounds__(kSortThreads)
    fps_sort_kernel(int n, int bits, const float* __restrict__ xyz_all, float4* __restrict__ sorted_all)
{
    extern __shared__ int cnt[];  // 8^bits counters
    __shared__ float s_min[3][kSortThreads / 32], s_max[3][kSortThreads / 32];
    __shared__ int s_warp[kSortThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* xyz = xyz_all + static_cast<size_t>(blockIdx.x) * n * 3;
    float4* sorted = sorted_all + static_cast<size_t>(blockIdx.x) * n;
    const int ncell = 1 << (3 * bits);

    float mn[3] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};
    float mx[3] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
    for (int k = tid; k < n; k += kSortThreads)
    {
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            const float v = __ldg(xyz + 3 * static_cast<size_t>(k) + a);
            if (fabsf(v) < 1.0e18f)  // the box of the finite coordinates
            {
                mn[a] = fminf(mn[a], v);
                mx[a] = fmaxf(mx[a], v);
            }
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
        if (lane == 0)
        {
            s_min[a][warp] = mn[a];
            s_max[a][warp] = mx[a];
        }
    }
    for (int c = tid; c < ncell; c += kSortThreads) cnt[c] = 0;
    __syncthreads();
    float ext = 0.f;
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
        float lo = s_min[a][0], hi = s_max[a][0];
        for (int w = 1; w < kSortThreads / 32; ++w)
        {
            lo = fminf(lo, s_min[a][w]);
            hi = fmaxf(hi, s_max[a][w]);
        }
        mn[a] = lo;
        ext = fmaxf(ext, hi - lo);
    }
    const float qmax = static_cast<float>((1 << bits) - 1);
    const float inv_h = (ext > 0.f && ext < CUDART_INF_F) ? static_cast<float>(1 << bits) * 0.999999f / ext : 0.f;
    auto cell_of_point = [&](float x, float y, float z) -> int {
        // fmaxf drops NaN, the clamp takes care of infinities: any cell is a correct cell
        const uint32_t qx = static_cast<uint32_t>(fminf(fmaxf((x - mn[0]) * inv_h, 0.f), qmax));
        const uint32_t qy = static_cast<uint32_t>(fminf(fmaxf((y - mn[1]) * inv_h, 0.f), qmax));
        const uint32_t qz = static_cast<uint32_t>(fminf(fmaxf((z - mn[2]) * inv_h, 0.f), qmax));
        return static_cast<int>(spread3(qx) | (spread3(qy) << 1) | (spread3(qz) << 2));
    };

    for (int k = tid; k < n; k += kSortThreads)
    {
        const float x = __ldg(xyz + 3 * static_cast<size_t>(k) + 0);
        const float y = __ldg(xyz + 3 * static_cast<size_t>(k) + 1);
        const float z = __ldg(xyz + 3 * static_cast<size_t>(k) + 2);
        atomicAdd(&cnt[cell_of_point(x, y, z)], 1);
    }
    __syncthreads();

    // exclusive prefix sum of the counters: a run of cells per thread, then the runs' totals
    const int per = ncell >= kSortThreads ? ncell / kSortThreads : 1;
    const int c0 = tid * per;
    int sum = 0;
    if (c0 < ncell)
        for (int c = c0; c < c0 + per; ++c) sum += cnt[c];
    int incl = sum;
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
    int run = (warp ? s_warp[warp - 1] : 0) + incl - sum;
    if (c0 < ncell)
        for (int c = c0; c < c0 + per; ++c)
        {
            const int v = cnt[c];
            cnt[c] = run;
            run += v;
        }
    __syncthreads();

    for (int k = tid; k < n; k += kSortThreads)
    {
        const float x = __ldg(xyz + 3 * static_cast<size_t>(k) + 0);
        const float y = __ldg(xyz + 3 * static_cast<size_t>(k) + 1);
        const float z = __ldg(xyz + 3 * static_cast<size_t>(k) + 2);
        const int pos = atomicAdd(&cnt[cell_of_point(x, y, z)], 1);
        sorted[pos] = make_float4(x, y, z, __int_as_float(k));
    }
}

// about four points per cell, at most 32^3 cells (128 KB of counters)
int fps_sort_bits(int n)
{
    int bits = 1;
    while (bits < 5 && (1ll << (3 * bits)) * 4 < n) ++bits;
    return bits;
}

int fps_launch_sort(int b, int n, const float* xyz, float4* sorted, cudaStream_t stream)
{
    const int bits = fps_sort_bits(n);
    const size_t smem = sizeof(int) << (3 * bits);
    prefer_max_shared(fps_sort_kernel);
    if (smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(fps_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("fps sort: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    count_launches(1), fps_sort_kernel<<<b, kSortThreads, smem, stream>>>(n, bits, xyz, sorted);
    return check_launch("fps sort");
}

// ---------------------------------------------------------------- large clouds
//
// Clouds too large for the register-resident kernel: one 16-CTA cluster of 512-thread
// CTAs per cloud; the running minimum lives in caller-provided global scratch (n floats
// per cloud, the reference's `temp`), coordinates are re-read every round (they stay in
// L2 for the clouds a B200 runs at once).  Thread g of the cluster owns points
// g, g + 8192, g + 16384, ...: all share (k mod bs), so the first maximum a thread meets
// is also the one the tie rule prefers.  The per-round exchange is the same three-stage
// arg-max as in the on-chip kernel.
constexpr int kFpsBigRanks = 16;
constexpr int kFpsBigThreads = 512;

__global__ void __launch_bounds__(kFpsBigThreads, 1)
    fps_global_kernel(int n, int m, int log2bs, const float* __restrict__ xyz_all,
                      float* __restrict__ temp_all, int32_t* __restrict__ idxs_all)
{
    __shared__ __align__(16) uint4 wmsg_a[64];
    __shared__ __align__(16) uint4 cmsg_a[64];
    __shared__ float wmsg_z[64];
    __shared__ float cmsg_z[64];
    __shared__ __align__(8) uint64_t mbar[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nwarps = kFpsBigThreads / 32;
    const int nranks = static_cast<int>(cluster_nctarank());
    const int rank = static_cast<int>(cluster_ctarank());
    const int cloud = blockIdx.x / nranks;
    const int total = nranks * kFpsBigThreads;
    const int gtid = rank * kFpsBigThreads + tid;

    const float* xyz = xyz_all + static_cast<size_t>(cloud) * n * 3;
    float* temp = temp_all + static_cast<size_t>(cloud) * n;
    int32_t* idxs = idxs_all + static_cast<size_t>(cloud) * m;

    // running minimum: 1e10, or negative for points that are never candidates
    for (int k = gtid; k < n; k += total)
    {
        const float x = __ldg(xyz + 3 * static_cast<size_t>(k) + 0);
        const float y = __ldg(xyz + 3 * static_cast<size_t>(k) + 1);
        const float z = __ldg(xyz + 3 * static_cast<size_t>(k) + 2);
        const float mag = sumsq_abc(x, y, z);
        temp[k] = (static_cast<double>(mag) <= 1e-3) ? -1.0f : 1e10f;
    }

    float cx = __ldg(xyz + 0), cy = __ldg(xyz + 1), cz = __ldg(xyz + 2);
    if (gtid == 0 && m > 0) idxs[0] = 0;
    if (tid == 0)
    {
        mbar_init(smem_u32(mbar + 0), 1);
        mbar_init(smem_u32(mbar + 1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    cluster_sync_all();

    uint32_t rem_a[2] = {0, 0}, rem_z[2] = {0, 0}, rem_bar[2] = {0, 0};
    if (warp == 0 && lane < nranks)
    {
#pragma unroll
        for (int par = 0; par < 2; ++par)
        {
            rem_a[par] = mapa_cluster(smem_u32(cmsg_a + par * 32 + rank), lane);
            rem_z[par] = mapa_cluster(smem_u32(cmsg_z + par * 32 + rank), lane);
            rem_bar[par] = mapa_cluster(smem_u32(mbar + par), lane);
        }
    }
    bool failed = false;

    for (int j = 1; j < m; ++j)
    {
        const int par = j & 1;
        if (tid == 0)
            mbar_arrive_expect_tx(smem_u32(mbar + par), static_cast<uint32_t>(nranks * kMsgBytes));

        // ---- this thread's points: update the running minimum, keep the first maximum.
        // Eight points per step with all loads issued first; the minimum is only written
        // back when it changed (late rounds change few points).
        float best = -1.0f, bx = 0.f, by = 0.f, bz = 0.f;
        int bk = 0;
        constexpr int U = 8;
        for (int k0 = gtid; k0 < n; k0 += U * total)
        {
            float x[U], y[U], z[U], t[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
            {
                const int k = k0 + u * total;
                const bool ok = k < n;
                x[u] = ok ? __ldg(xyz + 3 * static_cast<size_t>(k) + 0) : 0.f;
                y[u] = ok ? __ldg(xyz + 3 * static_cast<size_t>(k) + 1) : 0.f;
                z[u] = ok ? __ldg(xyz + 3 * static_cast<size_t>(k) + 2) : 0.f;
                t[u] = ok ? temp[k] : -1.0f;
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
            {
                const int k = k0 + u * total;
                const float d = fminf(sumsq_abc(x[u] - cx, y[u] - cy, z[u] - cz), t[u]);
                if (d < t[u]) temp[k] = d;
                if (d > best)
                {
                    best = d;
                    bk = k;
                    bx = x[u];
                    by = y[u];
                    bz = z[u];
                }
            }
        }

        // ---- stage 1: warp
        int key = __float_as_int(best);
        int src = warp_argmax(key, bk, log2bs);
        if (lane == src)
        {
            wmsg_a[par * 32 + warp] = make_uint4(static_cast<uint32_t>(key), static_cast<uint32_t>(bk),
                                                 __float_as_uint(bx), __float_as_uint(by));
            wmsg_z[par * 32 + warp] = bz;
        }
        __syncthreads();

        // ---- stage 2: CTA
        Msg msg;
        {
            int key2 = INT_MIN, k2 = 0;
            float x2 = 0.f, y2 = 0.f, z2 = 0.f;
            if (lane < nwarps)
            {
                const uint4 a = wmsg_a[par * 32 + lane];
                key2 = static_cast<int>(a.x);
                k2 = static_cast<int>(a.y);
                x2 = __uint_as_float(a.z);
                y2 = __uint_as_float(a.w);
                z2 = wmsg_z[par * 32 + lane];
            }
            src = warp_argmax(key2, k2, log2bs);
            msg.key = __shfl_sync(kFullMask, key2, src);
            msg.k = __shfl_sync(kFullMask, k2, src);
            msg.x = __shfl_sync(kFullMask, x2, src);
            msg.y = __shfl_sync(kFullMask, y2, src);
            msg.z = __shfl_sync(kFullMask, z2, src);
        }

        // ---- stage 3: cluster
        if (nranks > 1)
        {
            if (warp == 0 && lane < nranks)
                st_async_msg(rem_a[par], rem_z[par], rem_bar[par], static_cast<uint32_t>(msg.key),
                             static_cast<uint32_t>(msg.k), msg.x, msg.y, msg.z);
            // a warp whose wait ran out records it and stops waiting but keeps taking part
            // in every barrier and exchange (see the on-chip kernel)
            const uint32_t parity = static_cast<uint32_t>((j - 1) >> 1) & 1u;
            if (!failed && !mbar_wait_bounded(smem_u32(mbar + par), parity))
            {
                if (lane == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
                failed = true;
            }
            int key3 = INT_MIN, k3 = 0;
            float x3 = 0.f, y3 = 0.f, z3 = 0.f;
            if (lane < nranks)
            {
                const uint4 a = cmsg_a[par * 32 + lane];
                key3 = static_cast<int>(a.x);
                k3 = static_cast<int>(a.y);
                x3 = __uint_as_float(a.z);
                y3 = __uint_as_float(a.w);
                z3 = cmsg_z[par * 32 + lane];
            }
            src = warp_argmax(key3, k3, log2bs);
            msg.key = __shfl_sync(kFullMask, key3, src);
            msg.k = __shfl_sync(kFullMask, k3, src);
            msg.x = __shfl_sync(kFullMask, x3, src);
            msg.y = __shfl_sync(kFullMask, y3, src);
            msg.z = __shfl_sync(kFullMask, z3, src);
        }
        else if (tid == 0)
        {
            // one-CTA cluster: nobody completes the transaction count, do it locally
            asm volatile("mbarrier.complete_tx.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(mbar + par)),
                         "r"(static_cast<uint32_t>(nranks * kMsgBytes))
                         : "memory");
        }
        cx = msg.x;
        cy = msg.y;
        cz = msg.z;
        if (gtid == 0) idxs[j] = msg.key >= 0 ? msg.k : 0;
    }
    cluster_sync_all();
}

// ---------------------------------------------------------------- large clouds, sorted
//
// The same clouds on a spatially sorted copy.  The copy is cut into chunks of 128
// consecutive points (a compact region each); lane c of a warp keeps, in registers, the
// bounding box of the warp's chunk c, the chunk's largest running minimum and the point
// that holds it.  A round tests every chunk's box against the new sample: a chunk farther
// away than its largest minimum cannot change and is skipped.  The few chunks in reach are
// updated by their whole warp (four points per lane: coordinates from the sorted copy,
// minima from scratch, written back only where they changed).  Late rounds touch a few
// kilobytes per cloud instead of the whole cloud.
constexpr int kFpsChunk = 128;  // points per chunk: 32 lanes x 4

template <int CPL>  // chunks per lane: a warp owns 32 * CPL chunks
__global__ void __launch_bounds__(kFpsBigThreads, 1)
    fps_pruned_kernel(int n, int m, int log2bs, const float* __restrict__ xyz_all,
                      const float4* __restrict__ sorted_all, float* __restrict__ temp_all,
                      int32_t* __restrict__ idxs_all)
{
    __shared__ __align__(16) uint4 wmsg_a[64];
    __shared__ __align__(16) uint4 cmsg_a[64];
    __shared__ float wmsg_z[64];
    __shared__ float cmsg_z[64];
    __shared__ __align__(8) uint64_t mbar[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nwarps = kFpsBigThreads / 32;
    const int nranks = static_cast<int>(cluster_nctarank());
    const int rank = static_cast<int>(cluster_ctarank());
    const int cloud = blockIdx.x / nranks;
    const int gtid = rank * kFpsBigThreads + tid;

    const float* xyz = xyz_all + static_cast<size_t>(cloud) * n * 3;
    const float4* sorted = sorted_all + static_cast<size_t>(cloud) * n;
    float* temp = temp_all + static_cast<size_t>(cloud) * n;
    int32_t* idxs = idxs_all + static_cast<size_t>(cloud) * m;

    // Chunk (slot s, lane c) of warp w is chunk (s * 32 + c) * total_warps + w of the cloud:
    // neighbouring chunks belong to different warps, so the handful of chunks a sample
    // reaches are updated side by side instead of one after the other.
    const long long gwarp = static_cast<long long>(rank) * nwarps + warp;
    const long long total_warps = static_cast<long long>(nranks) * nwarps;
    float bmin[CPL][3], bmax[CPL][3], cmax[CPL], bx[CPL], by[CPL], bz[CPL];
    int bk[CPL];
#pragma unroll
    for (int s = 0; s < CPL; ++s)
    {
        float kmin[3] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};
        float kmax[3] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
        cmax[s] = -1.0f;
        bk[s] = 0;
        bx[s] = by[s] = bz[s] = 0.f;
        for (int c = 0; c < 32; ++c)
        {
            const long long base = (static_cast<long long>(s * 32 + c) * total_warps + gwarp) * kFpsChunk;
            if (base >= n) break;  // warp-uniform
            float lo[3] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};
            float hi[3] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            bool any_valid = false;
#pragma unroll
            for (int u = 0; u < kFpsChunk / 32; ++u)
            {
                const long long p = base + u * 32 + lane;
                if (p < n)
                {
                    const float4 v = __ldg(sorted + p);
                    const float mag = sumsq_abc(v.x, v.y, v.z);
                    const bool valid = !(static_cast<double>(mag) <= 1e-3);
                    temp[p] = valid ? 1e10f : -1.0f;
                    any_valid |= valid;
                    // fminf/fmaxf drop NaN: such a point never changes its minimum anyway
                    lo[0] = fminf(lo[0], v.x);
                    lo[1] = fminf(lo[1], v.y);
                    lo[2] = fminf(lo[2], v.z);
                    hi[0] = fmaxf(hi[0], v.x);
                    hi[1] = fmaxf(hi[1], v.y);
                    hi[2] = fmaxf(hi[2], v.z);
                }
            }
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1)
                {
                    lo[a] = fminf(lo[a], __shfl_xor_sync(kFullMask, lo[a], o));
                    hi[a] = fmaxf(hi[a], __shfl_xor_sync(kFullMask, hi[a], o));
                }
            const bool chunk_valid = __any_sync(kFullMask, any_valid) != 0;
            if (lane == c)
            {
#pragma unroll
                for (int a = 0; a < 3; ++a)
                {
                    kmin[a] = lo[a];
                    kmax[a] = hi[a];
                }
                cmax[s] = chunk_valid ? 1e10f : -1.0f;  // every chunk with a candidate is updated in round 1
            }
        }
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            bmin[s][a] = kmin[a];
            bmax[s][a] = kmax[a];
        }
    }

    float cx = __ldg(xyz + 0), cy = __ldg(xyz + 1), cz = __ldg(xyz + 2);
    if (gtid == 0 && m > 0) idxs[0] = 0;
    if (tid == 0)
    {
        mbar_init(smem_u32(mbar + 0), 1);
        mbar_init(smem_u32(mbar + 1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    cluster_sync_all();

    uint32_t rem_a[2] = {0, 0}, rem_z[2] = {0, 0}, rem_bar[2] = {0, 0};
    if (warp == 0 && lane < nranks)
    {
#pragma unroll
        for (int par = 0; par < 2; ++par)
        {
            rem_a[par] = mapa_cluster(smem_u32(cmsg_a + par * 32 + rank), lane);
            rem_z[par] = mapa_cluster(smem_u32(cmsg_z + par * 32 + rank), lane);
            rem_bar[par] = mapa_cluster(smem_u32(mbar + par), lane);
        }
    }
    bool failed = false;
    Msg wm = {INT_MIN, 0, 0.f, 0.f, 0.f};  // the warp's winner, recomputed when a chunk of it changed

    for (int j = 1; j < m; ++j)
    {
        const int par = j & 1;
        if (tid == 0)
            mbar_arrive_expect_tx(smem_u32(mbar + par), static_cast<uint32_t>(nranks * kMsgBytes));

        // ---- chunks in reach of the new sample
        bool touched = false;
#pragma unroll
        for (int s = 0; s < CPL; ++s)
        {
            const float ex = fmaxf(fmaxf(bmin[s][0] - cx, cx - bmax[s][0]), 0.f);
            const float ey = fmaxf(fmaxf(bmin[s][1] - cy, cy - bmax[s][1]), 0.f);
            const float ez = fmaxf(fmaxf(bmin[s][2] - cz, cz - bmax[s][2]), 0.f);
            const float lb = __fmaf_rn(ez, ez, __fmaf_rn(ex, ex, __fmul_rn(ey, ey)));
            // a computed distance is at least this bound less a few ulp; no skipping on tiny
            // bounds, where it may have lost precision.  A chunk without candidates
            // (largest minimum -1) is skipped whenever the bound is positive or its box is empty.
            const bool in_reach = !(__fmul_rn(lb, 0.9999f) > fmaxf(cmax[s], 1.0e-30f));
            uint32_t todo = __ballot_sync(kFullMask, in_reach);
            touched |= todo != 0u;
            while (todo != 0u)  // warp-uniform
            {
                const int c = __ffs(todo) - 1;
                todo &= todo - 1u;
                const long long base = (static_cast<long long>(s * 32 + c) * total_warps + gwarp) * kFpsChunk;
                float4 v[kFpsChunk / 32];
                float t[kFpsChunk / 32];
#pragma unroll
                for (int u = 0; u < kFpsChunk / 32; ++u)
                {
                    const long long p = base + u * 32 + lane;
                    const bool ok = p < n;
                    v[u] = ok ? __ldg(sorted + p) : make_float4(0.f, 0.f, 0.f, 0.f);
                    t[u] = ok ? temp[p] : -1.0f;
                }
                float best = -1.0f, mx = 0.f, my = 0.f, mz = 0.f;
                int mk = 0;
                uint32_t mrank = 0xFFFFFFFFu;
#pragma unroll
                for (int u = 0; u < kFpsChunk / 32; ++u)
                {
                    const float d = fminf(sumsq_abc(v[u].x - cx, v[u].y - cy, v[u].z - cz), t[u]);
                    if (d < t[u]) temp[base + u * 32 + lane] = d;
                    // among equal minima the original index decides (tie rank)
                    const int k = __float_as_int(v[u].w);
                    bool better = d > best;
                    if (d == best && d >= 0.f)
                    {
                        if (mrank == 0xFFFFFFFFu) mrank = fps_rank(mk, log2bs);
                        better = fps_rank(k, log2bs) < mrank;
                    }
                    if (better)
                    {
                        best = d;
                        mk = k;
                        mx = v[u].x;
                        my = v[u].y;
                        mz = v[u].z;
                        mrank = 0xFFFFFFFFu;
                    }
                }
                const int key = __float_as_int(best);
                const int src = warp_argmax(key, mk, log2bs);
                const int wkey = __shfl_sync(kFullMask, key, src);
                const int wk = __shfl_sync(kFullMask, mk, src);
                const float wx = __shfl_sync(kFullMask, mx, src);
                const float wy = __shfl_sync(kFullMask, my, src);
                const float wz = __shfl_sync(kFullMask, mz, src);
                if (lane == c)
                {
                    cmax[s] = __int_as_float(wkey);
                    bk[s] = wk;
                    bx[s] = wx;
                    by[s] = wy;
                    bz[s] = wz;
                }
            }
        }

        // ---- stage 1: the warp's winner over its chunks (unchanged if no chunk was touched)
        if (touched)  // warp-uniform
        {
            float best = cmax[0], x1 = bx[0], y1 = by[0], z1 = bz[0];
            int k1 = bk[0];
#pragma unroll
            for (int s = 1; s < CPL; ++s)
            {
                bool better = cmax[s] > best;
                if (cmax[s] == best && best >= 0.f) better = fps_rank(bk[s], log2bs) < fps_rank(k1, log2bs);
                if (better)
                {
                    best = cmax[s];
                    k1 = bk[s];
                    x1 = bx[s];
                    y1 = by[s];
                    z1 = bz[s];
                }
            }
            const int key = __float_as_int(best);
            const int src = warp_argmax(key, k1, log2bs);
            wm.key = __shfl_sync(kFullMask, key, src);
            wm.k = __shfl_sync(kFullMask, k1, src);
            wm.x = __shfl_sync(kFullMask, x1, src);
            wm.y = __shfl_sync(kFullMask, y1, src);
            wm.z = __shfl_sync(kFullMask, z1, src);
        }
        if (lane == 0)
        {
            wmsg_a[par * 32 + warp] = make_uint4(static_cast<uint32_t>(wm.key), static_cast<uint32_t>(wm.k),
                                                 __float_as_uint(wm.x), __float_as_uint(wm.y));
            wmsg_z[par * 32 + warp] = wm.z;
        }
        __syncthreads();

        // ---- stage 2: CTA
        Msg msg;
        {
            int key2 = INT_MIN, k2 = 0;
            float x2 = 0.f, y2 = 0.f, z2 = 0.f;
            if (lane < nwarps)
            {
                const uint4 a = wmsg_a[par * 32 + lane];
                key2 = static_cast<int>(a.x);
                k2 = static_cast<int>(a.y);
                x2 = __uint_as_float(a.z);
                y2 = __uint_as_float(a.w);
                z2 = wmsg_z[par * 32 + lane];
            }
            const int src = warp_argmax(key2, k2, log2bs);
            msg.key = __shfl_sync(kFullMask, key2, src);
            msg.k = __shfl_sync(kFullMask, k2, src);
            msg.x = __shfl_sync(kFullMask, x2, src);
            msg.y = __shfl_sync(kFullMask, y2, src);
            msg.z = __shfl_sync(kFullMask, z2, src);
        }

        // ---- stage 3: cluster
        if (nranks > 1)
        {
            if (warp == 0 && lane < nranks)
                st_async_msg(rem_a[par], rem_z[par], rem_bar[par], static_cast<uint32_t>(msg.key),
                             static_cast<uint32_t>(msg.k), msg.x, msg.y, msg.z);
            // a warp whose wait ran out records it and stops waiting but keeps taking part
            // in every barrier and exchange (see the on-chip kernel)
            const uint32_t parity = static_cast<uint32_t>((j - 1) >> 1) & 1u;
            if (!failed && !mbar_wait_bounded(smem_u32(mbar + par), parity))
            {
                if (lane == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
                failed = true;
            }
            int key3 = INT_MIN, k3 = 0;
            if (lane < nranks)
            {
                const uint2 a = *reinterpret_cast<const uint2*>(cmsg_a + par * 32 + lane);
                key3 = static_cast<int>(a.x);
                k3 = static_cast<int>(a.y);
            }
            const int src = warp_argmax(key3, k3, log2bs);
            const uint4 win = cmsg_a[par * 32 + src];
            msg.key = static_cast<int>(win.x);
            msg.k = static_cast<int>(win.y);
            msg.x = __uint_as_float(win.z);
            msg.y = __uint_as_float(win.w);
            msg.z = cmsg_z[par * 32 + src];
        }
        else if (tid == 0)
        {
            // one-CTA cluster: nobody completes the transaction count, do it locally
            asm volatile("mbarrier.complete_tx.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(mbar + par)),
                         "r"(static_cast<uint32_t>(nranks * kMsgBytes))
                         : "memory");
        }
        cx = msg.x;
        cy = msg.y;
        cz = msg.z;
        if (gtid == 0) idxs[j] = msg.key >= 0 ? msg.k : 0;
    }
    cluster_sync_all();
}

int fps_launch_global(int b, int n, int m, int log2bs, const float* xyz, float* temp,
                      int32_t* idxs, cudaStream_t stream)
{
    auto kernel = fps_global_kernel;
    prefer_max_shared(kernel);
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err != cudaSuccess)
    {
        set_error("fps: cluster size attribute: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(b) * kFpsBigRanks, 1, 1);
    cfg.blockDim = dim3(kFpsBigThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kFpsBigRanks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launches(1);
    err = cudaLaunchKernelEx(&cfg, kernel, n, m, log2bs, xyz, temp, idxs);
    if (err != cudaSuccess)
    {
        set_error("fps launch (large clouds): %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    return TPK_OK;
}

// Largest cloud the sorted large-cloud kernel takes: 256 warps x 32 lanes x 4 chunks x 128 points.
constexpr long long kFpsPrunedMaxPoints = 256ll * 32 * 4 * kFpsChunk;

template <int CPL>
int fps_launch_pruned_t(int b, int n, int m, int log2bs, const float* xyz, const float4* sorted, float* temp,
                        int32_t* idxs, cudaStream_t stream)
{
    auto kernel = fps_pruned_kernel<CPL>;
    prefer_max_shared(kernel);
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err != cudaSuccess)
    {
        set_error("fps: cluster size attribute: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(b) * kFpsBigRanks, 1, 1);
    cfg.blockDim = dim3(kFpsBigThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kFpsBigRanks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launches(1);
    err = cudaLaunchKernelEx(&cfg, kernel, n, m, log2bs, xyz, sorted, temp, idxs);
    if (err != cudaSuccess)
    {
        set_error("fps launch (large clouds, sorted): %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    return TPK_OK;
}

// scratch: the sorted copy (16 bytes per point), then the running minima (4 bytes per point)
int fps_launch_pruned(int b, int n, int m, int log2bs, const float* xyz, void* scratch, int32_t* idxs,
                      cudaStream_t stream)
{
    float4* sorted = static_cast<float4*>(scratch);
    float* temp = reinterpret_cast<float*>(sorted + static_cast<size_t>(b) * n);
    const int rc = fps_launch_sort(b, n, xyz, sorted, stream);
    if (rc != TPK_OK) return rc;
    const long long per_lane = (static_cast<long long>(n) + 256ll * 32 * kFpsChunk - 1) / (256ll * 32 * kFpsChunk);
    if (per_lane <= 1) return fps_launch_pruned_t<1>(b, n, m, log2bs, xyz, sorted, temp, idxs, stream);
    if (per_lane <= 2) return fps_launch_pruned_t<2>(b, n, m, log2bs, xyz, sorted, temp, idxs, stream);
    return fps_launch_pruned_t<4>(b, n, m, log2bs, xyz, sorted, temp, idxs, stream);
}

struct FpsConfig
{
    int nranks, nthreads, ppt;
};

size_t fps_smem_bytes(const FpsConfig& c)
{
    // 128 x 16 B + 128 x 4 B messages, 2 mbarriers, coordinates
    return 128 * 16 + 128 * 4 + 16 + static_cast<size_t>(c.ppt) * c.nthreads * 4 * sizeof(float);
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

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

bool fps_config_ok(const FpsConfig& e, int n)
{
    return (e.nranks >= 1 && e.nranks <= kFpsMaxRanks && is_pow2(e.nranks)) &&
           (e.nthreads >= 64 && e.nthreads <= kFpsMaxThreads && is_pow2(e.nthreads)) &&
           (e.ppt >= 1 && e.ppt <= kFpsMaxPpt && is_pow2(e.ppt)) && e.nthreads <= fps_max_threads(e.ppt) &&
           static_cast<long long>(e.nranks) * e.nthreads * e.ppt >= n;
}

// Picks cluster size, block size and points per thread for n points per cloud: few,
// fat threads (every warp and every CTA adds a stage to the per-round exchange), and
// as many CTAs per cloud as keep a CTA's share near 2048-4096 points.
bool fps_pick_config(int n, int m, FpsConfig* out)
{
    FpsConfig c;
    (void)m;
    c.nranks = n <= 4096 ? 1 : (n <= 8192 ? 4 : (n <= 32768 ? 8 : 16));
    const int per_cta = (n + c.nranks - 1) / c.nranks;
    if (per_cta <= 256)
        c.nthreads = 64;
    else if (per_cta <= 2048)
        c.nthreads = 128;
    else if (per_cta <= 4096)
        c.nthreads = c.nranks == 1 ? 256 : 128;
    else
        c.nthreads = 512;
    c.ppt = round_up_pow2((per_cta + c.nthreads - 1) / c.nthreads);
    if (c.ppt < 1) c.ppt = 1;
    if (!fps_config_ok(c, n)) return false;
    // test hook "fps_config=nranks:nthreads:ppt": another cluster shape on the same cloud
    char text[64];
    if (test_value("fps_config", text, sizeof(text)))
    {
        FpsConfig e = c;
        if (sscanf(text, "%d:%d:%d", &e.nranks, &e.nthreads, &e.ppt) == 3 && fps_config_ok(e, n)) c = e;
    }
    *out = c;
    return true;
}

template <int PPT, bool CLUSTERED, bool SORTED>
int fps_launch_t(const FpsConfig& c, int b, int n, int m, int log2bs, const float* xyz,
                 const float4* sorted, int32_t* idxs, cudaStream_t stream)
{
    auto kernel = fps_onchip_kernel<PPT, CLUSTERED, SORTED>;
    prefer_max_shared(kernel);
    const size_t smem = fps_smem_bytes(c);
    cudaError_t err;
    if (smem > kDynSmemOptIn)
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
    // flat exchange whenever the cluster has at most 32 warps (measured 5-8 % faster per round);
    // test hook "fps_tree" selects the three-stage exchange
    const int flat = (c.nranks > 1 && c.nranks * (c.nthreads / 32) <= 32 && !test_path("fps_tree")) ? 1 : 0;
    count_launches(1);
    err = cudaLaunchKernelEx(&cfg, kernel, n, m, log2bs, flat, xyz, sorted, idxs);
    if (err != cudaSuccess)
    {
        set_error("fps launch (cluster %d x %d threads x %d points): %s", c.nranks, c.nthreads,
                  c.ppt, cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    return TPK_OK;
}

size_t fps_batched_smem_bytes(const FpsConfig& c)
{
    // slot tables (2 x 32 x 24 B), 2 mbarriers, per-warp sort scratch (16 x 8 x 24 B) and own entry
    // (16 x 24 B), coordinates
    return 2 * 32 * 24 + 16 + 16 * kFpsBatchMax * 24 + 16 * 24 + static_cast<size_t>(c.ppt) * c.nthreads * 4 * sizeof(float);
}

template <int PPT, int MAXT, bool CLUSTERED>
int fps_launch_batched_t(const FpsConfig& c, int b, int n, int m, int log2bs, const float* xyz, const float4* sorted,
                         int32_t* idxs, cudaStream_t stream)
{
    auto kernel = fps_batched_kernel<PPT, MAXT, CLUSTERED>;
    prefer_max_shared(kernel);
    const size_t smem = fps_batched_smem_bytes(c);
    cudaError_t err;
    if (smem > kDynSmemOptIn)
    {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
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
    count_launches(1);
    err = cudaLaunchKernelEx(&cfg, kernel, n, m, log2bs, xyz, sorted, idxs);
    if (err != cudaSuccess)
    {
        set_error("fps launch (several samples per exchange, cluster %d x %d threads x %d points): %s", c.nranks,
                  c.nthreads, c.ppt, cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    return TPK_OK;
}

template <bool CLUSTERED>
int fps_launch_batched(const FpsConfig& c, int b, int n, int m, int log2bs, const float* xyz, const float4* sorted,
                       int32_t* idxs, cudaStream_t stream)
{
    // Blocks of four warps get their own build: with 512 threads as the bound the compiler has
    // 128 registers, too few to keep the loads of a merge in flight together.  The lean build
    // stays for batches whose CTAs only fit the GPU at once with it (measured on 64 clouds).
    const bool roomy = c.nthreads <= 128 && static_cast<long long>(b) * c.nranks <= 2ll * num_sms();
#define TPK_FPS_BATCHED_CASE(P)                                                                                      \
    case P:                                                                                                          \
        return roomy                                                                                                 \
                   ? fps_launch_batched_t<P, 128, CLUSTERED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream)          \
                   : fps_launch_batched_t<P, fps_max_threads(P), CLUSTERED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream)
    switch (c.ppt)
    {
        TPK_FPS_BATCHED_CASE(1);
        TPK_FPS_BATCHED_CASE(2);
        TPK_FPS_BATCHED_CASE(4);
        TPK_FPS_BATCHED_CASE(8);
        TPK_FPS_BATCHED_CASE(16);
        TPK_FPS_BATCHED_CASE(32);
    default: break;
    }
#undef TPK_FPS_BATCHED_CASE
    set_error("fps: unsupported points per thread %d", c.ppt);
    return TPK_ERR_UNSUPPORTED;
}

// The kernel with several samples per exchange takes clusters of at most 32 warps (one slot per
// warp) and 16 warps per CTA; test hook "fps_single" keeps the one-sample-per-exchange kernel.
bool fps_wants_batched(const FpsConfig& c)
{
    return c.nranks * (c.nthreads / 32) <= 32 && c.nthreads / 32 <= 16 && !test_path("fps_single");
}

// Cluster shape for that kernel: eight CTAs of four warps fill the 32 slots with the fewest
// warps per SM (measured best from 4096 to 32768 points per cloud, for 16 and for 64 clouds).
// Larger clouds keep the shape fps_pick_config chose, and with it the one-sample kernel.
void fps_batched_config(int n, FpsConfig* c)
{
    char text[8];
    if (test_value("fps_config", text, sizeof(text)) || test_path("fps_single")) return;
    FpsConfig e;
    e.nranks = 8;
    e.nthreads = 128;
    e.ppt = round_up_pow2((n + 1023) / 1024);
    if (fps_config_ok(e, n)) *c = e;
}

template <bool CLUSTERED, bool SORTED>
int fps_launch_s(const FpsConfig& c, int b, int n, int m, int log2bs, const float* xyz,
                 const float4* sorted, int32_t* idxs, cudaStream_t stream)
{
    switch (c.ppt)
    {
    case 1: return fps_launch_t<1, CLUSTERED, SORTED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream);
    case 2: return fps_launch_t<2, CLUSTERED, SORTED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream);
    case 4: return fps_launch_t<4, CLUSTERED, SORTED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream);
    case 8: return fps_launch_t<8, CLUSTERED, SORTED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream);
    case 16: return fps_launch_t<16, CLUSTERED, SORTED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream);
    case 32: return fps_launch_t<32, CLUSTERED, SORTED>(c, b, n, m, log2bs, xyz, sorted, idxs, stream);
    default: break;
    }
    set_error("fps: unsupported points per thread %d", c.ppt);
    return TPK_ERR_UNSUPPORTED;
}

// Which kernel family a call takes.  The sorted copy pays when a cloud has enough chunks for
// most of them to be skipped and enough rounds to earn back the sort.  Test hooks:
// "fps_global" (large-cloud kernels on any cloud), "fps_unsorted" (no sorted copy anywhere),
// "fps_sorted" (sorted copy whatever the size).
enum FpsPath
{
    kFpsOnchip,        // cluster per cloud, registers, no scratch
    kFpsOnchipSorted,  // cluster per cloud on the sorted copy (16 B/point)
    kFpsPruned,        // large clouds on the sorted copy (20 B/point)
    kFpsGlobal         // large clouds, unsorted (4 B/point)
};

FpsPath fps_pick_path(int n, int m, FpsConfig* c)
{
    if (test_path("fps_global") || !fps_pick_config(n, m, c))
        return (static_cast<long long>(n) <= kFpsPrunedMaxPoints && !test_path("fps_unsorted")) ? kFpsPruned
                                                                                                  : kFpsGlobal;
    if (test_path("fps_unsorted")) return kFpsOnchip;
    const bool worth = test_path("fps_sorted") || (n >= 4096 && m >= 128);
    return worth ? kFpsOnchipSorted : kFpsOnchip;
}

}  // namespace
}  // namespace tpk

extern "C" int64_t tpk_fps_scratch_bytes(int b, int n, int m)
{
    tpk::FpsConfig c;
    if (n <= 0 || b <= 0 || m <= 0) return 0;
    switch (tpk::fps_pick_path(n, m, &c))
    {
    case tpk::kFpsOnchip: return 0;
    // optional: the spatially sorted copy, (x, y, z, index) per point
    case tpk::kFpsOnchipSorted: return static_cast<int64_t>(b) * n * 16;
    // large clouds: the running minimum, one float per point, behind the sorted copy if one is used
    case tpk::kFpsPruned: return static_cast<int64_t>(b) * n * 20;
    default: return static_cast<int64_t>(b) * n * 4;
    }
}

extern "C" int tpk_furthest_point_sampling(int b, int n, int m, const float* xyz, void* scratch,
                                           int64_t scratch_bytes, int32_t* idxs, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "fps: negative size (b=%d n=%d m=%d)", b, n, m);
    if (b == 0 || m == 0) return TPK_OK;
    TPK_REQUIRE(n > 0, "fps: cannot sample %d points from an empty cloud", m);
    TPK_REQUIRE(xyz != nullptr && idxs != nullptr, "fps: NULL pointer");
    // block size of the reference launch (largest power of two <= n, capped at 512,
    // cuda/include/cuda_utils.h:16-21); it fixes the tie order
    int log2bs = floor_log2(n);
    if (log2bs > 9) log2bs = 9;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // a scratch buffer is either absent or large enough for the kernel that will use it
    const int64_t want = tpk_fps_scratch_bytes(b, n, m);
    if (scratch != nullptr && scratch_bytes < want)
    {
        set_error("fps: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch_bytes),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    FpsConfig c;
    const FpsPath path = fps_pick_path(n, m, &c);
    if (path == kFpsPruned || path == kFpsGlobal)
    {
        if (scratch == nullptr)
        {
            set_error("fps: clouds of %d points need tpk_fps_scratch_bytes() bytes of scratch", n);
            return TPK_ERR_SCRATCH;
        }
        if (path == kFpsPruned)
        {
            TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "fps: scratch must be 16-byte aligned");
            return fps_launch_pruned(b, n, m, log2bs, xyz, scratch, idxs, s);
        }
        return fps_launch_global(b, n, m, log2bs, xyz, static_cast<float*>(scratch), idxs, s);
    }
    if (path != kFpsOnchip && scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 15u) == 0)
    {
        float4* sorted = static_cast<float4*>(scratch);
        const int rc = fps_launch_sort(b, n, xyz, sorted, s);
        if (rc != TPK_OK) return rc;
        fps_batched_config(n, &c);
        if (fps_wants_batched(c))
            return c.nranks > 1 ? fps_launch_batched<true>(c, b, n, m, log2bs, xyz, sorted, idxs, s)
                                : fps_launch_batched<false>(c, b, n, m, log2bs, xyz, sorted, idxs, s);
        return c.nranks > 1 ? fps_launch_s<true, true>(c, b, n, m, log2bs, xyz, sorted, idxs, s)
                            : fps_launch_s<false, true>(c, b, n, m, log2bs, xyz, sorted, idxs, s);
    }
    return c.nranks > 1 ? fps_launch_s<true, false>(c, b, n, m, log2bs, xyz, nullptr, idxs, s)
                        : fps_launch_s<false, false>(c, b, n, m, log2bs, xyz, nullptr, idxs, s);
}

// Coordinates of the samples, new_xyz[b, j, :] = xyz[b, idxs[b, j], :].  A separate pass of a
// few microseconds: written from inside the sampling kernels the four stores per round sat on
// the critical path of every round (measured 5 % of the whole call).
namespace tpk
{
namespace
{
__global__ void __launch_bounds__(256)
    fps_gather_xyz_kernel(long long total, int n, int m, const float* __restrict__ xyz, const int32_t* __restrict__ idxs,
                          float* __restrict__ new_xyz)
{
    const long long t = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (t >= total) return;
    const long long cloud = t / m;
    const float* src = xyz + (cloud * n + __ldg(idxs + t)) * 3;
    new_xyz[3 * t + 0] = __ldg(src + 0);
    new_xyz[3 * t + 1] = __ldg(src + 1);
    new_xyz[3 * t + 2] = __ldg(src + 2);
}
}  // namespace
}  // namespace tpk

extern "C" int tpk_furthest_point_sampling_xyz(int b, int n, int m, const float* xyz, void* scratch,
                                               int64_t scratch_bytes, int32_t* idxs, float* new_xyz,
                                               void* stream)
{
    using namespace tpk;
    const int rc = tpk_furthest_point_sampling(b, n, m, xyz, scratch, scratch_bytes, idxs, stream);
    if (rc != TPK_OK || new_xyz == nullptr || b == 0 || m == 0) return rc;
    const long long total = static_cast<long long>(b) * m;
    const long long grid = (total + 255) / 256;
    TPK_REQUIRE(grid < (1ll << 31), "fps: too many samples");
    count_launches(1), fps_gather_xyz_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        total, n, m, xyz, idxs, new_xyz);
    return check_launch("fps gather");
}

// ------------------------------------------------------------- entry point without scratch
//
// Scratch for tpk_furthest_point_sampling_static: lives in the library image, so every
// GPU that loads the library holds these 8 MiB until the process exits.
constexpr long long kFpsStaticFloats = 2ll * 1024 * 1024;
static __device__ __align__(256) float g_fps_static_scratch[kFpsStaticFloats];

namespace
{
constexpr int kMaxDevices = 64;
// device address of the array, per device; threads that race on a device's first call all store
// the same address
std::atomic<float*> g_fps_static_ptr[kMaxDevices] = {};
}  // namespace

extern "C" int64_t tpk_fps_static_capacity(void) { return kFpsStaticFloats; }

extern "C" int tpk_furthest_point_sampling_static(int b, int n, int m, const float* xyz,
                                                  int32_t* idxs, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(b >= 0 && n >= 0 && m >= 0, "fps_static: negative size (b=%d n=%d m=%d)", b, n, m);
    if (b == 0 || m == 0) return TPK_OK;
    TPK_REQUIRE(n > 0, "fps_static: cannot sample %d points from an empty cloud", m);
    TPK_REQUIRE(xyz != nullptr && idxs != nullptr, "fps_static: NULL pointer");
    if (static_cast<long long>(b) * n > kFpsStaticFloats)
    {
        set_error("fps_static: b*n = %lld points exceed the built-in scratch of %lld points; "
                  "use tpk_furthest_point_sampling with caller-provided scratch",
                  static_cast<long long>(b) * n, kFpsStaticFloats);
        return TPK_ERR_UNSUPPORTED;
    }
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    {
        set_error("fps_static: cannot identify the current device: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    // In host code the array's name is only a handle; the kernel needs the address the
    // array has on the device that is current now.  Looked up once per device.
    float* scratch = g_fps_static_ptr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr)
    {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_fps_static_scratch);
        if (err != cudaSuccess || p == nullptr)
        {
            set_error("fps_static: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
        scratch = static_cast<float*>(p);
        g_fps_static_ptr[dev].store(scratch, std::memory_order_release);
    }
    int log2bs = floor_log2(n);
    if (log2bs > 9) log2bs = 9;
    // the kernel writes every scratch element it later reads (its first pass sets the
    // running minima), so whatever an earlier call left behind is irrelevant
    return fps_launch_global(b, n, m, log2bs, xyz, scratch, idxs, static_cast<cudaStream_t>(stream));
}

