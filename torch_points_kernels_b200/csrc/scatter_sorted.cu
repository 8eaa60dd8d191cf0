// Gradient of grouping_operation without atomics on the hot path (sm_100a).
//
//   grad_features[b, c, idx[b, p]] += grad_out[b, c, p]      p = position (centre, slot)
//
// is a scatter of every (batch, channel) row of grad_out (npoint*nsample values) into a row
// of n values, with the same idx for all c rows of a cloud.  The kernel in gather.cu keeps the
// small row in shared memory and adds with shared-memory float atomics, which cost about one
// shared-memory wavefront per lane.  Here the index is inverted once per call instead:
//
//   1. grouping_sort_kernel: the positions of a cloud are cut into tiles of at most 16384; the
//      (target, position) pairs of a tile are sorted by target (counting sort in shared memory)
//      and stored so that thread t of the second kernel owns entries [t*chunk, (t+1)*chunk) of
//      the sorted order and a warp reads them with coalesced loads.
//   2. grouping_bwd_sorted_kernel: a CTA owns one (batch, channel) row.  Per tile it stages
//      the row's gradient values in shared memory (TMA bulk copies, double-buffered), every
//      thread walks its entries: values of equal targets are summed in a register (a run) and
//      a finished run is added to the row's accumulator in shared memory with a plain
//      read-modify-write.  That is race-free because the entries are sorted: all entries of a
//      target in this tile lie inside one thread's chunk, unless the run touches an end of the
//      chunk - the first and the last run of a chunk are added with atomics.
//      Gathers and plain updates cost about one shared-memory wavefront per six lanes.
//
// The sum of a target's contributions is formed in another order than the reference's
// atomics form it (which have no fixed order either); results agree to rounding.
//
// Semantics: autograd's scatter-add backward of the gather at
// torch_points_kernels/torchpoints.py:129-146.
#include "tpk_common.cuh"

namespace tpk
{
TPK_DEFINE_STATUS_WORD()

namespace
{

constexpr int kSortedThreads = 512;
constexpr int kMaxTile = 16384;   // positions per tile: 15 bits of an entry hold 0..16384
constexpr int kMaxChunk = kMaxTile / kSortedThreads;
constexpr int kPosBits = 15;
constexpr uint32_t kPosMask = (1u << kPosBits) - 1u;
constexpr int kMaxTargets = (1 << (32 - kPosBits)) - 2;  // the key n (nothing to add) must fit too
constexpr size_t kSmemBudget = 200 * 1024;

struct SortedPlan
{
    int tile;    // positions per tile, a multiple of 512
    int chunk;   // entries per thread = tile / 512
    int tiles;   // tiles per cloud
    int bufs;    // staging buffers: 2 when a row has more than one tile
    size_t smem;
};

// Rounded-up row lengths in floats: the accumulator carries one extra slot (index n, where entries
// that add nothing go) and a staged tile one extra value (index tile, always 0).
__host__ __device__ inline int acc_stride(int n) { return (n + 1 + 3) & ~3; }
__host__ __device__ inline int tile_stride(int tile) { return tile + 4; }

// Rows of more than 32 KB only (measured on the pipeline's shapes, 16 clouds: 0.29 ms against
// 0.39 ms for rows of 64 KB; 0.18 against 0.165 for rows of 16 KB, where the atomic kernel keeps
// two rows per CTA and several CTAs per SM): one row per CTA and the longest tile that fits.
constexpr size_t kMinRowBytes = 32 * 1024;

bool make_plan(int n, long long ps, SortedPlan* out)
{
    if (n > kMaxTargets || ps <= 0 || static_cast<size_t>(n) * sizeof(float) <= kMinRowBytes) return false;
    for (int nominal = kMaxTile; nominal >= 2048; nominal >>= 1)
    {
        SortedPlan p;
        long long t = nominal;
        if (ps < t) t = (ps + kSortedThreads - 1) / kSortedThreads * kSortedThreads;
        p.tile = static_cast<int>(t);
        p.chunk = p.tile / kSortedThreads;
        p.tiles = static_cast<int>((ps + p.tile - 1) / p.tile);
        p.bufs = p.tiles > 1 ? 2 : 1;
        p.smem = (acc_stride(n) + static_cast<size_t>(p.bufs) * tile_stride(p.tile)) * sizeof(float);
        if (p.smem <= kSmemBudget)
        {
            *out = p;
            return true;
        }
    }
    return false;
}

// ------------------------------------------------------------------ 1. sort

// One CTA per (cloud, tile).  Keys 0..n-1 are targets; key n collects positions whose index
// addresses nothing (recorded in the status word) and the padding of the last tile: their
// entries point at the zero behind the staged tile and at the spare accumulator slot.
__global__ void __launch_bounds__(kSortedThreads)
    grouping_sort_kernel(int n, long long ps, int tile, int chunk, int tiles, const int64_t* __restrict__ idx,
                         uint32_t* __restrict__ entries)
{
    extern __shared__ uint32_t cnt[];  // n + 1 counters, then offsets
    __shared__ uint32_t warp_sums[kSortedThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cloud = blockIdx.x / tiles, t = blockIdx.x - cloud * tiles;
    const long long p0 = static_cast<long long>(t) * tile;
    const int len = static_cast<int>(min(static_cast<long long>(tile), ps - p0));
    const int64_t* ip = idx + static_cast<size_t>(cloud) * ps + p0;
    uint32_t* out = entries + (static_cast<size_t>(cloud) * tiles + t) * tile;
    const int nkeys = n + 1;

    // the keys of this thread's positions (p = tid, tid + 512, ...), loaded once with all loads in
    // flight together and kept in registers for both passes
    int keys[kMaxChunk];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < kMaxChunk; ++i)
    {
        const int p = tid + i * kSortedThreads;
        long long v = -1;
        if (p < len) v = __ldg(ip + p);
        const bool ok = static_cast<unsigned long long>(v) < static_cast<unsigned long long>(n);
        bad |= p < len && !ok;
        keys[i] = ok ? static_cast<int>(v) : n;
    }
    for (int i = tid; i < nkeys; i += kSortedThreads) cnt[i] = 0u;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kMaxChunk; ++i)
        if (tid + i * kSortedThreads < tile) atomicAdd(&cnt[keys[i]], 1u);
    __syncthreads();
    // exclusive scan of the counters: every thread a run of consecutive keys (odd length, so
    // that the threads of a warp start in different banks)
    const int seg = ((nkeys + kSortedThreads - 1) / kSortedThreads) | 1;
    const int k0 = min(tid * seg, nkeys), k1 = min(k0 + seg, nkeys);
    uint32_t local = 0;
    for (int k = k0; k < k1; ++k) local += cnt[k];
    uint32_t incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
    {
        const uint32_t v = __shfl_up_sync(kFullMask, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0)
    {
        uint32_t w = lane < kSortedThreads / 32 ? warp_sums[lane] : 0u;
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            const uint32_t v = __shfl_up_sync(kFullMask, wi, o);
            if (lane >= o) wi += v;
        }
        if (lane < kSortedThreads / 32) warp_sums[lane] = wi - w;
    }
    __syncthreads();
    uint32_t run = warp_sums[warp] + incl - local;
    for (int k = k0; k < k1; ++k)
    {
        const uint32_t v = cnt[k];
        cnt[k] = run;
        run += v;
    }
    __syncthreads();
    // scatter: sorted rank q -> the slot thread q / chunk reads in its step q % chunk
    const int per_warp = 32 * chunk;
#pragma unroll
    for (int i = 0; i < kMaxChunk; ++i)
    {
        const int p = tid + i * kSortedThreads;
        if (p < tile)
        {
            const int key = keys[i];
            const uint32_t q = atomicAdd(&cnt[key], 1u);
            const uint32_t owner = q / chunk, step = q - owner * chunk;
            const uint32_t slot = (owner >> 5) * per_warp + step * 32u + (owner & 31u);
            out[slot] = (static_cast<uint32_t>(key) << kPosBits) | static_cast<uint32_t>(key == n ? tile : p);
        }
    }
    if (bad) atomicOr(&g_dev_status, kStatusBadIndex);
}

// ------------------------------------------------------------------ 2. sums

__device__ __forceinline__ bool wait_parity_bounded(uint32_t mbar, uint32_t parity)
{
    unsigned long long t0 = 0;
    for (unsigned it = 1;; ++it)
    {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(mbar), "r"(parity)
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

// One CTA per (batch, channel) row.
__global__ void __launch_bounds__(kSortedThreads, 1)
    grouping_bwd_sorted_kernel(int n, long long ps, long long gbs, int tile, int chunk, int tiles, int bufs, int use_tma, int c,
                               const float* __restrict__ grad_out, const uint32_t* __restrict__ entries,
                               float* __restrict__ grad_small)
{
    extern __shared__ __align__(128) float smem[];
    __shared__ __align__(8) uint64_t mbar[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bi = blockIdx.x / c;
    const int astr = acc_stride(n), tstr = tile_stride(tile);
    float* acc = smem;            // [astr]
    float* stage = smem + astr;   // [bufs][tstr]
    const float* g = grad_out + static_cast<size_t>(bi) * gbs + static_cast<size_t>(blockIdx.x - bi * c) * ps;
    const uint32_t* ent = entries + static_cast<size_t>(bi) * tiles * tile + static_cast<size_t>(warp) * 32 * chunk + lane;

    for (int i = tid; i < astr; i += kSortedThreads) acc[i] = 0.f;
    // the value behind a staged tile, where entries that add nothing point
    if (tid < bufs) stage[static_cast<size_t>(tid) * tstr + tile] = 0.f;
    const uint32_t bar0 = static_cast<uint32_t>(__cvta_generic_to_shared(&mbar[0]));
    if (use_tma && tid == 0)
    {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // one thread asks for tile t of the row into buffer t % bufs
    auto request = [&](int t) {
        const long long p0 = static_cast<long long>(t) * tile;
        const uint32_t bytes = 4u * static_cast<uint32_t>(min(static_cast<long long>(tile), ps - p0));
        const uint32_t bar = bar0 + 8u * static_cast<uint32_t>(t % bufs);
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(stage + static_cast<size_t>(t % bufs) * tstr));
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                     "l"(g + p0), "r"(bytes), "r"(bar)
                     : "memory");
    };
    if (use_tma && tid == 0)
    {
        request(0);
        if (bufs > 1 && tiles > 1) request(1);
    }

    // this thread's entries of a tile are loaded one tile ahead
    uint32_t e[kMaxChunk], en[kMaxChunk];
#pragma unroll
    for (int i = 0; i < kMaxChunk; ++i)
        if (i < chunk) en[i] = __ldg(ent + i * 32);
    for (int t = 0; t < tiles; ++t)
    {
        const int buf = t % bufs;
#pragma unroll
        for (int i = 0; i < kMaxChunk; ++i) e[i] = en[i];
        if (t + 1 < tiles)
        {
            const uint32_t* et = ent + static_cast<size_t>(t + 1) * tile;
#pragma unroll
            for (int i = 0; i < kMaxChunk; ++i)
                if (i < chunk) en[i] = __ldg(et + i * 32);
        }
        const float* st = stage + static_cast<size_t>(buf) * tstr;
        if (use_tma)
        {
            const bool arrived = wait_parity_bounded(bar0 + 8u * static_cast<uint32_t>(buf), static_cast<uint32_t>(t / bufs) & 1u);
            // a copy that did not arrive in time is recorded; this and all later tiles are staged by hand
            if (__syncthreads_or(arrived ? 0 : 1))
            {
                use_tma = 0;
                if (tid == 0) atomicOr(&g_dev_status, kStatusWaitAbandoned);
            }
        }
        if (!use_tma)
        {
            const long long p0 = static_cast<long long>(t) * tile;
            const int len = static_cast<int>(min(static_cast<long long>(tile), ps - p0));
            float* sw = stage + static_cast<size_t>(buf) * tstr;
            for (int i = tid; i < len; i += kSortedThreads) sw[i] = __ldg(g + p0 + i);
            __syncthreads();
        }

        // Runs of equal targets.  A run that touches neither end of the chunk has its target to
        // itself in this tile (the entries are sorted) and is added with a plain read-modify-write;
        // the first and the last run of a chunk may continue in the neighbouring threads' chunks
        // and are added with atomics.
        uint32_t cur = e[0] >> kPosBits;
        float sum = st[e[0] & kPosMask];
        bool first = true;
#pragma unroll
        for (int i = 1; i < kMaxChunk; ++i)
        {
            if (i < chunk)  // uniform
            {
                const uint32_t tg = e[i] >> kPosBits;
                const bool changed = tg != cur;
                const float v = st[e[i] & kPosMask];
                if (changed && first) atomicAdd(acc + cur, sum);
                if (changed && !first) acc[cur] += sum;
                sum = changed ? v : sum + v;
                first = first && !changed;
                cur = tg;
            }
        }
        atomicAdd(acc + cur, sum);
        __syncthreads();  // the accumulator is consistent and every thread is done with this buffer
        if (use_tma && tid == 0 && t + bufs < tiles) request(t + bufs);
    }

    float* dst = grad_small + static_cast<size_t>(blockIdx.x) * n;
    for (int i = tid; i < n; i += kSortedThreads) dst[i] = acc[i];
}

int launch_sorted(const SortedPlan& p, int b, int c, int n, long long ps, long long gbs, const float* grad_out, const uint32_t* entries,
                  float* grad_small, cudaStream_t s)
{
    auto kernel = grouping_bwd_sorted_kernel;
    prefer_max_shared(kernel);
    if (p.smem > kDynSmemOptIn)
    {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(p.smem));
        if (err != cudaSuccess)
        {
            set_error("grouping_grad: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    const long long grid = static_cast<long long>(b) * c;
    TPK_REQUIRE(grid < (1ll << 31), "grouping_grad: too many rows");
    const int use_tma = (ps % 4 == 0) && (gbs % 4 == 0) && ((reinterpret_cast<uintptr_t>(grad_out) & 15u) == 0);
    count_launches(1), kernel<<<static_cast<unsigned>(grid), kSortedThreads, p.smem, s>>>(
                           n, ps, gbs, p.tile, p.chunk, p.tiles, p.bufs, use_tma, c, grad_out, entries, grad_small);
    return check_launch("grouping_grad (sorted)");
}

}  // namespace
}  // namespace tpk

extern "C" int64_t tpk_grouping_grad_scratch_bytes(int b, int c, int n, int npoint, int nsample)
{
    tpk::SortedPlan p;
    if (b <= 0 || c <= 0 || n <= 0 || npoint <= 0 || nsample <= 0) return 0;
    if (!tpk::make_plan(n, static_cast<long long>(npoint) * nsample, &p)) return 0;
    return static_cast<int64_t>(b) * p.tiles * p.tile * static_cast<int64_t>(sizeof(uint32_t));
}

namespace tpk
{
namespace
{
// grad_out rows as in grouping_grad_atomic (gbs = batch stride in floats)
int grouping_grad_with_scratch(int b, int c, int n, int npoint, int nsample, const float* grad_out, long long gbs,
                               const int64_t* idx, float* grad_features, void* scratch, int64_t scratch_bytes,
                               cudaStream_t s)
{
    TPK_REQUIRE(b >= 0 && c >= 0 && n >= 0 && npoint >= 0 && nsample >= 0, "grouping_grad: negative size");
    const int64_t want = tpk_grouping_grad_scratch_bytes(b, c, n, npoint, nsample);
    if (scratch != nullptr && scratch_bytes < want)
    {
        set_error("grouping_grad: scratch of %lld bytes given, %lld needed", static_cast<long long>(scratch_bytes),
                  static_cast<long long>(want));
        return TPK_ERR_SCRATCH;
    }
    SortedPlan p;
    const long long ps = static_cast<long long>(npoint) * nsample;
    if (scratch == nullptr || want == 0 || test_path("scatter_atomic") || test_path("scatter_global") ||
        !make_plan(n, ps, &p))
        return grouping_grad_atomic(b, c, n, npoint, nsample, grad_out, gbs, idx, grad_features, s);
    TPK_REQUIRE(grad_out && idx && grad_features, "grouping_grad: NULL pointer");
    TPK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 3u) == 0, "grouping_grad: scratch must be 4-byte aligned");
    uint32_t* entries = static_cast<uint32_t*>(scratch);
    {
        auto kernel = grouping_sort_kernel;
        prefer_max_shared(kernel);
        const size_t smem = static_cast<size_t>(n + 1) * sizeof(uint32_t);
        if (smem > kDynSmemOptIn)
        {
            cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (err != cudaSuccess)
            {
                set_error("grouping_grad: shared memory attribute: %s", cudaGetErrorString(err));
                return TPK_ERR_CUDA;
            }
        }
        const long long grid = static_cast<long long>(b) * p.tiles;
        TPK_REQUIRE(grid < (1ll << 31), "grouping_grad: too many tiles");
        count_launches(1), kernel<<<static_cast<unsigned>(grid), kSortedThreads, smem, s>>>(n, ps, p.tile, p.chunk, p.tiles, idx, entries);
        const int rc = check_launch("grouping_grad (sort)");
        if (rc != TPK_OK) return rc;
    }
    return launch_sorted(p, b, c, n, ps, gbs, grad_out, entries, grad_features, s);
}
}  // namespace
}  // namespace tpk

extern "C" int tpk_grouping_grad_ws(int b, int c, int n, int npoint, int nsample, const float* grad_out, const int64_t* idx,
                                    float* grad_features, void* scratch, int64_t scratch_bytes, void* stream)
{
    return tpk::grouping_grad_with_scratch(b, c, n, npoint, nsample, grad_out, static_cast<long long>(c) * npoint * nsample, idx,
                                           grad_features, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int tpk_sa_group_grad(int b, int c, int n, int npoint, int nsample, const float* grad_out, const int64_t* idx,
                                 float* grad_features, void* scratch, int64_t scratch_bytes, void* stream)
{
    // the feature rows of the (b, 3 + c, npoint, nsample) gradient: rows 3.. of every cloud
    const long long ps = static_cast<long long>(npoint) * nsample;
    return tpk::grouping_grad_with_scratch(b, c, n, npoint, nsample, grad_out ? grad_out + 3 * ps : nullptr, (3ll + c) * ps, idx,
                                           grad_features, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}
