// Region growing and instance IoU (the PointGroup helpers around partial_dense ball query)
// for sm_100a.
//
// grow_proximity: torch_points_kernels/cluster.py:8-46 of the reference runs a sequential
//   traversal on the CPU (numba): seeds in index order, a cluster = every point not yet
//   visited that can be reached from the seed along neighbour lists.  The lists are the
//   first nsample hits of a radius search, so the graph is directed (a crowded point may
//   not list a neighbour that lists it).  The traversal assigns point v to the smallest
//   index that can reach v along directed edges, which is a fixed point of "push the
//   smallest label seen so far along every edge": every thread owns a point, pushes its
//   label to the points it lists (atomicMin) and shortens its own label chain (the label of
//   my label is also an ancestor of mine).  The host repeats launches until nothing changes.
// instance_iou:   cuda/src/metrics_gpu.cu:9-43: the reference compares every point of a proposal
//   with every ground-truth instance; here a CTA histograms the proposal's labels once.
#include "tpk_common.cuh"

namespace tpk
{
namespace
{

constexpr int kClThreads = 256;

__global__ void __launch_bounds__(kClThreads)
    grow_labels_kernel(long long n, int nsample, const int64_t* __restrict__ neighbours, int32_t* __restrict__ labels,
                       int32_t* __restrict__ changed)
{
    const long long u = static_cast<long long>(blockIdx.x) * kClThreads + threadIdx.x;
    if (u >= n) return;
    bool moved = false;
    int lu = labels[u];
    // shorten the chain first: the label of my label reaches me too
    const int ll = labels[lu];
    if (ll < lu)
    {
        atomicMin(labels + u, ll);
        lu = ll;
        moved = true;
    }
    const int64_t* row = neighbours + u * nsample;
    for (int s = 0; s < nsample; ++s)
    {
        const long long v = __ldg(row + s);
        if (v == -1) break;  // the list ends at the first unused slot (cluster.py:25-26)
        if (v < 0 || v >= n) continue;
        if (atomicMin(labels + v, lu) > lu) moved = true;
    }
    if (moved) *changed = 1;
}

// One CTA per proposal: histogram of the ground-truth instance ids of its points, then one
// IoU per instance of the proposal's sample.
__global__ void __launch_bounds__(kClThreads)
    instance_iou_kernel(int n_proposals, long long total_gt, long long n_points, const int64_t* __restrict__ num_gt,
                        const int64_t* __restrict__ proposals_idx, const int64_t* __restrict__ proposals_offset,
                        const int64_t* __restrict__ instance_labels, const int64_t* __restrict__ offset_num_gt,
                        const int64_t* __restrict__ batch, const int64_t* __restrict__ instance_pointnum,
                        float* __restrict__ out)
{
    extern __shared__ int hist[];
    const int p = blockIdx.x;
    if (p >= n_proposals) return;
    const long long start = proposals_offset[p], end = proposals_offset[p + 1];
    if (end <= start) return;
    const long long first = proposals_idx[start];
    if (first < 0 || first >= n_points) return;
    const long long sample = batch[first];
    const int ninst = static_cast<int>(num_gt[sample]);
    const long long inst_off = offset_num_gt[sample];
    for (int i = threadIdx.x; i < ninst; i += kClThreads) hist[i] = 0;
    __syncthreads();
    for (long long i = start + threadIdx.x; i < end; i += kClThreads)
    {
        const long long idx = proposals_idx[i];
        if (idx < 0 || idx >= n_points) continue;
        const int lab = static_cast<int>(instance_labels[idx]);  // 0 is "no instance"
        if (lab >= 1 && lab <= ninst) atomicAdd(hist + lab - 1, 1);
    }
    __syncthreads();
    const int proposal_total = static_cast<int>(end - start);
    for (int i = threadIdx.x; i < ninst; i += kClThreads)
    {
        const int inter = hist[i];
        const int inst_total = static_cast<int>(instance_pointnum[inst_off + i]);
        // float / (float + double): evaluated in double, stored as float (metrics_gpu.cu:37-39)
        const double q = static_cast<double>(static_cast<float>(inter)) /
                         (static_cast<double>(static_cast<float>(proposal_total + inst_total - inter)) + 1e-5);
        out[static_cast<long long>(p) * total_gt + inst_off + i] = static_cast<float>(q);
    }
}

}  // namespace
}  // namespace tpk

extern "C" int tpk_grow_labels_step(int64_t n, int nsample, const int64_t* neighbours, int32_t* labels,
                                    int32_t* changed, int rounds, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(n >= 0 && nsample >= 0 && rounds >= 0, "grow_labels: negative size");
    TPK_REQUIRE(n < (1ll << 31), "grow_labels: too many points");
    if (n == 0 || rounds == 0) return TPK_OK;
    TPK_REQUIRE(labels && changed && (neighbours || nsample == 0), "grow_labels: NULL pointer");
    const unsigned g = static_cast<unsigned>((n + kClThreads - 1) / kClThreads);
    for (int r = 0; r < rounds; ++r)
        count_launches(1), grow_labels_kernel<<<g, kClThreads, 0, static_cast<cudaStream_t>(stream)>>>(n, nsample, neighbours,
                                                                                                   labels, changed);
    return check_launch("grow_labels");
}

extern "C" int tpk_instance_iou(int n_proposals, int64_t total_gt_instances, int64_t max_gt_instances, int64_t n_points,
                                const int64_t* num_gt_instances, const int64_t* proposals_idx,
                                const int64_t* proposals_offset, const int64_t* instance_labels,
                                const int64_t* offset_num_gt_instances, const int64_t* batch,
                                const int64_t* instance_pointnum, float* proposals_iou, void* stream)
{
    using namespace tpk;
    TPK_REQUIRE(n_proposals >= 0 && total_gt_instances >= 0 && max_gt_instances >= 0 && n_points >= 0,
                "instance_iou: negative size");
    if (n_proposals == 0 || total_gt_instances == 0) return TPK_OK;
    TPK_REQUIRE(num_gt_instances && proposals_idx && proposals_offset && instance_labels && offset_num_gt_instances && batch &&
                    instance_pointnum && proposals_iou,
                "instance_iou: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(proposals_iou, 0, sizeof(float) * static_cast<size_t>(n_proposals) * total_gt_instances, s);
    if (err != cudaSuccess)
    {
        set_error("instance_iou: memset: %s", cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    const size_t smem = sizeof(int) * static_cast<size_t>(max_gt_instances > 0 ? max_gt_instances : 1);
    if (smem > 200 * 1024)
    {
        set_error("instance_iou: %lld instances in one sample exceed the %d the kernel holds",
                  static_cast<long long>(max_gt_instances), 200 * 1024 / 4);
        return TPK_ERR_UNSUPPORTED;
    }
    if (smem > kDynSmemOptIn)
    {
        err = cudaFuncSetAttribute(instance_iou_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess)
        {
            set_error("instance_iou: shared memory attribute: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
    }
    count_launches(1), instance_iou_kernel<<<n_proposals, kClThreads, smem, s>>>(
        n_proposals, total_gt_instances, n_points, num_gt_instances, proposals_idx, proposals_offset, instance_labels,
        offset_num_gt_instances, batch, instance_pointnum, proposals_iou);
    return check_launch("instance_iou");
}
