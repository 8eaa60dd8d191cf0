/*
 * tpk_b200 — C ABI of the B200 (sm_100a) spatial-search kernels.
 *
 * One shared library, libtpk_b200.so, exports every function below with C linkage.
 * Conventions shared by all entry points:
 *   - every pointer is a DEVICE pointer on the current CUDA device unless stated
 *     otherwise; inputs are borrowed, outputs and scratch are owned by the caller;
 *   - the library allocates no device memory, keeps no per-call state and never
 *     synchronises the host: kernels are enqueued on `stream` (a cudaStream_t passed
 *     as void*, NULL = legacy default stream) and the call returns at once;
 *   - outputs need no pre-fill: the kernels write every element, including the
 *     padding values that are part of the contract (dense ball query idx 0 / dist -1,
 *     partial_dense -1 / -1, FPS 0, gradients start from 0);
 *   - layouts are dense row-major ("contiguous") with the dimension order given;
 *   - the return value is a tpk_status; nothing aborts the process.
 *
 * Each declaration cites the reference interface it stands in for, by path inside
 * torch-points-kernels 0.7.1.
 */
#ifndef TPK_B200_H
#define TPK_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define TPK_API __attribute__((visibility("default")))
#else
#define TPK_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tpk_status
{
    TPK_OK = 0,
    TPK_ERR_INVALID_ARGUMENT = 1, /* negative size, NULL pointer, k > n, ...            */
    TPK_ERR_CUDA = 2,             /* a CUDA runtime call or launch failed               */
    TPK_ERR_UNSUPPORTED = 3,      /* size outside what the kernels are instantiated for */
    TPK_ERR_SCRATCH = 4           /* scratch pointer missing or too small               */
} tpk_status;

/* Library version, e.g. 100 = 0.1.0. */
TPK_API int tpk_version(void);

/* Text of the last error recorded on the calling thread (never NULL). */
TPK_API const char* tpk_last_error(void);

/*
 * Sticky device-side status word of the current device: 0, or a combination of
 *   TPK_STATUS_WAIT_ABANDONED  a kernel gave up a bounded wait (cluster exchange or bulk copy
 *                              that did not complete within a second); its outputs are invalid;
 *   TPK_STATUS_BAD_INDEX       a gather/scatter kernel met an index outside its tensor; the
 *                              element was skipped (gathers write 0 for it) and nothing outside
 *                              the caller's tensors was touched.
 * Reading it synchronises the device.  `reset` != 0 clears it after reading.
 */
#define TPK_STATUS_WAIT_ABANDONED 1
#define TPK_STATUS_BAD_INDEX 2
TPK_API int tpk_device_status(int* status_out, int reset);

/*
 * Number of kernels the library has launched in this process so far, on any device and
 * stream.  A launch recorded by a stream capture counts once, when it is captured, not when
 * the graph is replayed.  For launch accounting in benchmarks; no counterpart in the reference.
 */
TPK_API int64_t tpk_kernel_launches(void);

/* ---------------------------------------------------------------- sampling ---- */

/*
 * Iterative furthest point sampling.  xyz (b,n,3) f32 -> idxs (b,m) int32.
 * First sample is index 0; squared distances; points with |p|^2 <= 1e-3 are never
 * candidates; ties resolve as in the reference's 512-thread tree reduction.
 * Replaces furthest_point_sampling_kernel_wrapper, cuda/src/sampling.cpp:5-6
 * (kernel cuda/src/sampling_gpu.cu:16-144), including the zero/1e10 fills of
 * cuda/src/sampling.cpp:14-18.
 *
 * scratch: scratch_bytes >= tpk_fps_scratch_bytes(b,n,m) bytes of device memory (16-byte
 * aligned).  Required for clouds of more than 131072 points (sorted copy + running minima);
 * optional below, where it holds a spatially sorted copy that lets most of the cloud skip most
 * rounds (NULL: the kernel without it, same result).  A buffer smaller than
 * tpk_fps_scratch_bytes returns TPK_ERR_SCRATCH and launches nothing.  Content on entry is
 * irrelevant.
 */
TPK_API int tpk_furthest_point_sampling(int b, int n, int m, const float* xyz, void* scratch,
                                int64_t scratch_bytes, int32_t* idxs, void* stream);

/*
 * The same, followed by a gather of the coordinates of the samples: new_xyz (b,m,3) f32,
 * i.e. xyz[b, idxs[b, j], :] (what callers otherwise do with several tensor operations);
 * NULL skips it.  No counterpart in the reference.
 */
TPK_API int tpk_furthest_point_sampling_xyz(int b, int n, int m, const float* xyz, void* scratch,
                                    int64_t scratch_bytes, int32_t* idxs, float* new_xyz,
                                    void* stream);
TPK_API int64_t tpk_fps_scratch_bytes(int b, int n, int m);

/*
 * Furthest point sampling for callers that may not allocate device memory.  Same
 * inputs, outputs and results as tpk_furthest_point_sampling, but the scratch (the
 * running minimum distance of every point) is a fixed array inside the library instead
 * of a caller buffer, and the call performs no cudaMalloc / cudaFree or any other
 * allocation.  It is meant for code that runs where allocation is off limits: a plugin's
 * enqueue hook in an inference runtime that owns all device memory, a real-time loop
 * that must not hit the allocator's lock, a process whose memory budget was handed out
 * in full at start-up.
 * Limits and rules:
 *   - b * n <= tpk_fps_static_capacity() (2 Mi points = 8 MiB, held by every GPU that
 *     loads the library until the process exits); larger requests return
 *     TPK_ERR_UNSUPPORTED and tpk_last_error() names the limit;
 *   - the first call on each device looks up the array's device address (with that
 *     device current); make that first call before starting any stream capture;
 *   - all calls on a device share the one array: two calls that overlap on the GPU
 *     (different streams, no ordering between them) race and give wrong indices.
 *     The array keeps the previous call's contents; every call rewrites what it reads.
 * No counterpart in the reference, whose FPS always allocates its scratch with torch
 * (cuda/src/sampling.cpp:17).
 */
TPK_API int tpk_furthest_point_sampling_static(int b, int n, int m, const float* xyz,
                                               int32_t* idxs, void* stream);
TPK_API int64_t tpk_fps_static_capacity(void);

/* --------------------------------------------------------------- ball query ---- */

/*
 * Dense radius search.  new_xyz (b,m,3) centres, xyz (b,n,3) candidates ->
 * idx (b,m,nsample) int64, dist (b,m,nsample) f32 squared distances.
 * First nsample candidates in index order with d2 < radius*radius; unused idx slots
 * repeat the first hit (0 when there is none); unused dist slots are -1.
 * Replaces query_ball_point_kernel_dense_wrapper, cuda/src/ball_query.cpp:5-7
 * (kernel cuda/src/ball_query_gpu.cu:9-52) and the fills of ball_query.cpp:26-29.
 */
TPK_API int tpk_ball_query_dense(int b, int n, int m, float radius, int nsample, const float* new_xyz,
                         const float* xyz, int64_t* idx, float* dist, void* stream);

/*
 * The same search with caller scratch: clouds are binned into a uniform grid (cells at
 * least one radius wide) and a centre only examines the 27 cells around it; centres in
 * very dense neighbourhoods, for which the early-exit scan is cheaper, fall through to
 * the scan.  Results are identical to tpk_ball_query_dense bit for bit.
 * scratch: tpk_ball_query_dense_scratch_bytes(b,n,m,nsample) bytes, 256-byte aligned;
 * when that returns 0 (small clouds, nsample > 128) or scratch is NULL the call is
 * tpk_ball_query_dense.  No counterpart in the reference.
 */
TPK_API int tpk_ball_query_dense_ws(int b, int n, int m, float radius, int nsample,
                                    const float* new_xyz, const float* xyz, int64_t* idx, float* dist,
                                    void* scratch, int64_t scratch_bytes, void* stream);
TPK_API int64_t tpk_ball_query_dense_scratch_bytes(int b, int n, int m, int nsample);

/*
 * Radius search on packed segments.  x (size_x,3) candidates, y (size_y,3) centres,
 * batch_x (size_x) / batch_y (size_y) sorted int64 segment ids ->
 * idx (size_y,nsample) int64 positions in x, dist (size_y,nsample) f32; test is
 * d2 <= radius*radius; unused slots are -1 in both outputs.
 * Replaces query_ball_point_kernel_partial_wrapper, cuda/src/ball_query.cpp:9-13
 * (kernel cuda/src/ball_query_gpu.cu:54-95) together with the host-side offset
 * construction of cuda/src/ball_query.cpp:64-73: segment ranges are found on the
 * device by binary search, so no device-to-host copy of batch_x[-1] takes place.
 */
TPK_API int tpk_ball_query_partial_dense(int64_t size_x, int64_t size_y, float radius, int nsample,
                                 const float* x, const float* y, const int64_t* batch_x,
                                 const int64_t* batch_y, int64_t* idx, float* dist, void* stream);

/*
 * The packed query with caller scratch: points are binned on a hashed uniform grid (cells one
 * radius wide, keyed by segment and cell) and a query looks at the 27 cells around it;
 * results are identical to tpk_ball_query_partial_dense bit for bit.  scratch:
 * tpk_ball_query_partial_dense_scratch_bytes(size_x,size_y,radius) bytes, 256-byte aligned;
 * when that returns 0 (fewer than 4096 points) or scratch is NULL the call is the plain one.
 * No counterpart in the reference.
 */
TPK_API int tpk_ball_query_partial_dense_ws(int64_t size_x, int64_t size_y, float radius, int nsample,
                                            const float* x, const float* y, const int64_t* batch_x,
                                            const int64_t* batch_y, int64_t* idx, float* dist, void* scratch,
                                            int64_t scratch_bytes, void* stream);
TPK_API int64_t tpk_ball_query_partial_dense_scratch_bytes(int64_t size_x, int64_t size_y, float radius);

/* ---------------------------------------------------------- nearest neighbours ---- */

/*
 * Three nearest known points per unknown point.  unknown (b,n,3), known (b,m,3) ->
 * dist2 (b,n,3) f32 SQUARED distances ascending, idx (b,n,3) int32.
 * Fewer than three known points leave +inf / 0 in the missing slots.
 * Replaces three_nn_kernel_wrapper, cuda/src/interpolate.cpp:5-6
 * (kernel cuda/src/interpolate_gpu.cu:9-65).
 */
TPK_API int tpk_three_nn(int b, int n, int m, const float* unknown, const float* known, float* dist2,
                 int32_t* idx, void* stream);

/*
 * The same search with caller scratch: the known points of every cloud are binned into a
 * uniform grid and a query grows a block of cells around itself until its third-best
 * distance is provably final.  Results are identical to tpk_three_nn bit for bit.
 * scratch: tpk_three_nn_scratch_bytes(b,n,m) bytes, 256-byte aligned; when that returns
 * 0 (fewer than 4096 known points per cloud) or scratch is NULL the call is tpk_three_nn.
 * No counterpart in the reference.
 */
TPK_API int tpk_three_nn_ws(int b, int n, int m, const float* unknown, const float* known, float* dist2,
                            int32_t* idx, void* scratch, int64_t scratch_bytes, void* stream);
TPK_API int64_t tpk_three_nn_scratch_bytes(int b, int n, int m);

/*
 * k nearest support points per query.  support (b,n,3), query (b,m,3) ->
 * idx (b,m,k) int64, dist2 (b,m,k) f32, ascending squared distance evaluated
 * unfused as ((dx*dx)+dy*dy)+dz*dz; equal distances keep index order.
 * The reference has this on the CPU only: dense_knn, cpu/src/knn.cpp:40-59
 * (nanoflann knnSearch, cpu/include/nanoflann.hpp:1367-1375); its Python wrapper
 * raises on CUDA tensors (torch_points_kernels/knn.py:16-17).
 * k > n returns TPK_ERR_INVALID_ARGUMENT (reference: cpu/src/knn.cpp:12-14).
 * 1 <= k <= TPK_KNN_MAX_K.
 */
#define TPK_KNN_MAX_K 64
TPK_API int tpk_knn_dense(int b, int n, int m, int k, const float* support, const float* query,
                  int64_t* idx, float* dist2, void* stream);

/*
 * The same on packed segments: support (size_s,3) / query (size_q,3) with sorted
 * int64 segment ids; idx are positions in the packed support array; a query whose
 * segment holds fewer than k support points gets -1 in the missing idx and dist2
 * slots.  No counterpart in the reference (its kNN is dense only); semantics are
 * dense_knn applied to each segment on its own.
 */
TPK_API int tpk_knn_partial_dense(int64_t size_s, int64_t size_q, int k, const float* support,
                          const float* query, const int64_t* batch_s, const int64_t* batch_q,
                          int64_t* idx, float* dist2, void* stream);

/*
 * Both searches with caller scratch: the support points are binned on a hashed uniform grid
 * (cells keyed by segment or cloud and cell; cell width chosen on the device from the support
 * points' density) and a query grows a block of cells around itself until its k-th best distance
 * is provably final; what the grid cannot settle (sparse regions, segments with fewer than k
 * points, coordinates that are not finite) is answered by the scan.  Results are identical to
 * tpk_knn_dense / tpk_knn_partial_dense bit for bit, equal distances included.  scratch:
 * tpk_knn_*_scratch_bytes(...) bytes, 256-byte aligned; when that returns 0 (small problems) or
 * scratch is NULL the call is the plain one.  The algorithmic counterpart in the reference is its
 * kd-tree, cpu/src/neighbors.cpp:295-339.
 */
TPK_API int tpk_knn_dense_ws(int b, int n, int m, int k, const float* support, const float* query,
                             int64_t* idx, float* dist2, void* scratch, int64_t scratch_bytes, void* stream);
TPK_API int64_t tpk_knn_dense_scratch_bytes(int b, int n, int m, int k);
TPK_API int tpk_knn_partial_dense_ws(int64_t size_s, int64_t size_q, int k, const float* support,
                                     const float* query, const int64_t* batch_s, const int64_t* batch_q,
                                     int64_t* idx, float* dist2, void* scratch, int64_t scratch_bytes,
                                     void* stream);
TPK_API int64_t tpk_knn_partial_dense_scratch_bytes(int64_t size_s, int64_t size_q, int k);

/* ------------------------------------------------------------- interpolation ---- */

/*
 * out[b,c,j] = sum_k points[b,c,idx[b,j,k]] * weight[b,j,k], k = 0..2.
 * points (b,c,m) f32, idx (b,n,3) int32, weight (b,n,3) f32 -> out (b,c,n) f32.
 * Replaces three_interpolate_kernel_wrapper, cuda/src/interpolate.cpp:7-8
 * (kernel cuda/src/interpolate_gpu.cu:78-107).
 */
TPK_API int tpk_three_interpolate(int b, int c, int m, int n, const float* points, const int32_t* idx,
                          const float* weight, float* out, void* stream);

/*
 * grad_points[b,c,idx[b,j,k]] += grad_out[b,c,j] * weight[b,j,k]; grad_points (b,c,m)
 * is fully written (starts from zero inside the call).
 * Replaces three_interpolate_grad_kernel_wrapper, cuda/src/interpolate.cpp:9-10
 * (kernel cuda/src/interpolate_gpu.cu:122-152) and the zero fill of interpolate.cpp:69-70.
 */
TPK_API int tpk_three_interpolate_grad(int b, int c, int n, int m, const float* grad_out,
                               const int32_t* idx, const float* weight, float* grad_points,
                               void* stream);

/* ------------------------------------------------------------------ grouping ---- */

/*
 * out[b,c,p,s] = features[b,c,idx[b,p,s]].  features (b,c,n) f32, idx
 * (b,npoint,nsample) int64 -> out (b,c,npoint,nsample) f32.
 * The reference has no native code here: it expands idx to (b,c,npoint*nsample)
 * int64 and calls torch.gather, torch_points_kernels/torchpoints.py:129-146.
 */
TPK_API int tpk_grouping(int b, int c, int n, int npoint, int nsample, const float* features,
                 const int64_t* idx, float* out, void* stream);

/*
 * grad_features[b,c,idx[b,p,s]] += grad_out[b,c,p,s]; grad_features (b,c,n) is fully
 * written.  Stands in for autograd's scatter-add backward of the gather at
 * torch_points_kernels/torchpoints.py:145.
 */
TPK_API int tpk_grouping_grad(int b, int c, int n, int npoint, int nsample, const float* grad_out,
                      const int64_t* idx, float* grad_features, void* stream);

/*
 * The same with caller scratch of tpk_grouping_grad_scratch_bytes(b,c,n,npoint,nsample) bytes:
 * the index is inverted once per call (positions sorted by target, per tile of positions) and
 * every row is then summed without atomics on the hot path, about twice as fast at the
 * pipeline's shapes.  Results equal tpk_grouping_grad's up to the order of the float additions
 * (neither order is fixed).  scratch NULL, or a shape the plan does not cover (0 bytes asked):
 * tpk_grouping_grad itself.
 */
TPK_API int tpk_grouping_grad_ws(int b, int c, int n, int npoint, int nsample, const float* grad_out,
                                 const int64_t* idx, float* grad_features, void* scratch, int64_t scratch_bytes,
                                 void* stream);
TPK_API int64_t tpk_grouping_grad_scratch_bytes(int b, int c, int n, int npoint, int nsample);

/* ----------------------------------------------------- fused set abstraction ---- */

/*
 * The grouping step of a PointNet++ set-abstraction layer in one call: gathers the centres
 * new_xyz[b,j] = xyz[b, fps_idx[b,j]], runs the dense ball query around them, and writes
 *   out[b, 0:3, j, s]   = xyz[b, idx[b,j,s], :] - new_xyz[b,j,:]      (relative coordinates)
 *   out[b, 3:3+c, j, s] = features[b, :, idx[b,j,s]]
 * i.e. torch.cat([grouping(xyz^T, idx) - new_xyz^T[..., None], grouping(features, idx)], 1)
 * without materialising the parts, bit-identical to that sequence.  xyz (b,n,3), features (b,c,n)
 * (NULL with c = 0), fps_idx (b,m) int32 -> new_xyz (b,m,3), idx (b,m,nsample) int64 (the ball
 * query's result, needed by the backward pass: tpk_grouping_grad on rows 3.. of the gradient),
 * out (b,3+c,m,nsample).  scratch: tpk_sa_group_scratch_bytes(b,n,m,nsample) bytes, 256-byte
 * aligned, required.  The unfused sequence in the reference's callers:
 * torch_points_kernels/torchpoints.py:129-146 (grouping), :171-218 (ball query).
 */
TPK_API int tpk_sa_group(int b, int n, int m, int c, float radius, int nsample, const float* xyz,
                         const float* features, const int32_t* fps_idx, float* new_xyz, int64_t* idx, float* out,
                         void* scratch, int64_t scratch_bytes, void* stream);
TPK_API int64_t tpk_sa_group_scratch_bytes(int b, int n, int m, int nsample);

/*
 * Gradient of tpk_sa_group with respect to the features: grad_out is the whole
 * (b, 3 + c, npoint, nsample) gradient of `out`; rows 3.. of every cloud are read in place
 * (callers of the unfused ops would slice and copy them) and scattered as tpk_grouping_grad_ws
 * does.  The coordinate rows carry no gradient to the features.  scratch:
 * tpk_grouping_grad_scratch_bytes(b, c, n, npoint, nsample) bytes, or NULL for the atomic kernels.
 */
TPK_API int tpk_sa_group_grad(int b, int c, int n, int npoint, int nsample, const float* grad_out,
                              const int64_t* idx, float* grad_features, void* scratch, int64_t scratch_bytes,
                              void* stream);

/* ------------------------------------------------------------------- chamfer ---- */

/*
 * Nearest neighbour in the other cloud, both directions.  xyz1 (b,n,3), xyz2 (b,m,3)
 * -> dist1 (b,n), dist2 (b,m) squared distances, idx1 (b,n), idx2 (b,m) int32;
 * lowest index wins among equal minima.  f32 and f64 variants, as the reference
 * dispatches both (cuda/src/chamfer_dist_gpu.cu:167-176).
 * Replaces chamfer_dist_kernel_wrapper, cuda/include/chamfer_dist.h:10
 * (kernel cuda/src/chamfer_dist_gpu.cu:8-155).
 */
TPK_API int tpk_chamfer_dist_f32(int b, int n, const float* xyz1, int m, const float* xyz2, float* dist1,
                         float* dist2, int32_t* idx1, int32_t* idx2, void* stream);
TPK_API int tpk_chamfer_dist_f64(int b, int n, const double* xyz1, int m, const double* xyz2,
                         double* dist1, double* dist2, int32_t* idx1, int32_t* idx2, void* stream);

/*
 * The float32 forward pass with caller scratch: each direction searches the uniform grid of
 * the other cloud (nearest point by (distance, index), i.e. the lowest index among equal
 * distances, as the reference's strict-'<' scan keeps it); results are identical to
 * tpk_chamfer_dist_f32 bit for bit.  scratch: tpk_chamfer_dist_scratch_bytes(b,n,m) bytes,
 * 256-byte aligned; when that returns 0 (both clouds below 1024 points) or scratch is NULL
 * the call is tpk_chamfer_dist_f32.  No counterpart in the reference.
 */
TPK_API int tpk_chamfer_dist_f32_ws(int b, int n, const float* xyz1, int m, const float* xyz2, float* dist1,
                                    float* dist2, int32_t* idx1, int32_t* idx2, void* scratch,
                                    int64_t scratch_bytes, void* stream);
TPK_API int64_t tpk_chamfer_dist_scratch_bytes(int b, int n, int m);

/*
 * Gradient of both directions w.r.t. both clouds; grad_xyz1 (b,n,3) and grad_xyz2
 * (b,m,3) are fully written.
 * Replaces chamfer_dist_grad_kernel_wrapper, cuda/include/chamfer_dist.h:12-15
 * (kernel cuda/src/chamfer_dist_gpu.cu:186-245).
 */
TPK_API int tpk_chamfer_dist_grad_f32(int b, int n, const float* xyz1, int m, const float* xyz2,
                              const int32_t* idx1, const int32_t* idx2, const float* grad_dist1,
                              const float* grad_dist2, float* grad_xyz1, float* grad_xyz2,
                              void* stream);
TPK_API int tpk_chamfer_dist_grad_f64(int b, int n, const double* xyz1, int m, const double* xyz2,
                              const int32_t* idx1, const int32_t* idx2, const double* grad_dist1,
                              const double* grad_dist2, double* grad_xyz1, double* grad_xyz2,
                              void* stream);

/* -------------------------------------------------- GRNet ops (next to chamfer) ---- */

/*
 * Point cloud -> density grid by trilinear weights.  ptcloud (b,n_pts,3), already scaled to grid
 * units; the grid spans [min, max] per axis (integers passed as float, as the reference does):
 * len = max - min + 1 vertices.  -> grid (b, len_x*len_y*len_z), fully written (starts from
 * zero inside the call); grid_pt_weights (b,n_pts,8,3) and grid_pt_indexes (b,n_pts,8) int32 are
 * the eight vertices' axis weights 1 - |x - x0| and flat indices, kept for the backward pass.
 * A vertex outside the grid gets index -1 and contributes nothing (the reference writes out of
 * bounds there) and sets TPK_STATUS_BAD_INDEX.  f32 and f64, as the reference dispatches both.
 * Replaces gridding_kernel_warpper, cuda/src/gridding_gpu.cu:163-197 (kernel :28-161).
 */
TPK_API int tpk_gridding_f32(int b, int n_pts, float min_x, float max_x, float min_y, float max_y, float min_z,
                             float max_z, const float* ptcloud, float* grid, float* grid_pt_weights,
                             int32_t* grid_pt_indexes, void* stream);
TPK_API int tpk_gridding_f64(int b, int n_pts, float min_x, float max_x, float min_y, float max_y, float min_z,
                             float max_z, const double* ptcloud, double* grid, double* grid_pt_weights,
                             int32_t* grid_pt_indexes, void* stream);

/*
 * grad_ptcloud (b,n_pts,3) from grad_grid (b,n_grid_vertices): per axis the sum over the eight
 * vertices of +-grad * (the other two weights), in the reference's order (bit-identical).
 * Replaces gridding_grad_kernel_warpper, cuda/src/gridding_gpu.cu:306-333 (kernel :199-304).
 */
TPK_API int tpk_gridding_grad_f32(int b, int n_pts, int64_t n_grid_vertices, const float* grid_pt_weights,
                                  const int32_t* grid_pt_indexes, const float* grad_grid, float* grad_ptcloud,
                                  void* stream);
TPK_API int tpk_gridding_grad_f64(int b, int n_pts, int64_t n_grid_vertices, const double* grid_pt_weights,
                                  const int32_t* grid_pt_indexes, const double* grad_grid, double* grad_ptcloud,
                                  void* stream);

/*
 * Features of the (2*neighborhood_size)^3 grid vertices around every point.  ptcloud (b,n_pts,3)
 * in grid units, cubic_features (b,channels,scale,scale,scale) -> point_features
 * (b,n_pts,n_vertices,channels), fully written (0 for vertices outside the grid), and
 * grid_pt_indexes (b,n_pts,n_vertices) int32 (-1 outside the grid).
 * Replaces cubic_feature_sampling_kernel_wrapper, cuda/src/cubic_feature_sampling_gpu.cu:99-128.
 */
TPK_API int tpk_cubic_feature_sampling_f32(int b, int n_pts, int channels, int scale, int neighborhood_size,
                                           const float* ptcloud, const float* cubic_features,
                                           float* point_features, int32_t* grid_pt_indexes, void* stream);
TPK_API int tpk_cubic_feature_sampling_f64(int b, int n_pts, int channels, int scale, int neighborhood_size,
                                           const double* ptcloud, const double* cubic_features,
                                           double* point_features, int32_t* grid_pt_indexes, void* stream);

/*
 * Scatter-add of grad_point_features into grad_cubic_features (b,channels,scale^3), fully written;
 * grad_ptcloud (b,n_pts,3) is zero (floor and ceil are flat); either output may be NULL.
 * Replaces cubic_feature_sampling_grad_kernel_wrapper, cubic_feature_sampling_gpu.cu:179-213.
 */
TPK_API int tpk_cubic_feature_sampling_grad_f32(int b, int n_pts, int channels, int scale, int neighborhood_size,
                                                const float* grad_point_features, const int32_t* grid_pt_indexes,
                                                float* grad_ptcloud, float* grad_cubic_features, void* stream);
TPK_API int tpk_cubic_feature_sampling_grad_f64(int b, int n_pts, int channels, int scale, int neighborhood_size,
                                                const double* grad_point_features, const int32_t* grid_pt_indexes,
                                                double* grad_ptcloud, double* grad_cubic_features, void* stream);

/* ------------------------------------------- clustering and instance metrics ---- */

/*
 * `rounds` rounds of label propagation for region growing.  neighbours (n,nsample) int64: the
 * lists a partial_dense ball query of the points against themselves returns (-1 ends a list);
 * labels (n) int32, initialised by the caller to 0..n-1.  A round pushes every point's label to
 * the points it lists (minimum wins) and shortens label chains.  *changed (device int32, zeroed
 * by the caller) is set to 1 by any round that changed a label: repeat until it stays 0.  At the
 * fixed point labels[v] is the smallest index that reaches v along the lists, which is the seed
 * of the cluster the reference's sequential traversal puts v in
 * (torch_points_kernels/cluster.py:8-37).
 */
TPK_API int tpk_grow_labels_step(int64_t n, int nsample, const int64_t* neighbours, int32_t* labels,
                                 int32_t* changed, int rounds, void* stream);

/*
 * IoU of every proposal with every ground-truth instance of its sample; proposals_iou
 * (n_proposals,total_gt_instances) f32 is fully written (0 for other samples' instances).
 * Arguments as instance_iou_kernel_wrapper, cuda/src/metrics_gpu.cu:50-62 (kernel :9-43), plus
 * n_points (length of instance_labels and batch) so that indices can be checked.
 */
TPK_API int tpk_instance_iou(int n_proposals, int64_t total_gt_instances, int64_t max_gt_instances,
                             int64_t n_points, const int64_t* num_gt_instances, const int64_t* proposals_idx,
                             const int64_t* proposals_offset, const int64_t* instance_labels,
                             const int64_t* offset_num_gt_instances, const int64_t* batch,
                             const int64_t* instance_pointnum, float* proposals_iou, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TPK_B200_H */
