/*
 * tk3d.h -- C ABI of libtk3d_b200.so: the torkit3d neighbour-search / sampling operators,
 * hand-written for NVIDIA B200 (sm_100a).
 *
 * These entry points are what the reference's Python operators bind instead of the nine functions
 * of its pybind11 module `torkit3d._C` (torkit3d/csrc/torkit3d.cpp:13-21).  Each declaration names
 * the reference prototype it replaces.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer into the current CUDA device's memory unless stated;
 *     tensors are dense, row-major ("contiguous") in the shapes written beside them;
 *   - `dtype` is TK3D_F32 or TK3D_F64 and applies to every `void*` floating-point tensor;
 *     indices are int64 unless an entry point says otherwise;
 *   - the caller allocates and owns every output and scratch buffer; the library allocates no
 *     device memory and never synchronises the host.  Between calls it keeps only per-device
 *     caches of facts that cannot change (the SM count, which kernels already had their
 *     shared-memory limit raised, the address of the array behind tk3d_fps_static_scratch);
 *     these are valid for the lifetime of the device's primary context, i.e. until the process
 *     ends or the device is reset;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default
 *     stream) of the device that is current on the calling thread;
 *   - every output element is written by the call (no pre-zeroing needed);
 *   - the return value is TK3D_OK or an error code; argument errors are detected before anything
 *     is launched.  Nothing throws.  tk3d_strerror() names a code, tk3d_last_error() gives the
 *     calling thread's most recent detailed message (including the CUDA error text for
 *     TK3D_ERR_CUDA);
 *   - the squared distance is ((dx*dx + dy*dy) + dz*dz) with dx = ref.x - query.x, every
 *     operation rounded on its own (no fused multiply-add), so indices are reproducible bit for
 *     bit; ties always go to the lowest index.
 */
#ifndef TK3D_H_
#define TK3D_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TK3D_F32 0
#define TK3D_F64 1

/* type of an index tensor, for the *_layout entry points */
#define TK3D_I64 0
#define TK3D_I32 1

#define TK3D_OK 0
#define TK3D_ERR_NULL 1        /* a required pointer is NULL */
#define TK3D_ERR_SHAPE 2       /* a size is negative, or too large for the implementation */
#define TK3D_ERR_K 3           /* k / num_samples out of range for the given cloud */
#define TK3D_ERR_DTYPE 4       /* dtype is neither TK3D_F32 nor TK3D_F64 */
#define TK3D_ERR_CUDA 5        /* a CUDA runtime call or kernel launch failed */
#define TK3D_ERR_SCRATCH 6     /* scratch buffer missing or too small */
#define TK3D_ERR_UNSUPPORTED 7 /* valid request the library does not implement */

/* Library version (major*10000 + minor*100 + patch). */
int tk3d_version(void);
/* Static description of an error code. */
const char *tk3d_strerror(int code);
/* Detailed message of the calling thread's last failing call ("" if none). */
const char *tk3d_last_error(void);

/*
 * Chamfer forward, both directions in one call.
 * Replaces chamfer_distance_forward_cuda (torkit3d/csrc/include/chamfer_distance.h:6-8,
 * torkit3d/csrc/cuda/chamfer_distance_kernel.cu:91-151).
 *   xyz1 [B,N1,3], xyz2 [B,N2,3]                          in
 *   dist1 [B,N1], idx1 [B,N1], dist2 [B,N2], idx2 [B,N2]  out (squared distance, arg-min; an empty
 *                                                         partner cloud gives +inf / -1)
 *   sums  [2] float64, optional (NULL to skip)            out: sum(dist1), sum(dist2) over the call,
 *         accumulated in the kernel epilogue so a loss needs no further reduction pass.
 */
int tk3d_chamfer_fwd(const void *xyz1, const void *xyz2, int64_t B, int64_t N1, int64_t N2, void *dist1,
                     int64_t *idx1, void *dist2, int64_t *idx2, double *sums, int dtype, void *stream);

/*
 * Chamfer backward: gradients w.r.t. both clouds.
 * Replaces chamfer_distance_backward_cuda (torkit3d/csrc/include/chamfer_distance.h:10-16,
 * torkit3d/csrc/cuda/chamfer_distance_kernel.cu:200-274).
 *   grad_dist1 [B,N1], grad_dist2 [B,N2], xyz1, xyz2, idx1, idx2   in
 *   grad_xyz1 [B,N1,3], grad_xyz2 [B,N2,3]                         out
 * grad_xyz1[i] = 2 g1[i] (p1_i - p2_idx1[i]) - sum_{j: idx2[j]=i} 2 g2[j] (p2_j - p1_i), and the
 * mirror image for grad_xyz2.  The scattered terms use floating-point atomics.  Indices outside
 * [0, partner size) contribute nothing.
 */
int tk3d_chamfer_bwd(const void *grad_dist1, const void *grad_dist2, const void *xyz1, const void *xyz2,
                     const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1, int64_t N2,
                     void *grad_xyz1, void *grad_xyz2, int dtype, void *stream);

/*
 * Mean chamfer loss helpers (no counterpart in the reference, whose callers spell these steps as
 * element-wise PyTorch expressions): with sums = [sum(dist1), sum(dist2)] from tk3d_chamfer_fwd
 * (all-reduced over the ranks of a sharded batch), count1 = global number of cloud-1 points and
 * count2 likewise,
 *   tk3d_chamfer_mean_loss   loss[0] = sums[0]/count1 + sums[1]/count2          (one element of `dtype`)
 *   tk3d_chamfer_bwd_mean    gradients of that loss: tk3d_chamfer_bwd with the per-point upstream
 *                            gradients grad_loss[0]/count1 and grad_loss[0]/count2 (grad_loss is a
 *                            device scalar of `dtype`), without materialising them.
 */
int tk3d_chamfer_mean_loss(const double *sums, double count1, double count2, void *loss, int dtype, void *stream);
int tk3d_chamfer_bwd_mean(const void *grad_loss, double count1, double count2, const void *xyz1, const void *xyz2,
                          const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1, int64_t N2,
                          void *grad_xyz1, void *grad_xyz2, int dtype, void *stream);

/*
 * Brute-force k nearest neighbours.
 * Replaces knn_distance_cuda (torkit3d/csrc/include/knn_distance.h:7-11,
 * torkit3d/csrc/cuda/knn_distance_kernel.cu:187-298), both of its `version`s.
 *   query [B,N1,3], key [B,N2,3]                in;  requires 1 <= k <= N2
 *   distance [B,N1,k] (squared), index [B,N1,k]  out; each row is sorted ascending by
 *                                                (distance, index).  (The reference leaves rows in
 *                                                an unspecified order; the retained set is equal.)
 */
int tk3d_knn(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k, void *distance,
             int64_t *index, int dtype, void *stream);

/*
 * Farthest point sampling, first sample = point 0, lowest index among exact maxima.
 * Replaces sample_farthest_points_cuda (torkit3d/csrc/include/sample_farthest_points.h:6-8,
 * torkit3d/csrc/cuda/sample_farthest_points_kernel.cu:106-165).
 *   points [B,N,3]   in;  requires 1 <= num_samples <= N
 *   index  [B,S]     out
 *   scratch          device buffer of at least tk3d_fps_scratch_bytes(B,N,dtype) bytes (the running
 *                    minimum distance of clouds too large to keep on chip); may be NULL when that
 *                    function returns 0.  Contents on entry are ignored.  (float32 clouds of 16385
 *                    to 262144 points and float64 clouds of 8193 to 131072 points run on a
 *                    thread-block cluster and leave it untouched; it is
 *                    what the call falls back on when the device refuses the cluster launch.)
 */
size_t tk3d_fps_scratch_bytes(int64_t B, int64_t N, int dtype);
int tk3d_fps(const void *points, int64_t B, int64_t N, int64_t num_samples, int64_t *index, void *scratch,
             size_t scratch_bytes, int dtype, void *stream);

/*
 * Farthest point sampling without any caller-provided or freshly allocated scratch memory.
 * It has no counterpart in the reference (whose sample_farthest_points_cuda allocates its scratch
 * tensor on every call).  It is meant for callers that cannot allocate device memory where they
 * sample: inside a region where their framework forbids allocation, with a memory budget fixed at
 * start-up, or from plain C without an allocator at hand.
 *   points [B,N,3] in;  index [B,S] out;  same result as tk3d_fps, bit for bit.
 * The running minimum distances live in a fixed 8 MiB array inside the library image
 * (tk3d_fps_static_scratch_capacity() bytes; every GPU that loads the library holds one copy until
 * the process exits), so B*N may not exceed capacity/4 (fp32: 2,097,152) or capacity/8 (fp64:
 * 1,048,576) elements; larger problems return TK3D_ERR_SCRATCH and must use tk3d_fps.
 * The call allocates nothing and frees nothing.  The first call on each device looks up the
 * array's device address (a synchronous CUDA runtime query), so make that first call outside any
 * stream capture.  All calls on one device share the one array: two calls whose kernels can run
 * at the same time on that device (different streams, or different host threads) corrupt each
 * other -- order them on one stream or with events.  Nothing needs clearing between calls.
 * Every size runs the streaming kernel; for fp32 clouds of at most 16384 points (fp64: 8192) tk3d_fps
 * needs no scratch at all (pass NULL) and is faster.
 */
size_t tk3d_fps_static_scratch_capacity(void);
int tk3d_fps_static_scratch(const void *points, int64_t B, int64_t N, int64_t num_samples, int64_t *index,
                            int dtype, void *stream);

/*
 * Ball query: the first k key indices (ascending) with squared distance < radius*radius (radius is
 * squared in `dtype` after conversion from float); short rows are padded with their first hit, rows
 * without a hit are all -1.
 * Replaces ball_query_cuda (torkit3d/csrc/include/ball_query.h:6-10,
 * torkit3d/csrc/cuda/ball_query_kernel.cu:105-173).
 *   query [B,N1,3], key [B,N2,3]   in;  k >= 1
 *   index [B,N1,k]                 out
 */
int tk3d_ball_query(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, float radius,
                    int64_t k, int64_t *index, int dtype, void *stream);

/*
 * group_points forward: out[b,c,m,j] = in[b,c,index[b,m,j]].
 * Replaces group_points_forward_cuda (torkit3d/csrc/include/group_points.h:6-8,
 * torkit3d/csrc/cuda/group_points_kernel.cu:8-31).
 *   in [B,C,N1], index [B,N2,K]   in
 *   out [B,C,N2,K]                out
 * An index outside [0,N1) yields 0 (the reference faults the device instead); when `status` is not
 * NULL, bit 0 of *status (a device int32 the caller zeroed) is set if any such index was seen.
 *   scratch   optional device buffer of tk3d_group_fwd_scratch_bytes(...) bytes.  When that function
 *             returns non-zero and the buffer is given, the features are first transposed into it
 *             ([B,N1,C]) so that every gather reads whole contiguous rows -- several times faster
 *             when the output is much larger than the features.  Without it (NULL) the call gathers
 *             from the native layout.  Results are identical.  The function returns 0 for the
 *             shapes served by the channel-row kernel (fp32, N1 a multiple of 4 between 256 and
 *             24576, at least 1024 index entries per cloud), which stages every channel's N1
 *             features in shared memory and needs no scratch.
 */
size_t tk3d_group_fwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype);
int tk3d_group_fwd(const void *in, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K,
                   void *out, int32_t *status, void *scratch, size_t scratch_bytes, int dtype, void *stream);

/*
 * group_points backward: grad_in[b,c,index[b,m,j]] += grad_out[b,c,m,j] (grad_in is zeroed first).
 * Replaces group_points_backward_cuda (torkit3d/csrc/include/group_points.h:10-13,
 * torkit3d/csrc/cuda/group_points_kernel.cu:67-114).  Out-of-range indices are skipped and
 * reported through `status` as above.  `scratch` (optional, tk3d_group_bwd_scratch_bytes(...) bytes): the
 * gradients are accumulated with 16-byte vector atomics into a transposed [B,N1,C] buffer and transposed
 * back, instead of scattered single-float atomics.  Its contents on entry are ignored.
 */
size_t tk3d_group_bwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype);
int tk3d_group_bwd(const void *grad_out, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2,
                   int64_t K, void *grad_in, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                   void *stream);

/*
 * Feature interpolation forward: out[b,c,m] = sum_{i<K} in[b,c,index[b,m,i]] * weight[b,m,i].
 * Replaces interpolate_forward_cuda (torkit3d/csrc/include/interpolate.h:7-10,
 * torkit3d/csrc/cuda/interpolate_kernel.cu:49-103).  K must be 3, as in the reference.
 *   in [B,C,N1], index [B,N2,3], weight [B,N2,3]   in
 *   out [B,C,N2]                                   out
 *   scratch   optional, tk3d_interp_fwd_scratch_bytes(...) bytes: same role as in tk3d_group_fwd.
 */
size_t tk3d_interp_fwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int dtype);
int tk3d_interp_fwd(const void *in, const int64_t *index, const void *weight, int64_t B, int64_t C, int64_t N1,
                    int64_t N2, int64_t K, void *out, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                    void *stream);

/*
 * Feature interpolation backward (w.r.t. the features only):
 * grad_in[b,c,index[b,m,i]] += grad_out[b,c,m] * weight[b,m,i] (grad_in is zeroed first).
 * Replaces interpolate_backward_cuda (torkit3d/csrc/include/interpolate.h:12-16,
 * torkit3d/csrc/cuda/interpolate_kernel.cu:147-201).  `scratch` (optional,
 * tk3d_interp_bwd_scratch_bytes(...) bytes) has the same role as in tk3d_group_bwd.
 */
size_t tk3d_interp_bwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int dtype);
int tk3d_interp_bwd(const void *grad_out, const int64_t *index, const void *weight, int64_t B, int64_t C,
                    int64_t N1, int64_t N2, int64_t K, void *grad_in, int32_t *status, void *scratch,
                    size_t scratch_bytes, int dtype, void *stream);

/*
 * Features kept as rows.  The gathers above read rows of a [B,N,C] copy of the features, which they
 * build in `scratch` on every call.  A caller that gathers from the same features more than once --
 * query slabs of one scene, several groupings of one cloud, forward passes between two updates of
 * the features -- builds that copy once with tk3d_feature_rows and hands it to the *_rows forms,
 * which then launch the gather alone.  No counterpart in the reference, whose kernels read the
 * [B,C,N] tensor directly (torkit3d/csrc/cuda/group_points_kernel.cu:8-31, interpolate_kernel.cu:8-47).
 * float32 only, C <= 512, B <= 65535; index_dtype TK3D_I64 or TK3D_I32.
 *   tk3d_feature_rows:    feature [B,C,N] in;  rows [B,N,C] out (B*N*C*4 bytes)
 *   tk3d_interp_fwd_rows: rows [B,N1,C], index [B,N2,3], weight [B,N2,3] in;  out [B,C,N2]
 *   tk3d_group_fwd_rows:  rows [B,N1,C], index [B,N2,K] in;  out [B,C,N2,K]
 */
int tk3d_feature_rows(const void *feature, int64_t B, int64_t C, int64_t N, void *rows, int dtype, void *stream);
int tk3d_interp_fwd_rows(const void *rows, const void *index, int index_dtype, const void *weight, int64_t B,
                         int64_t C, int64_t N1, int64_t N2, int64_t K, void *out, int32_t *status, int dtype,
                         void *stream);
int tk3d_group_fwd_rows(const void *rows, const void *index, int index_dtype, int64_t B, int64_t C, int64_t N1,
                        int64_t N2, int64_t K, void *out, int32_t *status, int dtype, void *stream);

/*
 * Inverse squared-distance weights of the k nearest neighbours:
 * inv = 1 / max(d, 1e-10), weight = inv / sum(inv) over the last axis.
 * Replaces the element-wise PyTorch expressions of FeatureInterpolator.forward
 * (torkit3d/layers/pointnet2.py:128-130).
 *   distance [rows,k] (squared) in;  weight [rows,k] out;  1 <= k <= 8
 */
int tk3d_three_nn_weight(const void *distance, int64_t rows, int64_t k, void *weight, int dtype, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Layout variants of the operators above.  The reference's Python operators copy channel-first
 * clouds with .transpose(1, 2).contiguous() before every call (torkit3d/ops/ball_query.py:32-36,
 * torkit3d/ops/sample_farthest_points.py:28-30, torkit3d/ops/knn_points.py:40-44,
 * torkit3d/ops/chamfer_distance.py:49-52); these entry points read the [B,3,N] tensor in place.
 *   xyz_channel_first  0 = every xyz argument is [B,N,3] (exactly the plain entry point),
 *                      1 = every xyz argument -- and every xyz gradient -- is [B,3,N]
 *   index_dtype        TK3D_I64 (the reference's type) or TK3D_I32 (half the index bytes; every
 *                      index fits because clouds are limited to 2^30 points); `index` then points
 *                      at int32 elements of the same shape
 * Results are identical to the plain entry points, element for element.
 */
int tk3d_chamfer_fwd_layout(const void *xyz1, const void *xyz2, int64_t B, int64_t N1, int64_t N2,
                            int xyz_channel_first, void *dist1, int64_t *idx1, void *dist2, int64_t *idx2,
                            double *sums, int dtype, void *stream);
int tk3d_chamfer_bwd_layout(const void *grad_dist1, const void *grad_dist2, const void *xyz1, const void *xyz2,
                            const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1, int64_t N2,
                            int xyz_channel_first, void *grad_xyz1, void *grad_xyz2, int dtype, void *stream);
int tk3d_chamfer_bwd_mean_layout(const void *grad_loss, double count1, double count2, const void *xyz1,
                                 const void *xyz2, const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1,
                                 int64_t N2, int xyz_channel_first, void *grad_xyz1, void *grad_xyz2, int dtype,
                                 void *stream);
int tk3d_knn_layout(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                    int xyz_channel_first, void *distance, void *index, int index_dtype, int dtype, void *stream);
int tk3d_fps_layout(const void *points, int64_t B, int64_t N, int64_t num_samples, int xyz_channel_first,
                    int64_t *index, void *scratch, size_t scratch_bytes, int dtype, void *stream);
int tk3d_ball_query_layout(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, float radius,
                           int64_t k, int xyz_channel_first, void *index, int index_dtype, int dtype, void *stream);
/* tk3d_group_fwd reading an index tensor of `index_dtype` (e.g. the int32 output of the two calls
 * above); everything else as tk3d_group_fwd. */
int tk3d_group_fwd_layout(const void *in, const void *index, int index_dtype, int64_t B, int64_t C, int64_t N1,
                          int64_t N2, int64_t K, void *out, int32_t *status, void *scratch, size_t scratch_bytes,
                          int dtype, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Fused front ends of the PointNet++ layers that call the operators above.  They replace Python
 * glue of the reference, not entry points of its extension; fp32 only.
 * `xyz_channel_first` selects the coordinate layout of every xyz argument of the call:
 * 0 = [B,N,3] (the layout of the operators above), 1 = [B,3,N] (the layout the reference's layers
 * receive and transpose with .transpose(1,2).contiguous() before every operator call).
 */

/*
 * Farthest point sampling that also returns the sampled coordinates.
 * Replaces sample_farthest_points(points, S, transpose=True) followed by
 * batch_index_select(points, fps_index, dim=2) (torkit3d/models/classification/pointnet2.py:73-74,
 * torkit3d/nn/functional.py:34-69).
 *   points  [B,N,3] or [B,3,N] in;  index [B,S] out (as tk3d_fps, bit for bit)
 *   sampled [B,S,3] or [B,3,S] out, same layout and dtype as points
 *   scratch as for tk3d_fps.
 */
int tk3d_fps_gather(const void *points, int64_t B, int64_t N, int64_t num_samples, int xyz_channel_first,
                    int64_t *index, void *sampled, void *scratch, size_t scratch_bytes, int dtype, void *stream);

/*
 * Set-abstraction grouping: ball query + group_points of the features + group_points of the
 * coordinates + centring + concatenation, i.e. everything SetAbstraction.forward does before its
 * MLP (torkit3d/layers/pointnet2.py:43-58 with query_neighbor = BallQuery), in two launches (one
 * transpose of the features into `scratch`, one fused kernel).
 *   points    [B,N,3]|[B,3,N]  in   coordinates of the N input points ("in_xyz")
 *   centroids [B,M,3]|[B,3,M]  in   coordinates of the M group centres ("out_xyz")
 *   feature   [B,C,N]          in   may be NULL when C == 0
 *   out       [B,C+3,M,K]      out  channels [0,C): feature[b,c,index[b,m,k]];
 *                                   channels [C,C+3): points[b,index[b,m,k],:] - centroids[b,m,:]
 *                                   ([B,C,M,K] when use_xyz == 0)
 *   index32   [B,M,K] int32    out  optional (NULL to skip): the ball-query result, identical to
 *                                   tk3d_ball_query's; the backward needs it
 *   status    int32            in/out optional: bit 0 is OR-ed in when a centre has no neighbour
 *                                   (its K entries are -1; its feature channels are 0 and its
 *                                   coordinate channels are -centroid)
 *   scratch   tk3d_sa_group_scratch_bytes(...) bytes, required when C > 0
 * tk3d_sa_group_supported() tells whether the shape is served (fp32, C <= 512, 1 <= K <= 128);
 * otherwise compose tk3d_ball_query and tk3d_group_fwd.
 */
int tk3d_sa_group_supported(int64_t B, int64_t C, int64_t N, int64_t M, int64_t K, int dtype);
size_t tk3d_sa_group_scratch_bytes(int64_t B, int64_t C, int64_t N, int64_t M, int64_t K, int dtype);
int tk3d_sa_group_fwd(const void *points, const void *centroids, const void *feature, int64_t B, int64_t C,
                      int64_t N, int64_t M, float radius, int64_t K, int xyz_channel_first, int use_xyz, void *out,
                      int32_t *index32, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                      void *stream);

/*
 * Backward of tk3d_sa_group_fwd.  grad_out is the gradient of `out` ([B,C+3,M,K], dense).
 *   grad_feature   [B,C,N]            out, optional: scatter-add of the first C channels
 *   grad_points    like points        out, optional: scatter-add of the coordinate channels
 *   grad_centroids like centroids     out, optional: minus the sum over K of the coordinate channels
 * Each output is fully written (zeroed first where it accumulates).  `scratch` as in the forward.
 */
int tk3d_sa_group_bwd(const void *grad_out, const int32_t *index32, int64_t B, int64_t C, int64_t N, int64_t M,
                      int64_t K, int xyz_channel_first, int use_xyz, void *grad_feature, void *grad_points,
                      void *grad_centroids, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                      void *stream);

/*
 * Feature propagation front end: three nearest keys of every query + inverse-distance weights +
 * weighted gather, i.e. FeatureInterpolator.forward (torkit3d/layers/pointnet2.py:114-133), in
 * three launches (3-NN with the weights computed in its epilogue, transpose, gather).
 *   query_xyz   [B,Nq,3]|[B,3,Nq] in;  key_xyz [B,Nk,3]|[B,3,Nk] in (Nk >= 3)
 *   key_feature [B,C,Nk] in;  out [B,C,Nq] out
 *   index32 [B,Nq,3] int32 out, weight [B,Nq,3] out: the neighbours (ascending distance, ties to
 *                    the lower index, as tk3d_knn) and w_i = (1/max(d_i,eps)) / sum_j (1/max(d_j,eps))
 *   scratch     tk3d_three_nn_interp_scratch_bytes(...) bytes, required when C > 0
 * The backward (w.r.t. the features, as in the reference) takes index32 and weight back.
 */
size_t tk3d_three_nn_interp_scratch_bytes(int64_t B, int64_t C, int64_t Nq, int64_t Nk, int dtype);
int tk3d_three_nn_interp_fwd(const void *query_xyz, const void *key_xyz, const void *key_feature, int64_t B,
                             int64_t C, int64_t Nq, int64_t Nk, int xyz_channel_first, float eps, void *out,
                             int32_t *index32, void *weight, int32_t *status, void *scratch, size_t scratch_bytes,
                             int dtype, void *stream);
int tk3d_three_nn_interp_bwd(const void *grad_out, const int32_t *index32, const void *weight, int64_t B, int64_t C,
                             int64_t Nq, int64_t Nk, void *grad_feature, int32_t *status, void *scratch,
                             size_t scratch_bytes, int dtype, void *stream);

/*
 * EdgeConv edge features: group_points of the key features + subtraction of the query feature +
 * concatenation with the broadcast query feature, i.e. get_edge_feature_custom
 * (torkit3d/ops/edge_conv.py:73-93), in one pass over the output.  fp32 and fp64.
 *   query_feature [B,C,N1] in;  key_feature [B,C,N2] in;  index [B,N1,K] int64 in
 *   out [B,2C,N1,K] out ([B,C,N1,K] when include_query == 0):
 *       out[b,c,n,k]   = key_feature[b,c,index[b,n,k]] - query_feature[b,c,n]
 *       out[b,C+c,n,k] = query_feature[b,c,n]
 *   An index outside [0,N2) gathers 0 and ORs bit 0 into *status (optional).
 *   scratch (optional, tk3d_edge_feature_scratch_bytes(...) bytes; 0 = no fast path for the shape):
 *   same role as in tk3d_group_fwd / tk3d_group_bwd.
 * Backward: grad_key[b,c,index[b,n,k]] += grad_out[b,c,n,k];
 *           grad_query[b,c,n] = sum_k (grad_out[b,C+c,n,k] - grad_out[b,c,n,k]).
 * Either gradient pointer may be NULL; each one given is fully written.
 */
size_t tk3d_edge_feature_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype);
int tk3d_edge_feature_fwd(const void *query_feature, const void *key_feature, const int64_t *index, int64_t B,
                          int64_t C, int64_t N1, int64_t N2, int64_t K, int include_query, void *out,
                          int32_t *status, void *scratch, size_t scratch_bytes, int dtype, void *stream);
int tk3d_edge_feature_bwd(const void *grad_out, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2,
                          int64_t K, int include_query, void *grad_query, void *grad_key, int32_t *status,
                          void *scratch, size_t scratch_bytes, int dtype, void *stream);

/*
 * Brute-force k nearest neighbours in a C-dimensional feature space (float32 only, k <= 128).
 * Replaces the cdist + topk formulation of torkit3d/ops/native.py:4-30 where DGCNN builds its
 * dynamic graph on features (torkit3d/models/classification/dgcnn.py:58-61).
 *   query [B,C,N1], key [B,C,N2] in  (channel_first != 0), or [B,N1,C], [B,N2,C] (channel_first == 0);
 *                                    requires 1 <= k <= N2
 *   distance [B,N1,k] out: SQUARED distances, acc = fma(d_c, d_c, acc) over c = 0..C-1 in order with
 *                          d_c = key_c - query_c (cdist's matrix-product rounding is unspecified)
 *   index [B,N1,k] out;    each row sorted ascending by (distance, index)
 */
int tk3d_feature_knn(const void *query, const void *key, int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t k,
                     int channel_first, void *distance, int64_t *index, int dtype, void *stream);

/*
 * Range-checked build.  libtk3d_b200_bounds.so is this library compiled with -DTK3D_BOUNDS: every
 * coordinate load and every index-tensor access of the operators is checked against the extent of
 * its tensor, a violation is counted and redirected to element 0.  tk3d_bounds_violations()
 * synchronises the device and returns the number of violations since the library was loaded; in the
 * regular build, which carries no checks, it returns -1.  (The reference's only run-time checks on
 * this path are the device-side asserts of torkit3d/csrc/cuda/group_points_kernel.cu:62 and
 * interpolate_kernel.cu:40,141, which abort the CUDA context.)
 */
long long tk3d_bounds_violations(void);

/*
 * Bounded waits.  One kind of kernel waits for other thread blocks: farthest point sampling of
 * float32 clouds of 4097 to 262144 points (float64: 2049 to 131072) runs on a thread-block cluster
 * whose warps wait, in every step,
 * for the candidates of all other warps of the cluster (an mbarrier in shared memory).  Every such
 * wait gives up after one second; the warp then stops, which makes the other warps of its cluster
 * give up as well, index[b][i..] of that cloud is set to -1 from the first step that was not
 * completed, and the kernel ends normally: the CUDA context stays usable.
 * tk3d_fps_expired_waits() synchronises nothing itself beyond a 4-byte copy from the device and
 * returns the number of waits that gave up on the current device since the library was loaded
 * (0 in normal operation; -1 if the counter cannot be read).
 *
 * tk3d_diag_fps_wait_limit() is a diagnostic with no counterpart in the reference, for testing
 * that path without a fault: it runs the cluster kernel on points [B,N,3] (float32, 4096 < N <=
 * 131072) with the waits limited to limit_ms (1..1000) and with one warp of every cluster sending
 * nothing in step drop_step (>= 1; -1: every warp sends, i.e. a normal run), so that every wait of
 * that step runs out.  index [B,num_samples] then holds the regular result up to drop_step - 1
 * and -1 from drop_step on.
 */
long long tk3d_fps_expired_waits(void);
int tk3d_diag_fps_wait_limit(const void *points, int64_t B, int64_t N, int64_t num_samples, int64_t *index,
                             int64_t limit_ms, int64_t drop_step, void *stream);

/*
 * Diagnostic with no counterpart in the reference: launches a kernel of dependent FP32 fused
 * multiply-add chains (`iters` x 64 FMAs per thread, 8 blocks of 256 threads per SM) on `stream`.
 * *flop (a HOST double, optional) receives the number of floating-point operations the launch
 * performs; timing the launch with CUDA events gives the device's sustained FP32 FMA rate, the
 * roofline of the distance kernels.  `sink` is a device float that is never actually written.
 */
int tk3d_diag_ffma(int64_t iters, float *sink, double *flop, void *stream);

/*
 * Diagnostic with no counterpart in the reference: the name of the kernel that tk3d_chamfer_fwd
 * launches for these sizes on the current device (a static string; launches nothing).  The fp32
 * forward has three: "chamfer_fwd_fast_kernel<1>" (small inputs, one query per thread),
 * "chamfer_fwd_smwide_kernel" (one 896-thread block per SM, for one or two nearly full rounds of
 * 256-query tasks) and "chamfer_fwd_fast_kernel<2>" (everything larger); fp64 has
 * "chamfer_fwd_generic_kernel".  Profilers and benchmarks use it to label their figures.
 */
const char *tk3d_chamfer_fwd_kernel_name(int64_t B, int64_t N1, int64_t N2, int dtype);

#ifdef __cplusplus
}
#endif
#endif /* TK3D_H_ */
