/*
 * C ABI of the B200-native svox hot path: octree point query and
 * differentiable volume rendering.
 *
 * Each entry point replaces one function of the reference's pybind11
 * module `svox.csrc` (svox/csrc/svox.cpp:106-113).  All pointers are
 * DEVICE pointers unless stated otherwise.  Outputs are caller-allocated;
 * the library itself only takes a small per-call jump table over the top
 * levels of the tree (<= 8 MB, normally 128 KB) from the CUDA stream-ordered
 * pool and returns it on the same stream.  Every call is asynchronous on
 * `stream` (a cudaStream_t passed as void*) and returns an svoxb_status.
 *
 * Layouts (identical to the reference's tensors, svox/svox.py:122-127):
 *   data   (M, N, N, N, K) float32, a leaf record is K contiguous floats:
 *          channel-major colour coefficients then the density
 *   child  (M, N, N, N)    int32, 0 = leaf, otherwise child_node - node
 *   offset, scaling (3)    float32 in device memory; tree-space position is
 *          offset + scaling * world_position
 */
#ifndef SVOX_B200_H
#define SVOX_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    SVOXB_OK = 0,
    SVOXB_ERR_NULL = 1,        /* a required pointer is null                 */
    SVOXB_ERR_SHAPE = 2,       /* a size is negative / inconsistent          */
    SVOXB_ERR_FORMAT = 3,      /* data format not supported by this build    */
    SVOXB_ERR_OPTION = 4,      /* invalid render option (e.g. step_size <= 0)*/
    SVOXB_ERR_CUDA = 5,        /* a CUDA runtime call failed                 */
    SVOXB_ERR_TREE = 6,        /* device status: descent left the node array */
    SVOXB_ERR_MARCH = 7,       /* device status: a ray hit the step cap      */
    SVOXB_ERR_TOO_LARGE = 8    /* size beyond a documented maximum           */
} svoxb_status;

/* Data formats (svox/csrc/include/data_spec.hpp:44-49). */
enum { SVOXB_FORMAT_RGBA = 0, SVOXB_FORMAT_SH = 1, SVOXB_FORMAT_SG = 2, SVOXB_FORMAT_ASG = 3 };

/* Replaces TreeSpec / PackedTreeSpec (svox/csrc/include/data_spec.hpp:66-89,
 * data_spec_packed.cuh:56-81). */
typedef struct {
    const float* data;
    const int32_t* child;
    const float* offset;
    const float* scaling;
    int64_t M;  /* number of nodes (capacity)  */
    int32_t N;  /* branching factor per axis   */
    int32_t K;  /* floats per leaf record      */
    /* Weight accumulation of the forward render (TreeSpec::_weight_accum,
     * svox/csrc/rt_kernel.cu:298-304): optional (M,N,N,N) float buffer; every
     * contributing sample adds its weight to the entry of its leaf, or raises it
     * to the weight if weight_accum_max is set.  Null: off. */
    float* weight_accum;
    int32_t weight_accum_max;
    int32_t reserved_;
    /* Lobe parameters of the Gaussian colour bases (TreeSpec::extra_data,
     * svox/csrc/rt_kernel.cu:120-140), row-major (extra_rows, extra_cols); used
     * only by SVOXB_FORMAT_SG (row i: sharpness, lobe axis xyz; extra_cols >= 4)
     * and SVOXB_FORMAT_ASG (row i: two bandwidths, then the x, y and z axes of the
     * lobe's frame; extra_cols >= 11), with extra_rows >= basis_dim.  Null otherwise. */
    const float* extra_data;
    int32_t extra_rows;
    int32_t extra_cols;
} svoxb_tree;

/* Replaces RaysSpec (svox/csrc/include/data_spec.hpp:51-64): three (Q, 3)
 * contiguous float arrays.  vdirs is used as given (not normalised). */
typedef struct {
    const float* origins;
    const float* dirs;
    const float* vdirs;
    int64_t Q;
} svoxb_rays;

/* Replaces CameraSpec (svox/csrc/include/data_spec.hpp:91-104).  c2w points
 * to a row-major (3 or 4, 4) camera-to-world matrix in device memory. */
typedef struct {
    const float* c2w;
    float fx;
    float fy;
    int32_t width;
    int32_t height;
} svoxb_camera;

/* Field for field the reference's RenderOptions
 * (svox/csrc/include/data_spec.hpp:107-126); density_softplus is an int. */
typedef struct {
    float step_size;
    float background_brightness;
    int32_t format;
    int32_t basis_dim;
    int32_t ndc_width;
    int32_t ndc_height;
    float ndc_focal;
    int32_t min_comp;
    int32_t max_comp;
    float sigma_thresh;
    float stop_thresh;
    int32_t density_softplus;
    float rgb_padding;
} svoxb_render_options;

/* query_vertical (svox/csrc/svox_kernel.cu:120-143): for each of Q points
 * (indices, (Q,3)) write the K values of the containing leaf to values_out
 * (Q,K) and its packed id node*N^3 + u*N^2 + v*N + w to node_ids_out (Q).
 * Either output may be null. */
int svoxb_query_vertical(const svoxb_tree* tree, const float* indices, int64_t Q,
                         float* values_out, int64_t* node_ids_out, void* stream);

/* query_vertical_backward (svox/csrc/svox_kernel.cu:160-182): scatter-add
 * grad_output (Q,Kg) into grad_data_out (M,N,N,N,Kg).  With zero_first != 0
 * the output is cleared first (the reference returns a fresh zero tensor). */
int svoxb_query_vertical_backward(const svoxb_tree* tree, const float* indices, int64_t Q,
                                  const float* grad_output, int32_t Kg, float* grad_data_out,
                                  int zero_first, void* stream);

/* assign_vertical (svox/csrc/svox_kernel.cu:80-89,145-158): overwrite the first
 * Kv floats (1 <= Kv <= K) of the record of each point's leaf with row q of
 * values (Q, Kv).  data_out is the tree's own data array (writable).  Points
 * that share a leaf race with each other, as in the reference: which row a
 * float ends up with is then unspecified. */
int svoxb_assign_vertical(const svoxb_tree* tree, const float* indices, int64_t Q,
                          const float* values, int32_t Kv, float* data_out, void* stream);

/* calc_corners (svox/csrc/svox_kernel.cu:91-115,184-203): lower corner, in
 * tree-local [0,1)^3 coordinates, of each cell (node, i, j, k) of indexer
 * (Q, 4) int64, found by walking parent_depth ((M, 2) int32: packed index of
 * the parent cell, depth) up to the root.  out is (Q, 3). */
int svoxb_calc_corners(const svoxb_tree* tree, const int32_t* parent_depth,
                       const int64_t* indexer, int64_t Q, float* out, void* stream);

/* volume_render (svox/csrc/rt_kernel.cu:1019-1036): out is (Q, out_dim),
 * out_dim = (K-1)/basis_dim, or K-1 for RGBA. */
int svoxb_volume_render(const svoxb_tree* tree, const svoxb_rays* rays,
                        const svoxb_render_options* opt, float* out, void* stream);

/* volume_render_image (svox/csrc/rt_kernel.cu:1038-1057): out is
 * (height, width, out_dim), pixel (ix, iy) at row iy. */
int svoxb_volume_render_image(const svoxb_tree* tree, const svoxb_camera* cam,
                              const svoxb_render_options* opt, float* out, void* stream);

/* volume_render_backward (svox/csrc/rt_kernel.cu:1059-1083): scatter-add the
 * gradient of sum(grad_output * out) w.r.t. data into grad_data_out (shaped
 * like data).  As in the reference the gradient is that of the render
 * WITHOUT sigma_thresh / stop_thresh.
 * fwd_out: optional (may be null) output of the forward call for the same
 * inputs; if given and both thresholds are zero, one march per ray is
 * enough instead of the reference's two. */
int svoxb_volume_render_backward(const svoxb_tree* tree, const svoxb_rays* rays,
                                 const svoxb_render_options* opt, const float* grad_output,
                                 const float* fwd_out, float* grad_data_out, int zero_first,
                                 void* stream);

/* volume_render_image_backward (svox/csrc/rt_kernel.cu:1085-1109). */
int svoxb_volume_render_image_backward(const svoxb_tree* tree, const svoxb_camera* cam,
                                       const svoxb_render_options* opt,
                                       const float* grad_output, const float* fwd_out,
                                       float* grad_data_out, int zero_first, void* stream);

/* Rendering many views of a tree that does not change in between (no
 * counterpart in the reference).  The forward render needs an index of the
 * tree (density-annotated child array, leaf table, bricks) that depends on
 * child, data's densities, opt->sigma_thresh and opt->density_softplus; the
 * plain entry points rebuild it on every call because data may have changed.
 * Here the caller keeps it: svoxb_render_scratch_words int32 words of device
 * memory, filled once by svoxb_render_scratch_build and passed to any number
 * of svoxb_volume_render[_image]_prepared calls -- valid until the tree or those
 * two options change.  Octrees with three colour channels of 1, 4, 9, 16 or
 * 25 basis functions (SH, SG or ASG) only (else SVOXB_ERR_FORMAT: use the
 * plain entry points). */
int64_t svoxb_render_scratch_words(const svoxb_tree* tree);
int svoxb_render_scratch_build(const svoxb_tree* tree, const svoxb_render_options* opt,
                               int32_t* scratch, void* stream);
int svoxb_volume_render_prepared(const svoxb_tree* tree, const svoxb_rays* rays,
                                 const svoxb_render_options* opt, const int32_t* scratch,
                                 float* out, void* stream);
int svoxb_volume_render_image_prepared(const svoxb_tree* tree, const svoxb_camera* cam,
                                       const svoxb_render_options* opt, const int32_t* scratch,
                                       float* out, void* stream);

/* Logged forward + replay backward (no counterpart in the reference; the
 * pair computes what volume_render followed by volume_render_backward
 * computes, svox/csrc/rt_kernel.cu:1019-1083).  The logged forward also
 * writes every contributing sample (leaf slot, ray, weight, transmittance,
 * step, colour sigmoids, the ray's colour sums so far) into `log`, a
 * caller-allocated int32 device buffer of svoxb_item_log_words(capacity_chunks)
 * words (one chunk = 32 samples).  The replay backward streams that log instead
 * of marching the rays and reading the leaf records again: it sorts the
 * samples by leaf range (scratch from the stream's memory pool, 32 bytes per
 * sample) and reduces the gradient range by range so that it stays in L2.
 * Only for octrees with three colour channels of 1, 4, 9, 16 or 25 basis
 * functions (SH, SG or ASG) and sigma_thresh =
 * stop_thresh = 0 (else SVOXB_ERR_FORMAT / SVOXB_ERR_OPTION).  `data` must not change between the two calls.
 *
 * A log that was too small must not be replayed.  `chunks_used` says who
 * checks that:
 *   0    nobody has read the count back.  The replay kernels read it on the
 *        device and do nothing if the forward asked for more chunks than
 *        `capacity_chunks`; a marching backward (as
 *        svoxb_volume_render_backward) is enqueued behind them that does its
 *        work only in that case.  No host synchronisation; the scratch is
 *        sized for the whole log; the result is the gradient either way.
 *   > 0  the caller read the count with svoxb_item_log_used (which
 *        synchronises) and found it <= capacity_chunks: the scratch is sized
 *        for that many chunks and no fallback is enqueued.  With a larger
 *        count the caller must call svoxb_volume_render_backward instead.
 * If the scratch cannot be had, the call marches like
 * svoxb_volume_render_backward. */
int64_t svoxb_item_log_words(int64_t capacity_chunks);
int svoxb_volume_render_logged(const svoxb_tree* tree, const svoxb_rays* rays,
                               const svoxb_render_options* opt, float* out, int32_t* log,
                               int64_t capacity_chunks, void* stream);
int svoxb_volume_render_image_logged(const svoxb_tree* tree, const svoxb_camera* cam,
                                     const svoxb_render_options* opt, float* out, int32_t* log,
                                     int64_t capacity_chunks, void* stream);
int svoxb_volume_render_backward_replay(const svoxb_tree* tree, const svoxb_rays* rays,
                                        const svoxb_render_options* opt,
                                        const float* grad_output, const float* fwd_out,
                                        int32_t* log, int64_t capacity_chunks,
                                        int64_t chunks_used, float* grad_data_out,
                                        int zero_first, void* stream);
int svoxb_volume_render_image_backward_replay(const svoxb_tree* tree, const svoxb_camera* cam,
                                              const svoxb_render_options* opt,
                                              const float* grad_output, const float* fwd_out,
                                              int32_t* log, int64_t capacity_chunks,
                                              int64_t chunks_used, float* grad_data_out,
                                              int zero_first, void* stream);
/* Third result of se_grad / se_grad_persp (svox/csrc/rt_kernel.cu:479-715,
 * 1111-1173): the diagonal of the Gauss-Newton matrix of the squared error
 * 1/2 sum (render - colour)^2, i.e. for every element of data the sum over rays
 * and channels of (d render / d element)^2.  Computed from the item log of a
 * logged forward like the replay backward (same restrictions, same scratch);
 * chunks_used must be the count read with svoxb_item_log_used (there is no
 * marching fallback for this result: 0 is refused with SVOXB_ERR_OPTION);
 * SVOXB_ERR_TOO_LARGE if the scratch cannot be had.  The first two results of
 * se_grad are the logged forward's output and the replay backward with
 * grad_output = render - colour. */
int svoxb_volume_render_hessdiag_replay(const svoxb_tree* tree, const svoxb_rays* rays,
                                        const svoxb_render_options* opt, const float* fwd_out,
                                        int32_t* log, int64_t capacity_chunks,
                                        int64_t chunks_used, float* hessdiag_out,
                                        int zero_first, void* stream);
int svoxb_volume_render_image_hessdiag_replay(const svoxb_tree* tree, const svoxb_camera* cam,
                                              const svoxb_render_options* opt,
                                              const float* fwd_out, int32_t* log,
                                              int64_t capacity_chunks, int64_t chunks_used,
                                              float* hessdiag_out, int zero_first,
                                              void* stream);

/* se_grad / se_grad_persp (svox/csrc/rt_kernel.cu:479-715,846-897,1111-1173)
 * for any record layout with at most 4 output channels (the reference's bound,
 * :1123): RGBA, N != 2, basis sizes without a specialised kernel.  One march per ray
 * adds the gradient of 1/2 sum (fwd_out - color_ref)^2 w.r.t. data into
 * grad_data_out and its Gauss-Newton diagonal into hessdiag_out (both shaped
 * like data).  fwd_out is the output of svoxb_volume_render[_image] for the same
 * inputs with both thresholds zero (the reference's kernel knows none);
 * color_ref is shaped like it. */
int svoxb_se_grad_march(const svoxb_tree* tree, const svoxb_rays* rays,
                        const svoxb_render_options* opt, const float* fwd_out,
                        const float* color_ref, float* grad_data_out, float* hessdiag_out,
                        int zero_first, void* stream);
int svoxb_se_grad_image_march(const svoxb_tree* tree, const svoxb_camera* cam,
                              const svoxb_render_options* opt, const float* fwd_out,
                              const float* color_ref, float* grad_data_out, float* hessdiag_out,
                              int zero_first, void* stream);

/* The replay backward in steps, for callers that overlap the all-reduce of the
 * gradient with its computation (no counterpart in the reference).  _begin
 * sorts the logged samples by leaf range (arguments as for
 * svoxb_volume_render_backward_replay, chunks_used included;
 * SVOXB_ERR_TOO_LARGE if the scratch cannot be had) and returns a job.
 * grad_data_out is the gradient buffer, zeroed by the caller: with
 * chunks_used = 0 the marching fallback for an overflowed log is enqueued here,
 * BEFORE the parts, so that a part's rows are final after its scatter
 * whichever of the two produced them -- every process of a data-parallel job
 * can then issue the same collectives without agreeing on a route first.
 * The leaf slots are cut into `n_parts` (1..16) consecutive ranges (whole
 * bins, svoxb_replay_bin_shift); svoxb_replay_part_range gives the slots
 * [begin, end) of a part, i.e. rows [begin*K, end*K) of the flat gradient.
 * svoxb_replay_scatter adds the gradient of one part into grad_data_out; with
 * reserve_sms > 0 it leaves that many SMs free for a collective kernel running
 * beside it.  svoxb_replay_end releases the scratch on `stream`. */
int svoxb_replay_begin(const svoxb_tree* tree, const svoxb_rays* rays,
                       const svoxb_render_options* opt, const float* grad_output,
                       const float* fwd_out, int32_t* log, int64_t capacity_chunks,
                       int64_t chunks_used, int n_parts, float* grad_data_out, void* stream,
                       void** job);
int svoxb_replay_image_begin(const svoxb_tree* tree, const svoxb_camera* cam,
                             const svoxb_render_options* opt, const float* grad_output,
                             const float* fwd_out, int32_t* log, int64_t capacity_chunks,
                             int64_t chunks_used, int n_parts, float* grad_data_out,
                             void* stream, void** job);
int svoxb_replay_part_range(const void* job, int part, int64_t* slot_begin, int64_t* slot_end);
/* log2 of the leaf slots per bin for a tree of M nodes and K floats per record. */
int svoxb_replay_bin_shift(int64_t M, int32_t K);
int svoxb_replay_scatter(const void* job, int part, float* grad_data_out, int reserve_sms,
                         void* stream);
int svoxb_replay_end(void* job, void* stream);

/* Chunks the logged forward asked for (synchronises `stream`); more than the log's
 * capacity means that it overflowed. */
int svoxb_item_log_used(const int32_t* log, int64_t* chunks_used, void* stream);

/* Forward ray render that allocates nothing (no counterpart in the
 * reference).  Same inputs, outputs and results as svoxb_volume_render, for
 * hosts that may not touch a device allocator while rendering: an application
 * that hands the whole device heap to its own manager, a plug-in inside a
 * real-time loop that forbids allocation, a process with a memory budget fixed
 * at start-up.  The per-call scratch lives in a static device array instead:
 * 17 MiB that every GPU which loads the library holds until exit.
 *
 * Limits: octrees (N = 2) with SH colour in three channels (K = 3 * basis_dim
 * + 1) and at most SVOXB_NOALLOC_MAX_NODES nodes; a larger tree is refused
 * with SVOXB_ERR_TOO_LARGE, another layout with SVOXB_ERR_FORMAT, before
 * anything is launched.
 *
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture,
 * and from one host thread (the look-up is cached without a lock; threads
 * racing on a device's first call would all store the same address).
 * All calls share the one array.  Each call overwrites the parts it reads, so
 * nothing has to be cleared between calls, but two calls whose kernels
 * overlap on the GPU (different streams, no ordering between them) race on
 * it: keep calls to this entry point ordered on a device. */
#define SVOXB_NOALLOC_MAX_NODES (1 << 19)
int svoxb_volume_render_noalloc(const svoxb_tree* tree, const svoxb_rays* rays,
                                const svoxb_render_options* opt, float* out, void* stream);

/* Per-ray march statistics for a ray batch (no counterpart in the
 * reference; it is how the byte model of the roofline is counted): number of
 * sampled leaves, of samples passing the forward density test
 * (sigma > sigma_thresh, up to the early stop) and of samples with sigma > 0
 * (what the backward pass touches).  Each output is (Q) int32 and may be null. */
int svoxb_march_stats(const svoxb_tree* tree, const svoxb_rays* rays,
                      const svoxb_render_options* opt, int32_t* visits, int32_t* contrib_fwd,
                      int32_t* contrib_bwd, void* stream);

/* Device-side anomaly report.  The kernels bound every loop (the
 * reference's descent and march are unbounded, svox/csrc/include/
 * common.cuh:67-88, rt_kernel.cu:261) and record SVOXB_ERR_TREE /
 * SVOXB_ERR_MARCH in a per-device status word instead of hanging.  This
 * call synchronises `stream`, returns the word of the current device and
 * optionally clears it. */
int svoxb_device_status(int clear, void* stream);

/* Text for a status code (replaces the reference's printf in
 * CUDA_CHECK_ERRORS, svox/csrc/include/common.cuh:98-101). */
const char* svoxb_strerror(int status);

/* Text of the last CUDA runtime error seen by this library on the calling
 * thread (empty string if none). */
const char* svoxb_last_cuda_error(void);

/* Leave `n` multiprocessors without a block in the library's persistent kernels (the
 * march, the passes of the replay backward), for kernels of the caller that run beside
 * them on another stream -- typically a collective that reduces the previous step's
 * gradient while this step computes (no counterpart in the reference).  Process-wide,
 * takes effect at the next launch; returns the previous value; n < 0 only queries. */
int svoxb_reserve_sms(int n);

/* Multi-GPU: sum of the gradient over all GPUs, in place, through NVSwitch
 * multicast memory (no counterpart in the reference, which is single-GPU).
 * Every rank holds its n_floats values in a buffer that is bound, at the same
 * offset on every GPU, into one multicast object; `multicast` is this
 * process's address of that object's range (e.g. the multicast_ptr of a
 * torch.distributed._symmetric_memory allocation).  Rank `rank` of `world`
 * sums its 1/world slice inside the switch (multimem.ld_reduce) and writes
 * the sums to all GPUs (multimem.st).  The kernel waits for nobody: the
 * caller orders it between two barriers across the ranks on the same stream
 * (all gradients complete before; all slices written after).  n_floats a
 * multiple of 4, the address 16-byte aligned. */
int svoxb_allreduce_multimem(float* multicast, int64_t n_floats, int rank, int world,
                             void* stream);

/* Library version, "major.minor.patch". */
const char* svoxb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SVOX_B200_H */
