/*
 * igs_b200 -- C ABI of the sm_100a (B200) implementation of IGS's differentiable,
 * weight-normalised 2D gaussian splatting (forward and backward).
 *
 * The reference (KohakuBlueleaf/IGS) has no FFI of its own: its inner op is a
 * torch.autograd.Function written in Python.  The entry points below are what a
 * binding for that op would call; each cites the reference code it replaces
 * (paths relative to the reference tree).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on `device` unless stated otherwise; all
 *     tensors are fp32 and contiguous except x / y, which carry element strides;
 *   - `stream` is a cudaStream_t passed as void*; nothing synchronises the stream
 *     except igs_read_status, igs_read_status_static,
 *     igs_read_executed and igs_profile_read;
 *   - the library never allocates: scratch comes in through `workspace`, whose
 *     size igs_workspace_bytes reports; the first 256 bytes of a workspace hold a
 *     status word the kernels set if one of their bounded waits gives up;
 *   - return value: 0 = ok, negative = IGS_ERR_* argument error, positive = a
 *     cudaError_t from launching.  No entry point throws or aborts.
 *   - entry points may be called from any host thread (autograd runs backward on
 *     its own thread); they select `device` themselves and restore the previous one.
 *
 * Layouts (the reference's):  positions [B,N,2], scales [B,N,2], rotations [B,N],
 * alphas [B,N], colors [B,N,C], cov_inv_xx [B,N], x / y logical [B,H,W] with strides
 * (batch, row, column) in elements, out / gout [B,C,H,W], wsum [B,H,W].
 */
#ifndef IGS_B200_H
#define IGS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IGS_OK 0
#define IGS_ERR_ARG (-1)        /* null pointer, negative size, unsupported value */
#define IGS_ERR_WORKSPACE (-2)  /* workspace missing or smaller than igs_workspace_bytes */
#define IGS_ERR_LIMIT (-3)      /* size beyond a documented limit */
#define IGS_ERR_DEVICE (-4)     /* device cannot be selected or is not sm_100 */
#define IGS_ERR_STATUS (-5)     /* a kernel reported a timed-out wait (igs_read_status) */

/* gradient of the per-pixel normalisation term, see igs_backward_* */
#define IGS_GRAD_REFERENCE 0  /* gS = -sum_c g_c^2 / S^2, src/igs/gs2d.py:370 (and :176) */
#define IGS_GRAD_EXACT 1      /* gS = -sum_c (g_c/S) out_c, autograd of src/igs/gs2d.py:24-44 */

/*
 * `hints` of igs_forward_* / igs_backward_*: what the caller already knows about its data,
 * OR-ed together; 0 = nothing.  Without a hint the library finds both facts out on the
 * device and launches every kernel instantiation that could apply (those the data does
 * not call for return at once); a hint only removes launches.  Both hints name the
 * instantiation that is correct for any data, so a wrong hint costs time, never a bit of
 * the result.
 *   IGS_HINT_WIDE_GAUSSIANS: few gaussians are narrow (igs_read_status_words, word 2): only
 *                            the plain kernels are launched, not the culling ones;
 *   IGS_HINT_GENERAL_GRID:   x / y are not a separable grid (x by column, y by row): only
 *                            the general kernels are launched, and the grid is not checked.
 * A caller that knows its grid IS separable says so through the strides: row stride 0 for
 * x and column stride 0 for y (then nothing is checked and only the separable kernels run).
 */
#define IGS_HINT_WIDE_GAUSSIANS 1
#define IGS_HINT_GENERAL_GRID 2

int igs_version(void);
const char* igs_strerror(int code);

/* Number of kernels this library has launched in this process so far. */
long long igs_launch_count(void);

/*
 * Scratch sizes for one forward / one backward call of the given shape on `device`.
 * Either output pointer may be NULL.
 */
int igs_workspace_bytes(int B, int N, int H, int W, int C, int device, size_t* forward_bytes,
                        size_t* backward_bytes);

/*
 * Forward from scales and rotations.  Replaces GaussianSplatting2D.render with
 * fused=True (src/igs/gs2d.py:524-596): scales, rotations -> inverse covariance
 * (:549-580), then the fused splat (:275-337).
 *   normalize != 0: out [B,C,H,W] = numerator / (weight_sum + eps), wsum [B,H,W] =
 *                   weight_sum without eps (what the reference saves, :334);
 *   normalize == 0: out receives the UN-normalised sums [B,C+1,H,W] (C numerator
 *                   planes, then the weight-sum plane), wsum is ignored.  Used when
 *                   gaussians are sharded across GPUs and the sums are all-reduced
 *                   before igs_normalize.
 *   order: NULL, or a permutation [B,N] (int32; igs_spatial_order makes a good one): the
 *                   gaussians are summed in that order.  In a spatial order, 128 consecutive
 *                   gaussians share a patch of the image, and with narrow gaussians a CTA
 *                   does not even load the groups whose patch misses its pixels.  The image
 *                   then differs from an order-less call by fp32 rounding (another order
 *                   of summation); with the same order it is the same bits on every call.
 */
int igs_forward_sr(const float* positions, const float* scales, const float* rotations,
                   const float* alphas, const float* colors, const float* x, const int64_t* x_strides,
                   const float* y, const int64_t* y_strides, int B, int N, int H, int W, int C,
                   float eps, int normalize, float* out, float* wsum, const int* order, int hints,
                   void* workspace, size_t workspace_bytes, int device, void* stream);

/*
 * Forward from inverse-covariance entries.  Replaces
 * GaussianSplatting2DChunkedKernel.forward / GaussianSplatting2DKernel.forward
 * (src/igs/gs2d.py:275-337, :68-144), the entry the reference's benchmark calls
 * directly (scripts/profiling.py:97-100).  cov_inv may be indefinite.
 */
int igs_forward_cov(const float* positions, const float* cov_inv_00, const float* cov_inv_01,
                    const float* cov_inv_11, const float* alphas, const float* colors, const float* x,
                    const int64_t* x_strides, const float* y, const int64_t* y_strides, int B, int N,
                    int H, int W, int C, float eps, int normalize, float* out, float* wsum,
                    const int* order, int hints, void* workspace, size_t workspace_bytes, int device,
                    void* stream);

/*
 * igs_forward_sr without a workspace argument, for hosts that cannot allocate device
 * memory (a plug-in inside another application's memory budget, a loop that must stay
 * off the driver's allocator).  No counterpart in the reference: it is an addition of
 * this library.  Same arguments and return codes as igs_forward_sr (minus order, hints and
 * the workspace) and the same results up to the order of summation (the gaussian splits
 * may differ, see below); the scratch is a fixed array of IGS_STATIC_SCRATCH_BYTES inside
 * the library's device image (held on every GPU that loads the library until the process
 * exits).
 *   - returns IGS_ERR_LIMIT when the shape needs more scratch than that: with C <= 4
 *     the records take 48 bytes per gaussian (B*N*48 <= 8 MiB, about 170k gaussians);
 *     gaussian splits are dropped first if their partial sums would not fit;
 *   - calls no cudaMalloc / cudaFree and no allocating library routine (per-kernel
 *     profiling, igs_profile_enable, must stay off: it creates events);
 *   - all calls on a device share the one array: calls whose kernels could overlap on
 *     the GPU must be ordered on one stream by the caller;
 *   - every call looks up the array's device address (cudaGetSymbolAddress, with `device`
 *     current); the first such call on a device may load the library's device code, so
 *     make it at start-up, before any stream capture begins;
 *   - a kernel that gave up on a bounded wait reports through the array's status word:
 *     igs_read_status_static reads it.
 */
#define IGS_STATIC_SCRATCH_BYTES (8u << 20)
int igs_forward_sr_static(const float* positions, const float* scales, const float* rotations,
                          const float* alphas, const float* colors, const float* x,
                          const int64_t* x_strides, const float* y, const int64_t* y_strides, int B, int N,
                          int H, int W, int C, float eps, int normalize, float* out, float* wsum, int device,
                          void* stream);

/*
 * sums [B,C+1,H,W] -> out [B,C,H,W], wsum [B,H,W].  The division of
 * src/igs/gs2d.py:323, split off so that an all-reduce can run in between.
 */
int igs_normalize(const float* sums, int B, int H, int W, int C, float eps, float* out, float* wsum,
                  int device, void* stream);

/*
 * Backward to scales and rotations.  Replaces
 * GaussianSplatting2DChunkedKernel.backward (src/igs/gs2d.py:339-465) followed by
 * autograd through the covariance construction (:549-580).
 *   wsum: as written by the forward; out: the forward image, read only when
 *   grad_mode == IGS_GRAD_EXACT (may be NULL otherwise); gout [B,C,H,W] is NOT
 *   modified (the reference divides it in place, :371).
 *   d_x, d_y [B,H,W] contiguous, both NULL to skip (src/igs/gs2d.py:433-434).
 *   order: NULL, or a permutation [B,N] (int32) of each batch element's gaussians giving
 *   the order in which threads take them (igs_spatial_order makes a good one).  In a
 *   spatial order the 32 gaussians of a warp share a patch of the image, and the skipping
 *   kernel lets each warp visit only the pixels its patch reaches.  Passing an order also selects a
 *   finer partition of the rows into slabs (fixed by the shape), so that the few slabs
 *   a patch touches still fill the GPU.  The gradients do not depend on WHICH permutation
 *   is passed, bit for bit; against order == NULL they agree to fp32 rounding (the
 *   per-slab sums associate differently).  The array must hold a permutation of 0..N-1 per
 *   batch element; entries outside that range are not followed (that gaussian's gradient
 *   is then missing), repeated entries make two threads write the same gradient.
 */
int igs_backward_sr(const float* positions, const float* scales, const float* rotations,
                    const float* alphas, const float* colors, const float* x, const int64_t* x_strides,
                    const float* y, const int64_t* y_strides, const float* wsum, const float* out,
                    const float* gout, int B, int N, int H, int W, int C, float eps, int grad_mode,
                    float* d_positions, float* d_scales, float* d_rotations, float* d_alphas,
                    float* d_colors, float* d_x, float* d_y, const int* order, int hints, void* workspace,
                    size_t workspace_bytes, int device, void* stream);

/*
 * Backward to inverse-covariance entries.  Replaces
 * GaussianSplatting2DChunkedKernel.backward (src/igs/gs2d.py:339-465); returns the
 * same eight gradients (:455-465).
 */
int igs_backward_cov(const float* positions, const float* cov_inv_00, const float* cov_inv_01,
                     const float* cov_inv_11, const float* alphas, const float* colors, const float* x,
                     const int64_t* x_strides, const float* y, const int64_t* y_strides,
                     const float* wsum, const float* out, const float* gout, int B, int N, int H, int W,
                     int C, float eps, int grad_mode, float* d_positions, float* d_cov_inv_00,
                     float* d_cov_inv_01, float* d_cov_inv_11, float* d_alphas, float* d_colors,
                     float* d_x, float* d_y, const int* order, int hints, void* workspace,
                     size_t workspace_bytes, int device, void* stream);

/*
 * The splat driven directly by the module's projection output.  Replaces what
 * GaussianSplatting2D.forward does between its Linear layer and render
 * (src/igs/gs2d.py:635-675): split of gs_feature [B,N,6+C] into position (2), log-scale
 * (2), rotation (1), an unused opacity logit (1) and colours (C); scales = exp(log-scale)
 * + eps; opacities all ones; optional pos_map offset added to the positions (:655-667).
 * The forward reads the rows in place; the backward writes d_feature [B,N,6+C] in place
 * of autograd through split / exp / add (column 5, the unused logit, gets zeros).
 *   pos_offset: [B,N,2] contiguous or NULL; its gradient equals d_feature[..., 0:2].
 *   Everything else as igs_forward_sr / igs_backward_sr; no d_x / d_y at this level.
 */
int igs_forward_feature(const float* gs_feature, const float* pos_offset, const float* x,
                        const int64_t* x_strides, const float* y, const int64_t* y_strides, int B, int N,
                        int H, int W, int C, float eps, int normalize, float* out, float* wsum,
                        const int* order, int hints, void* workspace, size_t workspace_bytes, int device,
                        void* stream);
int igs_backward_feature(const float* gs_feature, const float* pos_offset, const float* x,
                         const int64_t* x_strides, const float* y, const int64_t* y_strides,
                         const float* wsum, const float* out, const float* gout, int B, int N, int H,
                         int W, int C, float eps, int grad_mode, float* d_feature, const int* order,
                         int hints, void* workspace, size_t workspace_bytes, int device, void* stream);

/*
 * Synchronises `stream`, copies the workspace's status word to *host_status
 * (HOST pointer) and returns IGS_ERR_STATUS if it is non-zero.
 */
int igs_read_status(const void* workspace, int device, void* stream, int* host_status);

/*
 * The same check for igs_forward_sr_static, whose caller has no workspace pointer: reads
 * the status word of the library's fixed scratch array on `device` (what the last
 * igs_forward_sr_static call on that device left).  Synchronises `stream`.
 */
int igs_read_status_static(int device, void* stream, int* host_status);

/*
 * Asynchronous read of what the last forward or backward on this workspace found out about
 * its data: queues on `stream` a copy of the first IGS_STATUS_WORDS words of the status
 * area into host_words (HOST pointer to IGS_STATUS_WORDS ints, pinned for a copy that does
 * not block) and returns at once; the values are there when the stream has reached that
 * point.  Never synchronises.
 *   word 0: non-zero if a kernel gave up on a bounded wait (the result is then invalid);
 *   word 1: bit 0 = the grid is NOT separable (only set when the library had to check),
 *           bit 1 = an axis is not non-decreasing, bit 2 = a non-finite upstream value;
 *   word 2: the number of narrow gaussians (see igs_read_narrow_count).
 * A host remembers these to pass `hints` (or stride-0 grid views) on later calls.
 */
#define IGS_STATUS_WORDS 8
int igs_read_status_words(const void* workspace, int device, void* stream, int* host_words);

/*
 * Launch geometry the library would use (for reports): pixels per forward CTA,
 * gaussian splits, backward threads per CTA and pixel slabs.  Any pointer may be NULL.
 */
int igs_describe_plan(int B, int N, int H, int W, int C, int device, int* fwd_tile_pixels,
                      int* fwd_splits, int* bwd_threads, int* bwd_slabs);

/*
 * For reports: whether kernels specialised for separable grids (x by column, y by row; what
 * xy_grid makes) exist for C channels, forward and backward (1 / 0).  They issue fewer
 * FMA-pipe instructions per evaluation than the general kernels.  Either pointer may be NULL.
 */
int igs_describe_kernels(int C, int* forward_separable, int* backward_separable);

/*
 * Lossless culling, on by default.  A weight ex2(q) is exactly zero once its exponent is
 * below -126, so a gaussian whose zero-weight box misses a tile of pixels contributes
 * exactly nothing there; the kernels skip such (gaussian, tile) combinations when
 * enough gaussians are narrow for the test to pay.  Results are bit-identical with
 * culling off (this switch exists to verify that, and for timing).  Process-wide.
 */
int igs_set_culling(int on);

/*
 * A spatial order for the `order` argument of igs_backward_*: order[b, slot] = index of
 * the gaussian taken in that slot, neighbours in the image next to each other (Hilbert-curve
 * order of a 64 x 64 lattice over the sampled extent; x, y and their strides as for the
 * forward, only the first row of x and the first column of y are read).  Worth computing
 * when most gaussians are narrow (igs_read_narrow_count) and the grid is separable: the
 * backward then skips most pixel runs.  A stable counting sort: gaussians of one lattice
 * cell keep their index order and the permutation is the same on every run.  No
 * counterpart in the reference,
 * whose backward is a dense torch expression (src/igs/gs2d.py:331-436).
 *   workspace: igs_spatial_order_workspace_bytes(B, N) bytes of device memory.
 */
size_t igs_spatial_order_workspace_bytes(int B, int N);
int igs_spatial_order(const float* positions, const float* x, const int64_t* x_strides, const float* y,
                      const int64_t* y_strides, int B, int N, int H, int W, int* order,
                      void* workspace, size_t workspace_bytes, int device, void* stream);

/*
 * The same sort on another key: per axis the centre of the gaussian's zero-weight box
 * clipped to the sampled extent.  A narrow gaussian inside the image keeps its own centre, a
 * box that sticks out on one side is placed by how far it reaches in, and a box that covers
 * the whole extent lands on the image's centre line next to all others like it, so that one
 * image-wide gaussian does not sit in a warp of narrow ones and make it visit every pixel.
 * The parameters are read where they lie, in the layout of the parameter-level or of the
 * feature-level entry points: gaussian i (over B*N) has its centre at
 * positions[i * position_stride .. +1] (plus position_offsets[2i .. +1] when that is not
 * NULL), its scales (logarithms of them with log_scales = 1) at scales[i * scale_stride ..
 * +1] and its angle at rotations[i * rotation_stride].  rotations = NULL: the larger scale
 * stands in for both axes; scales = NULL: igs_spatial_order.  Same workspace, same
 * determinism.  No counterpart in the reference.
 */
int igs_spatial_order_boxes(const float* positions, int64_t position_stride, const float* position_offsets,
                            const float* scales, int64_t scale_stride, int log_scales,
                            const float* rotations, int64_t rotation_stride, const float* x,
                            const int64_t* x_strides, const float* y, const int64_t* y_strides, int B, int N,
                            int H, int W, int* order, void* workspace, size_t workspace_bytes, int device,
                            void* stream);

/*
 * Asynchronous read of the narrow-gaussian count the last forward or backward on this
 * workspace left: the number of gaussians (over the whole batch) whose zero-weight box
 * covers less than three quarters of the sampled extent in x or y.  The copy is queued on
 * `stream` into *host_count (HOST pointer, pinned for a copy that does not block); the
 * value is there once the stream has reached that point.  The culling kernels are selected
 * on the device when count * 8 >= B * N; a host uses the same test to decide whether a
 * spatial order pays.
 */
int igs_read_narrow_count(const void* workspace, int device, void* stream, int* host_count);

/*
 * For reports: the number of (gaussian, pixel) evaluations the culling kernel of the last
 * forward or backward on this workspace did NOT skip (tile padding included), or 0 when
 * the plain kernel ran (it evaluates all B*N*H*W).  With several channel chunks the count
 * covers all of them.  Copies to *host_count (HOST pointer) and waits for the stream.
 */
int igs_read_executed(const void* workspace, int device, void* stream, unsigned long long* host_count);

/*
 * The L2 loss behind the renderer in the reference's fit scripts
 * (F.mse_loss(rendered_image, target_image), scripts/2dgs_img_comp.py:135,
 * scripts/gs2d_test.py:56), as two calls so that a host-side autograd can hand the
 * upstream scalar to the second:
 *   igs_mse_loss: *loss (device scalar) = mean((out - target)^2) over n elements;
 *   igs_mse_grad: gout[i] = upstream * 2 (out[i] - target[i]) / n, upstream a device
 *                 scalar or NULL for 1.
 * No atomics: the loss is repeatable to the bit.  workspace: IGS_MSE_WORKSPACE_BYTES.
 */
#define IGS_MSE_WORKSPACE_BYTES 4096
int igs_mse_loss(const float* out, const float* target, long long n, float* loss, void* workspace,
                 size_t workspace_bytes, int device, void* stream);
int igs_mse_grad(const float* out, const float* target, long long n, const float* upstream, float* gout,
                 int device, void* stream);

/*
 * Render, mean-squared-error loss and all gradients in one call: what one step of the
 * reference's per-image fit computes (scripts/2dgs_img_comp.py: the model's forward
 * :107-126, `GaussianSplatting2D.render(position, color, exp(log_scale) + eps, rotation,
 * ones, grids)`, the L2 term of its loss :132-143, `F.mse_loss(rendered_image,
 * target_image)`, and autograd back through both).
 *   loss  (device scalar)  = mean((image - target)^2) over B*C*H*W elements;
 *   d_*                    = upstream * d loss / d parameter, by the backward of
 *                            igs_backward_sr in `grad_mode`;
 *   log_scales != 0: `scales` holds log-scales, scale = exp(v) + eps, and d_scales is the
 *                    gradient with respect to the log-scales (the fit's parametrisation);
 *   alphas == NULL (with d_alphas == NULL): all opacities are one, as the fit script has them;
 *   upstream: device scalar d objective / d loss, or NULL for 1;
 *   out: receives the image [B,C,H,W], or NULL if the caller does not need it.
 * On a grid that is separable by its strides (x row stride 0, y column stride 0: what
 * xy_grid makes) with at most 4 channels the steps are fused: the forward's prologue also
 * packs the backward's records, and one kernel turns the forward's un-normalised sums into
 * the image, the loss and the backward's per-pixel terms, so neither the upstream gradient
 * nor the weight sums ever go to memory.  Any other input runs the same steps one after the
 * other; the results are the same to fp32 rounding either way.  No atomics: loss and
 * gradients are repeatable to the bit.  order, hints: as for igs_forward_sr.
 */
int igs_render_mse_workspace_bytes(int B, int N, int H, int W, int C, int device, size_t* bytes);
int igs_render_mse_sr(const float* positions, const float* scales, const float* rotations,
                      const float* alphas, const float* colors, int log_scales, const float* x,
                      const int64_t* x_strides, const float* y, const int64_t* y_strides,
                      const float* target, int B, int N, int H, int W, int C, float eps, int grad_mode,
                      const float* upstream, float* loss, float* out, float* d_positions,
                      float* d_scales, float* d_rotations, float* d_alphas, float* d_colors,
                      const int* order, int hints, void* workspace, size_t workspace_bytes, int device,
                      void* stream);

/*
 * Per-kernel device timing for reports.  While enabled, every kernel launch of the
 * library is bracketed by CUDA events recorded on the launch's own stream;
 * igs_profile_read waits for the recorded events and returns the accumulated device
 * time and launch count of one kernel since the last igs_profile_reset.  The devices
 * that recorded events must still be alive when reading.  Off by default.
 * igs_profile_enable: 0 = off, 1 = every kernel, 2 = the two splat kernels only (forward,
 * backward): an event pair costs a few microseconds of host and stream time per launch, which
 * a sub-millisecond step notices.
 */
#define IGS_KERNEL_PACK 0         /* per-gaussian prologue */
#define IGS_KERNEL_FORWARD 1      /* forward splat */
#define IGS_KERNEL_REDUCE 2       /* split reduction / normalisation */
#define IGS_KERNEL_PIXEL_TERMS 3  /* per-pixel upstream terms */
#define IGS_KERNEL_BACKWARD 4     /* backward splat */
#define IGS_KERNEL_FINALIZE 5     /* per-gaussian gradient epilogue */
#define IGS_KERNEL_COORD_GRAD 6   /* d_x, d_y */
#define IGS_KERNEL_GRID_CHECK 7   /* separable-grid detection */
#define IGS_KERNEL_COUNT 8
int igs_profile_enable(int on);
int igs_profile_reset(void);
int igs_profile_read(int kernel_id, double* total_ms, long long* launches);

#ifdef __cplusplus
}
#endif
#endif /* IGS_B200_H */
