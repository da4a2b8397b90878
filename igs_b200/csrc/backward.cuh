// Argument blocks and launchers of the backward kernels.
#pragma once

#include "pack.cuh"
#include "plan.cuh"

namespace igs {

// per-pixel upstream terms -> pair records, all channel chunks in one pass
struct PixelTermArgs {
    const float* x;
    const float* y;
    long long xs_b, xs_h, xs_w, ys_b, ys_h, ys_w;
    const float* wsum;  // [B, HW]
    const float* out;   // [B, C, HW]  (exact mode only)
    const float* gout;  // [B, C, HW]
    float* prec[MAX_CHUNKS];  // [B, npairs, bwd_rec_floats(ct)]  or, separable, [B, nrp*ncb, bwd_sep_rec_floats(ct)]
                              // or, separable with 8 / 16 channels, [B, H, W, row-record floats] (backward_row.cu)
    float* axes;              // row layout only: receives y[b, h], [B, H]
    const int* grid_sel;      // grid word (bit 0 = not a separable grid) picking the kernel; nullptr = run
    int* flags;               // grid word: receives UPSTREAM_NOT_FINITE (separable kernel), or nullptr
    Chunks ch;
    long long npairs;
    int nrp, ncb;             // separable: row pairs and 4-column blocks per row pair
    int B, H, W, C;
    int mode;
    float eps;
};

struct BwdArgs {
    const float* geo;     // [B, N, 8]
    const float* colors;  // [B, N, C]
    const float* prec;    // records of this chunk
    const float* axes;    // row-streaming kernel (backward_row.cu): y[b, h], [B, H]
    const int* order;     // [B, N] permutation: processing slot -> gaussian index, or nullptr
    float* part;          // [n_slab, B, planes, N], N running over processing slots
    int* status;
    // Selection on the device (nullptr = run unconditionally): a kernel returns at once
    // unless the word picks it.
    const int* grid_sel;   // grid word: bit 0 = not a separable grid -> general / separable kernel
    unsigned long long* exec_count;  // skipping kernel: evaluations it did not skip (may be null)
    // task list of the ordered skipping path (backward_warp.cu); nullptr elsewhere
    int4* tasks;        // [task_capacity]: {batch element, group of 32 slots, slab, -}
    int4* group_rect;   // [B, ceil(N/32)]: rows lo..hi and column blocks lo..hi the group's box meets
    int* slab_range;    // [B, N]: first slab | (last slab + 1) << 16 that hold partial sums of the slot
    int* task_count;    // tasks on the list
    int* task_next;     // next task to hand out
    int task_capacity;
    const int* cull_sel;   // count of narrow gaussians: at least one in eight (and monotone axes,
    const int* grid_word;  //   bit 1 of the grid word clear) -> skipping / plain separable kernel
    long long npairs, pairs_per_slab;
    int nrp, ncb, rp_per_slab;  // separable: row pairs, blocks per row pair, row pairs per slab
    int n_slab;                 // slabs of the partition in use
    int B, N, C;
    int c0, cr;
    int planes;
    int moment_plane0;  // first of this chunk's 6 moment planes
    int color_plane0;   // first colour plane (+ c0 + c)
};

struct FinalizeArgs {
    ParamLayout lay;    // strides of the parameter arrays AND of their gradient arrays
    const float* part;  // [n_slab, B, planes, N]
    const int* slab_range;  // nullptr: every slab holds partial sums; else per slot, as in BwdArgs
    const int* order;       // nullptr, or [B, N]: the gaussian of every slot
    const float* pos;
    const float* shape0;  // scales | cov_inv_00
    const float* shape1;  // rotations | cov_inv_01
    const float* shape2;  // - | cov_inv_11
    const float* alpha;  // or nullptr for all ones
    float* d_pos;     // [B,N,2]
    float* d_shape0;  // d_scales [B,N,2] | d_cov_inv_00 [B,N]
    float* d_shape1;  // d_rotations [B,N] | d_cov_inv_01
    float* d_shape2;  // - | d_cov_inv_11
    float* d_alpha;   // [B,N], or nullptr
    float* d_colors;  // [B,N,C]
    int B, N, C, n_slab, planes, n_chunks;
    int kind;
    float eps;
};

// coordinate gradients (pixel-owner pass, only when the caller asks for d_x / d_y)
struct CoordGradArgs {
    const float* geo;
    const float* colors;
    const float* x;
    const float* y;
    long long xs_b, xs_h, xs_w, ys_b, ys_h, ys_w;
    const float* wsum;
    const float* out;
    const float* gout;
    float* d_x;  // [B, HW]
    float* d_y;
    int B, N, H, W, C;
    int mode;
    float eps;
};

cudaError_t launch_pixel_terms(const PixelTermArgs& a, bool separable, cudaStream_t s);
cudaError_t launch_backward_chunk(int ct, bool separable, bool culling, const BwdArgs& a, const BwdPlan& p,
                                  cudaStream_t s);
bool backward_has_separable(int ct);
cudaError_t launch_pixel_terms_sep(const PixelTermArgs& a, cudaStream_t s);
cudaError_t launch_backward_sep_chunk(int ct, bool culling, const BwdArgs& a, const BwdPlan& p, cudaStream_t s);
cudaError_t launch_backward_warp_chunk(int ct, const BwdArgs& a, const BwdPlan& p, int sm_count, cudaStream_t s);
// separable grids, chunks of 8 and 16 channels: two gaussians per f32x2, pixels stream row by row
bool backward_has_row_kernel(int ct);
int backward_row_ctas_per_sm(int ct, int device);
int backward_row_record_floats(int ct);
cudaError_t launch_pixel_terms_row(const PixelTermArgs& a, cudaStream_t s);
cudaError_t launch_backward_row_chunk(int ct, bool culling, const BwdArgs& a, const BwdPlan& p, cudaStream_t s);
cudaError_t launch_finalize(const FinalizeArgs& a, cudaStream_t s);
cudaError_t launch_coord_grad(const CoordGradArgs& a, cudaStream_t s);

}  // namespace igs
