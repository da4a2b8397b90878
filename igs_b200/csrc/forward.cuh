// Argument blocks and launchers of the forward kernels.
#pragma once

#include "plan.cuh"

namespace igs {

struct FwdArgs {
    const float* frec;  // forward records of this channel chunk, [B, N, fwd_rec_floats(ct)]
    const float* x;
    const float* y;
    long long xs_b, xs_h, xs_w, ys_b, ys_h, ys_w;  // element strides of x and y
    float* out;      // [B, C, HW]      (in_kernel_normalize)
    float* wsum;     // [B, HW]         (in_kernel_normalize && write_s)
    float* partial;  // [n_split, B, C+1, HW] otherwise
    int* status;
    // Selection on the device (nullptr = run unconditionally): an instantiation returns at
    // once unless the word picks it.
    const int* grid_sel;   // grid word: bit 0 = not a separable grid -> general / separable
    const int* cull_sel;   // count of narrow gaussians: at least one in eight -> culling / plain
    unsigned long long* exec_count;  // culling kernel: evaluations it did not skip (may be null)
    // culling kernel, records in a spatial order: {x0,x1,y0,y1} around each stage's gaussians,
    // [B, chunks_per_b, 4]; stages whose box misses the CTA's pixels are not even loaded
    const float* cbox;
    int chunks_per_b;
    int tiles_x;           // separable tiling: CTAs per tile row
    int B, N, H, W, C;
    int c0, cr;  // first channel and real channel count of this chunk
    int per_split;
    int in_kernel_normalize;
    int write_s;
    float eps;
};

struct ReduceArgs {
    const float* partial;  // [n_split, B, C+1, HW]
    float* out;            // normalize: [B, C, HW]; else [B, C+1, HW]
    float* wsum;           // normalize: [B, HW]
    long long HW;
    int B, C, n_split, normalize;
    float eps;
};

cudaError_t launch_forward_chunk(int ct, bool separable, bool culling, const FwdArgs& a, const FwdPlan& p,
                                 cudaStream_t s);
cudaError_t launch_reduce_normalize(const ReduceArgs& a, cudaStream_t s);

}  // namespace igs
