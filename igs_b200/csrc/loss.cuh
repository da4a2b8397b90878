// Argument block and launcher of the fused loss + pixel-terms kernel (loss.cu).
#pragma once

#include "common.cuh"

namespace igs {

constexpr int LOSS_TERMS_THREADS = 128;

struct LossTermArgs {
    const float* partial;   // un-normalised sums of the forward, [n_split][B][C+1][H*W]
    const float* target;    // [B, C, H*W]
    const float* x;         // separable grid: x[b, 0, w], y[b, h, 0]
    const float* y;
    long long xs_b, xs_w, ys_b, ys_h;
    const float* upstream;  // device scalar d(objective)/d(loss), or nullptr for 1
    float* out;             // [B, C, H*W] image, or nullptr
    float* wsum;            // [B, H*W] weight sums, or nullptr
    float* prec;            // the separable backward's block records, [B, nrp*ncb, bwd_sep_rec_floats(ct)]
    float* loss_partial;    // [loss_terms_blocks(...)]
    int* flags;             // grid word of the status area: receives UPSTREAM_NOT_FINITE
    long long n_total;      // B*C*H*W, the divisor of the mean
    int n_split;
    int B, H, W, C, nrp, ncb, ct;
    int mode;
    float eps;
};

long long loss_terms_blocks(int B, int nrp, int ncb);
// launches the kernel and the one-block finish that leaves mean((out - target)^2) in *loss
cudaError_t launch_loss_terms_sep(const LossTermArgs& a, float* loss, cudaStream_t s);

}  // namespace igs
