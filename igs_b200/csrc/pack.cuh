// Per-gaussian prologue: raw parameters -> kernel records.
#pragma once

#include "plan.cuh"

namespace igs {

enum ShapeKind { SHAPE_SCALE_ROT = 0, SHAPE_COV_INV = 1 };

struct PackArgs {
    ParamLayout lay;
    const float* pos;     // [M,2]
    const float* shape0;  // scales [M,2]  | cov_inv_00 [M]
    const float* shape1;  // rotations [M] | cov_inv_01 [M]
    const float* shape2;  // unused        | cov_inv_11 [M]
    const float* alpha;   // [M], or nullptr for all ones
    const float* colors;  // [M,C]
    const float* x;       // sample coordinates (only their extent is read) or nullptr
    const float* y;
    long long xs_b, xs_w, ys_b, ys_h;
    const int* order;     // [B,N]: record slot -> gaussian (forward records only), or nullptr
    float* cbox;          // [B, ceil(N / chunk_g), 4]: box around each stage's gaussians, or nullptr
    int chunk_g;
    int* narrow_count;    // device counter of narrow gaussians, or nullptr
    int* grid_flag;       // receives GRID_NOT_MONOTONE when an axis is not non-decreasing, or nullptr
    int B, N, H, W;       // batch, gaussians per batch element, image size
    float* geo;           // [M,8] or nullptr
    float* frec[MAX_CHUNKS];  // per channel chunk, [M, fwd_rec_floats(ct)] or nullptr
    Chunks ch;
    long long M;
    int C;
    float eps;
    int kind;
};

cudaError_t launch_pack(const PackArgs& a, cudaStream_t s);
cudaError_t launch_stage_boxes(const PackArgs& a, cudaStream_t s);  // after launch_pack, when a.cbox is set

// scales, rotation -> inverse-covariance entries (closed form of R S (R S)^T + eps I
// inverted); shared by the prologue and by the gradient epilogue.
struct CovInv {
    float c00, c01, c11;
    float a, b, d, det, cs, sn;
};

__device__ __forceinline__ CovInv cov_inv_from_scale_rot(float sx, float sy, float theta, float eps) {
    CovInv r;
    sincosf(theta, &r.sn, &r.cs);
    const float p = sx * sx, q = sy * sy;
    r.a = r.cs * r.cs * p + r.sn * r.sn * q + eps;
    r.b = r.cs * r.sn * (p - q);
    r.d = r.sn * r.sn * p + r.cs * r.cs * q + eps;
    // det(R diag(p,q) R^T + eps I) = (p+eps)(q+eps): rotation invariant, no cancellation
    r.det = (p + eps) * (q + eps);
    r.c00 = r.d / r.det;
    r.c01 = -r.b / r.det;
    r.c11 = r.a / r.det;
    return r;
}

}  // namespace igs
