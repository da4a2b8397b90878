// Separable-grid detection shared by the forward and backward entry points.
#pragma once

#include "common.cuh"

namespace igs {

enum GridKind {
    GRID_GENERAL = 0,          // run the general kernels only
    GRID_SEPARABLE = 1,        // known on the host (stride-0 views): separable kernels only
    GRID_CHECK_ON_DEVICE = 2,  // check the data; launch both kinds, the flag picks one
};

struct GridCheckArgs {
    const float* x;
    const float* y;
    long long xs_b, xs_h, xs_w, ys_b, ys_h, ys_w;
    int* flag;
    int B, H, W;
};

GridKind classify_grid(long long xs_h, long long ys_w, int H, int W, bool kernels_available);
cudaError_t launch_grid_check(const GridCheckArgs& a, cudaStream_t s);

}  // namespace igs
