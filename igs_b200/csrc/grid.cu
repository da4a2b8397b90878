// Decides on the device whether the sample coordinates form a separable grid:
// x[b,h,w] == x[b,0,w] and y[b,h,w] == y[b,h,0] for every pixel (what xy_grid produces,
// also after it has been materialised per batch element).  The result is a flag in the
// workspace that the splat kernels read, so no host synchronisation is needed.
#include "grid.cuh"

namespace igs {

__global__ void __launch_bounds__(256) grid_check_kernel(GridCheckArgs a) {
    const long long HW = (long long)a.H * a.W;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over B*HW
    bool bad = false;
    if (i < (long long)a.B * HW) {
        const long long b = i / HW, p = i - b * HW;
        const long long h = p / a.W, w = p - h * a.W;
        const float xv = a.x[b * a.xs_b + h * a.xs_h + w * a.xs_w];
        const float yv = a.y[b * a.ys_b + h * a.ys_h + w * a.ys_w];
        // bit comparison: the separable kernels must see exactly the values the general
        // one would (a NaN coordinate simply selects the general kernel)
        bad = (xv != a.x[b * a.xs_b + w * a.xs_w]) || (yv != a.y[b * a.ys_b + h * a.ys_h]);
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(a.flag, GRID_NOT_SEPARABLE);
}

GridKind classify_grid(long long xs_h, long long ys_w, int H, int W, bool kernels_available) {
    // tiny images do not fill the 2 x 4 patches; not worth a second code path
    if (!kernels_available || H < 4 || W < 16) return GRID_GENERAL;
    // stride-0 views (x broadcast over rows, y over columns) are separable by construction
    if ((xs_h == 0 || H == 1) && (ys_w == 0 || W == 1)) return GRID_SEPARABLE;
    return GRID_CHECK_ON_DEVICE;
}

cudaError_t launch_grid_check(const GridCheckArgs& a, cudaStream_t s) {
    const long long n = (long long)a.B * a.H * a.W;
    cudaError_t e = cudaMemsetAsync(a.flag, 0, sizeof(int), s);
    if (e != cudaSuccess || n <= 0) return e;
    {
        KernelTimer timer(K_GRID_CHECK, s);
        grid_check_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace igs
