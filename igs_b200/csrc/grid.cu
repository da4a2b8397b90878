// Decides on the device whether the sample coordinates form a separable grid:
// x[b,h,w] == x[b,0,w] and y[b,h,w] == y[b,h,0] for every pixel (what xy_grid produces,
// also after it has been materialised per batch element).  The result is a flag in the
// workspace that the splat kernels read, so no host synchronisation is needed.
#include "grid.cuh"

namespace igs {

__global__ void __launch_bounds__(256) grid_check_kernel(GridCheckArgs a) {
    // a thread checks four consecutive pixels of one row (one 16-byte load per array when the
    // rows are contiguous and aligned, which is the materialised-grid case this kernel exists for)
    const long long quads_w = (a.W + 3) / 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over B*H*quads_w
    bool bad = false;
    if (i < (long long)a.B * a.H * quads_w) {
        const long long b = i / (a.H * quads_w), r = i - b * a.H * quads_w;
        const long long h = r / quads_w, w0 = (r - h * quads_w) * 4;
        const float* xr = a.x + b * a.xs_b + h * a.xs_h;  // this row
        const float* yr = a.y + b * a.ys_b + h * a.ys_h;
        const float* x0 = a.x + b * a.xs_b;               // row 0
        const float y0 = yr[0];                            // column 0 of this row
        float xv[4], yv[4], xf[4];
        const bool vec = a.xs_w == 1 && a.ys_w == 1 && w0 + 3 < a.W &&
                         ((reinterpret_cast<uintptr_t>(xr + w0) | reinterpret_cast<uintptr_t>(yr + w0) |
                           reinterpret_cast<uintptr_t>(x0 + w0)) & 15) == 0;
        if (vec) {
            const float4 vx = *reinterpret_cast<const float4*>(xr + w0), vy = *reinterpret_cast<const float4*>(yr + w0);
            const float4 vf = *reinterpret_cast<const float4*>(x0 + w0);
            xv[0] = vx.x; xv[1] = vx.y; xv[2] = vx.z; xv[3] = vx.w;
            yv[0] = vy.x; yv[1] = vy.y; yv[2] = vy.z; yv[3] = vy.w;
            xf[0] = vf.x; xf[1] = vf.y; xf[2] = vf.z; xf[3] = vf.w;
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const long long w = w0 + k < a.W ? w0 + k : a.W - 1;
                xv[k] = xr[w * a.xs_w];
                yv[k] = yr[w * a.ys_w];
                xf[k] = x0[w * a.xs_w];
            }
        }
        // bit comparison: the separable kernels must see exactly the values the general
        // one would (a NaN coordinate simply selects the general kernel)
#pragma unroll
        for (int k = 0; k < 4; ++k) bad |= (xv[k] != xf[k]) || (yv[k] != y0);
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(a.flag, GRID_NOT_SEPARABLE);
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(a.flag, GRID_CHECKED);  // for hosts that remember the answer
}

GridKind classify_grid(long long xs_h, long long ys_w, int H, int W, bool kernels_available) {
    // tiny images do not fill the 2 x 4 patches; not worth a second code path
    if (!kernels_available || H < 4 || W < 16) return GRID_GENERAL;
    // stride-0 views (x broadcast over rows, y over columns) are separable by construction
    if ((xs_h == 0 || H == 1) && (ys_w == 0 || W == 1)) return GRID_SEPARABLE;
    return GRID_CHECK_ON_DEVICE;
}

cudaError_t launch_grid_check(const GridCheckArgs& a, cudaStream_t s) {
    const long long n = (long long)a.B * a.H * ((a.W + 3) / 4);
    if (n <= 0) return cudaSuccess;  // (the flag word was cleared with the rest of the status area)
    {
        KernelTimer timer(K_GRID_CHECK, s);
        grid_check_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace igs
