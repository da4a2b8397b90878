// igs_spatial_order: a permutation of each batch element's gaussians that puts spatial
// neighbours next to each other, for the `order` argument of igs_backward_*.
//
// Why.  With narrow gaussians the backward can skip every pixel outside a gaussian's
// zero-weight box, but it skips per warp: the kernel for ordered calls
// (backward_warp.cu) gives each thread one gaussian and lets a warp stream only the
// rectangle of pixel blocks the box around its 32 gaussians meets.  Gaussians in arbitrary
// order leave every warp with gaussians all over the image and nothing to skip; in spatial
// order a warp's gaussians share a small patch.  The gradients do not depend on the order,
// bit for bit: each gaussian's sums are taken over the same pixels in the same sequence
// whichever thread owns it.
//
// How.  A counting sort on the Hilbert-curve index of the gaussian's cell in a 64 x 64 lattice laid
// over the sampled extent (first row of x, first column of y): count per cell, exclusive
// scan per batch element, scatter through an atomic cursor per cell.  The order inside a
// cell is whatever the atomics give, and may differ from run to run; it is a permutation
// every time, and that is all the backward needs.
#include "common.cuh"

namespace igs {

constexpr int ORDER_CELLS_1D = 64;
constexpr int ORDER_CELLS = ORDER_CELLS_1D * ORDER_CELLS_1D;  // 4096 curve positions
constexpr int ORDER_SCAN_THREADS = 1024;

struct OrderArgs {
    const float* pos;  // [B,N,2]
    const float* x;
    const float* y;
    long long xs_b, xs_w, ys_b, ys_h;
    int* hist;             // [B, ORDER_CELLS]: counts, then cursors
    unsigned short* keys;  // [B*N]
    int* order;            // [B,N]
    int B, N, H, W;
};

// Position of cell (x, y) along the Hilbert curve through the lattice.  Consecutive
// positions are adjacent cells, so ANY run of consecutive gaussians (a warp's, a CTA's)
// stays compact; the Morton order jumps across the image wherever a run straddles a
// quadrant boundary.
__device__ __forceinline__ unsigned hilbert_index(unsigned x, unsigned y) {
    unsigned d = 0;
#pragma unroll
    for (unsigned s = ORDER_CELLS_1D / 2; s > 0; s >>= 1) {
        const unsigned rx = (x & s) ? 1u : 0u, ry = (y & s) ? 1u : 0u;
        d += s * s * ((3u * rx) ^ ry);
        if (ry == 0) {  // rotate the quadrant so that the sub-curve enters and leaves at the right corners
            if (rx == 1) {
                x = (ORDER_CELLS_1D - 1) - x;
                y = (ORDER_CELLS_1D - 1) - y;
            }
            const unsigned t = x;
            x = y;
            y = t;
        }
    }
    return d;
}

__device__ __forceinline__ int cell_of(float p, float e0, float e1) {
    const float lo = fminf(e0, e1), hi = fmaxf(e0, e1);
    const float span = hi - lo;
    float t = span > 0.f ? (p - lo) / span * (float)ORDER_CELLS_1D : 0.f;
    t = fminf(fmaxf(t, 0.f), (float)(ORDER_CELLS_1D - 1));  // NaN -> 0
    return (int)t;
}

__global__ void __launch_bounds__(256) order_count_kernel(OrderArgs a) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.B * a.N) return;
    const long long b = i / a.N;
    const float x0 = a.x[b * a.xs_b], x1 = a.x[b * a.xs_b + (long long)(a.W - 1) * a.xs_w];
    const float y0 = a.y[b * a.ys_b], y1 = a.y[b * a.ys_b + (long long)(a.H - 1) * a.ys_h];
    const int cx = cell_of(a.pos[2 * i], x0, x1), cy = cell_of(a.pos[2 * i + 1], y0, y1);
    const unsigned key = hilbert_index((unsigned)cx, (unsigned)cy);
    a.keys[i] = (unsigned short)key;
    atomicAdd(a.hist + b * ORDER_CELLS + key, 1);
}

// One CTA per batch element: counts -> exclusive prefix sums (the cursors' start values).
__global__ void __launch_bounds__(ORDER_SCAN_THREADS) order_scan_kernel(OrderArgs a) {
    constexpr int PER = ORDER_CELLS / ORDER_SCAN_THREADS;
    __shared__ int s_warp[ORDER_SCAN_THREADS / 32];
    int* h = a.hist + (long long)blockIdx.x * ORDER_CELLS + threadIdx.x * PER;
    int v[PER], sum = 0;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        v[k] = h[k];
        sum += v[k];
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = s_warp[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w += t;
        }
        s_warp[lane] = w;
    }
    __syncthreads();
    int run = incl - sum + (warp ? s_warp[warp - 1] : 0);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        h[k] = run;
        run += v[k];
    }
}

__global__ void __launch_bounds__(256) order_scatter_kernel(OrderArgs a) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.B * a.N) return;
    const long long b = i / a.N;
    const int slot = atomicAdd(a.hist + b * ORDER_CELLS + a.keys[i], 1);
    // slot < N by construction (the cursors partition [0,N)); the guard keeps a corrupted
    // workspace from turning into a stray write
    if (slot >= 0 && slot < a.N) a.order[b * a.N + slot] = (int)(i - b * a.N);
}

static size_t order_hist_bytes(int B) { return ((size_t)B * ORDER_CELLS * sizeof(int) + 255) / 256 * 256; }

}  // namespace igs

using namespace igs;

extern "C" size_t igs_spatial_order_workspace_bytes(int B, int N) {
    if (B <= 0 || N <= 0) return 256;
    return order_hist_bytes(B) + ((size_t)B * N * sizeof(unsigned short) + 255) / 256 * 256;
}

extern "C" int igs_spatial_order(const float* positions, const float* x, const int64_t* x_strides, const float* y,
                                 const int64_t* y_strides, int B, int N, int H, int W, int* order, void* workspace,
                                 size_t workspace_bytes, int device, void* stream) {
    if (B < 0 || N < 0 || H < 1 || W < 1) return IGS_ERR_ARG;
    if (B == 0 || N == 0) return IGS_OK;
    if (!positions || !x || !y || !x_strides || !y_strides || !order) return IGS_ERR_ARG;
    if (!workspace || workspace_bytes < igs_spatial_order_workspace_bytes(B, N)) return IGS_ERR_WORKSPACE;
    if ((long long)B * N > 0x7fffffffLL * 256) return IGS_ERR_LIMIT;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t s = (cudaStream_t)stream;

    OrderArgs a;
    a.pos = positions;
    a.x = x;
    a.y = y;
    a.xs_b = x_strides[0];
    a.xs_w = x_strides[2];
    a.ys_b = y_strides[0];
    a.ys_h = y_strides[1];
    a.hist = reinterpret_cast<int*>(workspace);
    a.keys = reinterpret_cast<unsigned short*>(reinterpret_cast<unsigned char*>(workspace) + order_hist_bytes(B));
    a.order = order;
    a.B = B;
    a.N = N;
    a.H = H;
    a.W = W;

    cudaError_t e = cudaMemsetAsync(a.hist, 0, (size_t)B * ORDER_CELLS * sizeof(int), s);
    if (e != cudaSuccess) return (int)e;
    const unsigned blocks = (unsigned)(((long long)B * N + 255) / 256);
    order_count_kernel<<<blocks, 256, 0, s>>>(a);
    count_launch();
    order_scan_kernel<<<(unsigned)B, ORDER_SCAN_THREADS, 0, s>>>(a);
    count_launch();
    order_scatter_kernel<<<blocks, 256, 0, s>>>(a);
    count_launch();
    return (int)cudaGetLastError();
}
