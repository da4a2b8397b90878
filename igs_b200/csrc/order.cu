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
// How.  A stable counting sort on the Hilbert-curve index of the gaussian's cell in a 64 x 64
// lattice laid over the sampled extent (first row of x, first column of y).  Gaussians are
// taken in blocks of 1024: each block counts its gaussians per cell; one CTA per batch
// element turns the counts into the first slot of every (cell, block); each block then ranks
// its gaussians within their cells in index order (warp by warp, __match_any_sync inside a
// warp).  Equal cells keep their original order, no result depends on the timing of an
// atomic, so the permutation is the same on every run.
//
// What is sorted.  igs_spatial_order: the centres.  igs_spatial_order_boxes: per axis the
// centre of the gaussian's zero-weight box CLIPPED to the sampled extent.  A narrow gaussian
// inside the image keeps its own centre; a box that sticks out on one side is placed by how
// far it reaches in; a box that covers the whole extent lands on the image's centre line,
// next to all others like it.  A warp of the backward (a stage of the forward) then holds
// gaussians whose clipped boxes nearly coincide -- a patch, a vertical or horizontal strip,
// or everything -- where a single image-wide gaussian among narrow ones would make its whole
// warp visit every pixel.
#include <cstring>

#include "common.cuh"

namespace igs {

constexpr int ORDER_CELLS_1D = 64;
constexpr int ORDER_CELLS = ORDER_CELLS_1D * ORDER_CELLS_1D;  // 4096 curve positions
constexpr int ORDER_SCAN_THREADS = 1024;

struct OrderArgs {
    const float* pos;      // gaussian i's centre at pos[i * pos_stride], i over B*N
    const float* pos_off;  // NULL, or [B,N,2] added to the centres
    const float* scales;   // NULL (sort the centres), or gaussian i's two scales at scales[i * scale_stride]
    const float* rot;      // NULL (the larger scale stands in for both axes), or the angle at rot[i * rot_stride]
    long long pos_stride, scale_stride, rot_stride;
    int log_scales;        // the scales are given as logarithms
    const float* x;
    const float* y;
    long long xs_b, xs_w, ys_b, ys_h;
    int* block_hist;       // [B, n_blocks, ORDER_CELLS]: per block of 1024 gaussians, count then first slot
    unsigned short* keys;  // [B*N]
    int* order;            // [B,N]
    int B, N, H, W, n_blocks;
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

constexpr int ORDER_BLOCK = 1024;  // gaussians per sorting block

// A gaussian's zero-weight box reaches this many standard deviations of the axis to either
// side of the centre: sqrt(130 / (0.5 log2 e)) (the box pack_kernel computes, unrounded).
constexpr float ORDER_REACH = 13.43f;

__device__ __forceinline__ unsigned order_key(const OrderArgs& a, long long b, long long i) {
    const float x0 = a.x[b * a.xs_b], x1 = a.x[b * a.xs_b + (long long)(a.W - 1) * a.xs_w];
    const float y0 = a.y[b * a.ys_b], y1 = a.y[b * a.ys_b + (long long)(a.H - 1) * a.ys_h];
    float px = a.pos[i * a.pos_stride], py = a.pos[i * a.pos_stride + 1];
    if (a.pos_off) {
        px += a.pos_off[2 * i];
        py += a.pos_off[2 * i + 1];
    }
    if (a.scales) {
        float s0 = a.scales[i * a.scale_stride], s1 = a.scales[i * a.scale_stride + 1];
        if (a.log_scales) {
            s0 = expf(s0);
            s1 = expf(s1);
        }
        float hx, hy;
        if (a.rot) {
            const float c = cosf(a.rot[i * a.rot_stride]), c2 = c * c;
            const float v0 = s0 * s0, v1 = s1 * s1;
            hx = ORDER_REACH * sqrtf(c2 * v0 + (1.f - c2) * v1);  // variance along x, along y
            hy = ORDER_REACH * sqrtf(c2 * v1 + (1.f - c2) * v0);
        } else {
            hx = hy = ORDER_REACH * fmaxf(fabsf(s0), fabsf(s1));
        }
        const float lx = fminf(x0, x1), ux = fmaxf(x0, x1), ly = fminf(y0, y1), uy = fmaxf(y0, y1);
        px = 0.5f * (fmaxf(px - hx, lx) + fminf(px + hx, ux));
        py = 0.5f * (fmaxf(py - hy, ly) + fminf(py + hy, uy));
    }
    const int cx = cell_of(px, x0, x1), cy = cell_of(py, y0, y1);
    return hilbert_index((unsigned)cx, (unsigned)cy);
}

// grid (blocks of gaussians, B): keys and this block's count per cell
__global__ void __launch_bounds__(ORDER_BLOCK) order_count_kernel(OrderArgs a) {
    __shared__ int s_hist[ORDER_CELLS];
    const int b = blockIdx.y, blk = blockIdx.x;
    for (int c = threadIdx.x; c < ORDER_CELLS; c += ORDER_BLOCK) s_hist[c] = 0;
    __syncthreads();
    const int n = blk * ORDER_BLOCK + threadIdx.x;
    if (n < a.N) {
        const long long i = (long long)b * a.N + n;
        const unsigned key = order_key(a, b, i);
        a.keys[i] = (unsigned short)key;
        atomicAdd(&s_hist[key], 1);  // integer counts: the result does not depend on the order of the adds
    }
    __syncthreads();
    int* bh = a.block_hist + ((long long)b * a.n_blocks + blk) * ORDER_CELLS;
    for (int c = threadIdx.x; c < ORDER_CELLS; c += ORDER_BLOCK) bh[c] = s_hist[c];
}

// One CTA per batch element, a thread per four neighbouring cells: the cells' totals over the
// blocks, their exclusive prefix sums (first slot of every cell), and then, advancing block by
// block, each block's count replaced by the first slot of that (cell, block).
__global__ void __launch_bounds__(ORDER_SCAN_THREADS) order_scan_kernel(OrderArgs a) {
    constexpr int PER = ORDER_CELLS / ORDER_SCAN_THREADS;
    static_assert(PER == 4, "a thread moves its cells as one int4");
    __shared__ int s_warp[ORDER_SCAN_THREADS / 32];
    int4* bh = reinterpret_cast<int4*>(a.block_hist + (long long)blockIdx.x * a.n_blocks * ORDER_CELLS) + threadIdx.x;
    constexpr int ROW = ORDER_CELLS / 4;  // int4 per block of gaussians
    int4 tot = make_int4(0, 0, 0, 0);
#pragma unroll 8
    for (int blk = 0; blk < a.n_blocks; ++blk) {
        const int4 v = bh[(long long)blk * ROW];
        tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
    }
    const int sum = tot.x + tot.y + tot.z + tot.w;
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
    int4 run;
    run.x = incl - sum + (warp ? s_warp[warp - 1] : 0);
    run.y = run.x + tot.x;
    run.z = run.y + tot.y;
    run.w = run.z + tot.z;
#pragma unroll 8
    for (int blk = 0; blk < a.n_blocks; ++blk) {
        const int4 v = bh[(long long)blk * ROW];
        bh[(long long)blk * ROW] = run;
        run.x += v.x; run.y += v.y; run.z += v.z; run.w += v.w;
    }
}

// grid (blocks of gaussians, B): slot = first slot of (cell, block) + rank of the gaussian
// among the block's gaussians of that cell, in index order
__global__ void __launch_bounds__(ORDER_BLOCK) order_scatter_kernel(OrderArgs a) {
    __shared__ int s_next[ORDER_CELLS];
    const int b = blockIdx.y, blk = blockIdx.x;
    const int* bh = a.block_hist + ((long long)b * a.n_blocks + blk) * ORDER_CELLS;
    for (int c = threadIdx.x; c < ORDER_CELLS; c += ORDER_BLOCK) s_next[c] = bh[c];
    __syncthreads();
    const int n = blk * ORDER_BLOCK + threadIdx.x;
    const bool valid = n < a.N;
    // threads past the end share a key no gaussian has, so they match only each other
    const unsigned key = valid ? a.keys[(long long)b * a.N + n] : 0xffffffffu;
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const bool leader = rank == 0;
    for (int w = 0; w < ORDER_BLOCK / 32; ++w) {  // warps in index order
        if (warp == w && valid) {
            const int slot = s_next[key] + rank;
            // slot < N by construction; the guard keeps a corrupted workspace from turning into a stray write
            if (slot >= 0 && slot < a.N) a.order[(long long)b * a.N + slot] = n;
        }
        __syncthreads();
        if (warp == w && valid && leader) s_next[key] += __popc(peers);
        __syncthreads();
    }
}

static size_t order_align(size_t v) { return (v + 255) / 256 * 256; }
static int order_blocks(int N) { return (N + ORDER_BLOCK - 1) / ORDER_BLOCK; }

}  // namespace igs

using namespace igs;

extern "C" size_t igs_spatial_order_workspace_bytes(int B, int N) {
    if (B <= 0 || N <= 0) return 256;
    return order_align((size_t)B * order_blocks(N) * ORDER_CELLS * sizeof(int)) +
           order_align((size_t)B * N * sizeof(unsigned short));
}

static int spatial_order_impl(OrderArgs a, const int64_t* x_strides, const int64_t* y_strides, int B, int N, int H,
                              int W, int* order, void* workspace, size_t workspace_bytes, int device, void* stream) {
    if (B < 0 || N < 0 || H < 1 || W < 1) return IGS_ERR_ARG;
    if (B == 0 || N == 0) return IGS_OK;
    if (!a.pos || !a.x || !a.y || !x_strides || !y_strides || !order) return IGS_ERR_ARG;
    if (B > 65535) return IGS_ERR_LIMIT;
    if (!workspace || workspace_bytes < igs_spatial_order_workspace_bytes(B, N)) return IGS_ERR_WORKSPACE;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t s = (cudaStream_t)stream;

    a.xs_b = x_strides[0];
    a.xs_w = x_strides[2];
    a.ys_b = y_strides[0];
    a.ys_h = y_strides[1];
    a.n_blocks = order_blocks(N);
    unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
    a.block_hist = reinterpret_cast<int*>(ws);
    ws += order_align((size_t)B * a.n_blocks * ORDER_CELLS * sizeof(int));
    a.keys = reinterpret_cast<unsigned short*>(ws);
    a.order = order;
    a.B = B;
    a.N = N;
    a.H = H;
    a.W = W;

    const dim3 blocks((unsigned)a.n_blocks, (unsigned)B);
    order_count_kernel<<<blocks, ORDER_BLOCK, 0, s>>>(a);
    count_launch();
    order_scan_kernel<<<(unsigned)B, ORDER_SCAN_THREADS, 0, s>>>(a);
    count_launch();
    order_scatter_kernel<<<blocks, ORDER_BLOCK, 0, s>>>(a);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int igs_spatial_order(const float* positions, const float* x, const int64_t* x_strides, const float* y,
                                 const int64_t* y_strides, int B, int N, int H, int W, int* order, void* workspace,
                                 size_t workspace_bytes, int device, void* stream) {
    OrderArgs a;
    std::memset(&a, 0, sizeof(a));
    a.pos = positions;
    a.pos_stride = 2;
    a.x = x;
    a.y = y;
    return spatial_order_impl(a, x_strides, y_strides, B, N, H, W, order, workspace, workspace_bytes, device, stream);
}

extern "C" int igs_spatial_order_boxes(const float* positions, int64_t position_stride, const float* position_offsets,
                                       const float* scales, int64_t scale_stride, int log_scales,
                                       const float* rotations, int64_t rotation_stride, const float* x,
                                       const int64_t* x_strides, const float* y, const int64_t* y_strides, int B, int N,
                                       int H, int W, int* order, void* workspace, size_t workspace_bytes, int device,
                                       void* stream) {
    if (position_stride < 2 || (scales && scale_stride < 2) || (rotations && rotation_stride < 1)) return IGS_ERR_ARG;
    if (rotations && !scales) return IGS_ERR_ARG;
    OrderArgs a;
    std::memset(&a, 0, sizeof(a));
    a.pos = positions;
    a.pos_stride = position_stride;
    a.pos_off = position_offsets;
    a.scales = scales;
    a.scale_stride = scale_stride;
    a.log_scales = log_scales ? 1 : 0;
    a.rot = rotations;
    a.rot_stride = rotation_stride;
    a.x = x;
    a.y = y;
    return spatial_order_impl(a, x_strides, y_strides, B, N, H, W, order, workspace, workspace_bytes, device, stream);
}
