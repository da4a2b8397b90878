// Mean-squared-error loss and its gradient for the per-image fit loop: the L2 term the
// reference's fit scripts put behind the renderer (F.mse_loss(rendered_image, target_image),
// scripts/2dgs_img_comp.py:135, scripts/gs2d_test.py:56).  Two entry points so that the
// gradient can take the upstream scalar autograd hands to backward:
//   igs_mse_loss: loss = mean((out - target)^2)             (two launches: partials, finish)
//   igs_mse_grad: gout = upstream * 2 (out - target) / n    (one launch)
// No atomics: block partial sums are written to the workspace and added in a fixed order by
// one block, so the loss is repeatable to the bit.
#include "common.cuh"

namespace igs {

constexpr int MSE_THREADS = 256;
constexpr int MSE_MAX_BLOCKS = 1024;

__device__ __forceinline__ float block_sum(float v, float* s_warp) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    if (threadIdx.x < 32) {
        t = threadIdx.x < MSE_THREADS / 32 ? s_warp[threadIdx.x] : 0.f;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
    }
    return t;  // valid in thread 0
}

__global__ void __launch_bounds__(MSE_THREADS) mse_partial_kernel(const float* __restrict__ out,
                                                                  const float* __restrict__ target, long long n,
                                                                  float* __restrict__ partial) {
    __shared__ float s_warp[MSE_THREADS / 32];
    float acc = 0.f;
    const long long stride = (long long)gridDim.x * MSE_THREADS;
    for (long long i = (long long)blockIdx.x * MSE_THREADS + threadIdx.x; i < n; i += stride) {
        const float d = out[i] - target[i];
        acc = fmaf(d, d, acc);
    }
    const float t = block_sum(acc, s_warp);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

__global__ void __launch_bounds__(MSE_THREADS) mse_finish_kernel(const float* __restrict__ partial, int n_partial,
                                                                 long long n, float* __restrict__ loss) {
    __shared__ float s_warp[MSE_THREADS / 32];
    float acc = 0.f;
    for (int i = threadIdx.x; i < n_partial; i += MSE_THREADS) acc += partial[i];
    const float t = block_sum(acc, s_warp);
    if (threadIdx.x == 0) *loss = t / (float)n;
}

__global__ void __launch_bounds__(MSE_THREADS) mse_grad_kernel(const float* __restrict__ out,
                                                               const float* __restrict__ target, long long n,
                                                               const float* __restrict__ upstream,
                                                               float* __restrict__ gout) {
    const float k = (upstream ? *upstream : 1.f) * 2.f / (float)n;
    const long long stride = (long long)gridDim.x * MSE_THREADS;
    for (long long i = (long long)blockIdx.x * MSE_THREADS + threadIdx.x; i < n; i += stride)
        gout[i] = k * (out[i] - target[i]);
}

static int mse_blocks(long long n) {
    const long long want = (n + 4LL * MSE_THREADS - 1) / (4LL * MSE_THREADS);  // about 4 elements per thread
    return (int)(want < 1 ? 1 : (want > MSE_MAX_BLOCKS ? MSE_MAX_BLOCKS : want));
}

}  // namespace igs

using namespace igs;

extern "C" int igs_mse_loss(const float* out, const float* target, long long n, float* loss, void* workspace,
                            size_t workspace_bytes, int device, void* stream) {
    if (!out || !target || !loss || n <= 0) return IGS_ERR_ARG;
    if (!workspace || workspace_bytes < IGS_MSE_WORKSPACE_BYTES) return IGS_ERR_WORKSPACE;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = mse_blocks(n);
    float* partial = static_cast<float*>(workspace);
    mse_partial_kernel<<<blocks, MSE_THREADS, 0, s>>>(out, target, n, partial);
    count_launch();
    mse_finish_kernel<<<1, MSE_THREADS, 0, s>>>(partial, blocks, n, loss);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int igs_mse_grad(const float* out, const float* target, long long n, const float* upstream, float* gout,
                            int device, void* stream) {
    if (!out || !target || !gout || n <= 0) return IGS_ERR_ARG;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    mse_grad_kernel<<<mse_blocks(n), MSE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(out, target, n, upstream, gout);
    count_launch();
    return (int)cudaGetLastError();
}
