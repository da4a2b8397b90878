// Mean-squared-error loss and its gradient for the per-image fit loop: the L2 term the
// reference's fit scripts put behind the renderer (F.mse_loss(rendered_image, target_image),
// scripts/2dgs_img_comp.py:135, scripts/gs2d_test.py:56).  Two entry points so that the
// gradient can take the upstream scalar autograd hands to backward:
//   igs_mse_loss: loss = mean((out - target)^2)             (two launches: partials, finish)
//   igs_mse_grad: gout = upstream * 2 (out - target) / n    (one launch)
// No atomics: block partial sums are written to the workspace and added in a fixed order by
// one block, so the loss is repeatable to the bit.
//
// loss_terms_sep_kernel is the fused form for the per-image fit (igs_render_mse_sr): it
// takes the forward's un-normalised sums and does, in one pass over the image, what
// otherwise takes the normalisation, the two loss kernels, the loss-gradient kernel and the
// backward's pixel-terms kernel -- without ever writing the upstream gradient to memory.
#include "loss.cuh"

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

// One thread per 2-row x 4-column block of pixels (the unit of the separable backward's
// records).  Per pixel: S and the numerators summed over the gaussian splits in split order,
// out = R / (S + eps), d = out - target, the block's share of sum d^2, the upstream gradient
// g = k * d with k = upstream * 2 / n, and from it the backward's terms gn = g / (S + eps),
// gS = -sum_c g_c^2 / (S + eps)^2 (reference mode) or -sum_c gn_c * out_c (exact mode): the
// same expressions, in the same order, as reduce_normalize_kernel, mse_grad_kernel and
// pixel_terms_sep_kernel, so that the fused and the unfused path agree to the last bit in
// everything but the order in which the loss is added up.
// VEC: the image width is a multiple of four and every plane starts on a 16-byte boundary, so a
// thread's four pixels of a row are one 16-byte load or store per plane.
template <bool VEC>
__global__ void __launch_bounds__(LOSS_TERMS_THREADS) loss_terms_sep_kernel(LossTermArgs a) {
    extern __shared__ __align__(16) float s_rec[];  // [blockDim.x][record floats], then 8 floats for the block sum
    constexpr int CMAX = 4;  // channels of a chunk the separable backward takes
    const int rs = bwd_sep_rec_floats(a.ct), pf = bwd_sep_pair_floats(a.ct);
    const long long per_b = (long long)a.nrp * a.ncb;
    const long long total = (long long)a.B * per_b;
    const long long i_raw = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool in_range = i_raw < total;
    const long long i = in_range ? i_raw : total - 1;
    const long long b = i / per_b, blk = i - b * per_b;
    const int rp = (int)(blk / a.ncb), cbk = (int)(blk - (long long)rp * a.ncb);
    const long long HW = (long long)a.H * a.W;
    const int h0 = rp * 2, w0 = cbk * 4;
    const long long split_stride = (long long)a.B * (a.C + 1) * HW;
    const float* part_b = a.partial + b * (a.C + 1) * HW;
    const float k = (a.upstream ? *a.upstream : 1.f) * 2.f / (float)a.n_total;

    float* rec = s_rec + (size_t)threadIdx.x * rs;
    float xv[4], yv[2];
#pragma unroll
    for (int q = 0; q < 4; ++q) xv[q] = a.x[b * a.xs_b + (long long)min(w0 + q, a.W - 1) * a.xs_w];
#pragma unroll
    for (int q = 0; q < 2; ++q) yv[q] = a.y[b * a.ys_b + (long long)min(h0 + q, a.H - 1) * a.ys_h];
    reinterpret_cast<float4*>(rec)[0] = make_float4(xv[0], xv[1], xv[2], xv[3]);
    reinterpret_cast<float4*>(rec)[1] = make_float4(yv[0], yv[1], 0.f, 0.f);

    // four pixels of one row of one plane (columns past the end repeat the last one)
    auto load4 = [&](const float* plane, long long row_off, float (&v)[4]) {
        if constexpr (VEC) {
            const float4 t = *reinterpret_cast<const float4*>(plane + row_off + w0);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] = plane[row_off + min(w0 + q, a.W - 1)];
        }
    };
    auto store4 = [&](float* plane, long long row_off, const float (&v)[4]) {
        if constexpr (VEC) {
            *reinterpret_cast<float4*>(plane + row_off + w0) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (w0 + q < a.W) plane[row_off + w0 + q] = v[q];
        }
    };

    // The sums over the gaussian splits, in split order, for both rows at once: the loads of
    // one split (two rows x (C + 1) planes) are independent of each other and all in flight
    // together; the kernel is bound by their latency, not by bandwidth.
    long long row_off2[2];
    float S2[2][4], R2[2][CMAX][4], T2[2][CMAX][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_off2[r] = (long long)min(h0 + r, a.H - 1) * a.W;
#pragma unroll
        for (int q = 0; q < 4; ++q) S2[r][q] = 0.f;
#pragma unroll
        for (int c = 0; c < CMAX; ++c) {
#pragma unroll
            for (int q = 0; q < 4; ++q) R2[r][c][q] = T2[r][c][q] = 0.f;
            if (c < a.C) load4(a.target + (b * a.C + c) * HW, row_off2[r], T2[r][c]);
        }
    }
    for (int sp = 0; sp < a.n_split; ++sp) {
        const float* ps = part_b + sp * split_stride;
        float tS[2][4], tR[2][CMAX][4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            load4(ps + (long long)a.C * HW, row_off2[r], tS[r]);
#pragma unroll
            for (int c = 0; c < CMAX; ++c)
                if (c < a.C) load4(ps + (long long)c * HW, row_off2[r], tR[r][c]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int q = 0; q < 4; ++q) S2[r][q] += tS[r][q];
#pragma unroll
            for (int c = 0; c < CMAX; ++c)
                if (c < a.C) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) R2[r][c][q] += tR[r][c][q];
                }
        }
    }

    bool bad = false;
    float lsum = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const bool row_valid = in_range && (h0 + r < a.H);
        const long long row_off = row_off2[r];
        float (&S)[4] = S2[r];
        float (&R)[CMAX][4] = R2[r];
        float (&T)[CMAX][4] = T2[r];
        float O[CMAX][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bool valid = row_valid && (w0 + q < a.W);
            const float Sp = S[q] + a.eps;
            float acc = 0.f;
            // pixel (r, q) is lane q & 1 of pixel pair 2 * r + (q >> 1)
            float* pr = rec + 8 + (r * 2 + (q >> 1)) * pf + (q & 1);
#pragma unroll
            for (int c = 0; c < CMAX; ++c) {
                O[c][q] = 0.f;
                if (c >= pf / 2 - 1) continue;
                float gn = 0.f;
                if (c < a.C) {
                    const float o = R[c][q] / Sp;
                    const float d = o - T[c][q];
                    const float g = k * d;
                    O[c][q] = o;
                    if (valid) lsum = fmaf(d, d, lsum);
                    acc += (a.mode == IGS_GRAD_REFERENCE) ? g * g : (g / Sp) * o;
                    gn = valid ? g / Sp : 0.f;
                    bad |= !isfinite(gn);
                }
                pr[2 + 2 * c] = gn;
            }
            const float gS = valid ? ((a.mode == IGS_GRAD_REFERENCE) ? -acc / (Sp * Sp) : -acc) : 0.f;
            bad |= !isfinite(gS);
            pr[0] = gS;
        }
        if (row_valid) {
            if (a.out) {
#pragma unroll
                for (int c = 0; c < CMAX; ++c)
                    if (c < a.C) store4(a.out + (b * a.C + c) * HW, row_off, O[c]);
            }
            if (a.wsum) store4(a.wsum + b * HW, row_off, S);
        }
    }
    __syncthreads();
    {
        // the CTA writes its records out in consecutive 16-byte pieces
        const long long first = (long long)blockIdx.x * blockDim.x;
        const long long n_here = total - first < (long long)blockDim.x ? total - first : (long long)blockDim.x;
        float4* dst = reinterpret_cast<float4*>(a.prec + first * rs);
        const float4* src4 = reinterpret_cast<const float4*>(s_rec);
        for (long long j = threadIdx.x; j < n_here * (rs / 4); j += blockDim.x) dst[j] = src4[j];
    }
    if (bad && a.flags) atomicOr(a.flags, UPSTREAM_NOT_FINITE);
    // this CTA's share of the loss (added up in a fixed order: repeatable to the bit)
    float* s_warp = s_rec + (size_t)blockDim.x * rs;
    __syncthreads();
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, d);
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = lsum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < LOSS_TERMS_THREADS / 32; ++w) t += s_warp[w];
        a.loss_partial[blockIdx.x] = t;
    }
}

long long loss_terms_blocks(int B, int nrp, int ncb) {
    return ((long long)B * nrp * ncb + LOSS_TERMS_THREADS - 1) / LOSS_TERMS_THREADS;
}

cudaError_t launch_loss_terms_sep(const LossTermArgs& a, float* loss, cudaStream_t s) {
    const long long blocks = loss_terms_blocks(a.B, a.nrp, a.ncb);
    if (blocks <= 0) return cudaSuccess;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (a.C > 4) return cudaErrorInvalidValue;  // (a chunk of the separable backward has at most four channels)
    const size_t smem = (size_t)LOSS_TERMS_THREADS * bwd_sep_rec_floats(a.ct) * sizeof(float) + 8 * sizeof(float);
    auto aligned16 = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = a.W % 4 == 0 && aligned16(a.partial) && aligned16(a.target) && aligned16(a.out) && aligned16(a.wsum);
    {
        KernelTimer timer(K_PIXEL_TERMS, s);
        if (vec)
            loss_terms_sep_kernel<true><<<(unsigned)blocks, LOSS_TERMS_THREADS, smem, s>>>(a);
        else
            loss_terms_sep_kernel<false><<<(unsigned)blocks, LOSS_TERMS_THREADS, smem, s>>>(a);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    mse_finish_kernel<<<1, MSE_THREADS, 0, s>>>(a.loss_partial, (int)blocks, a.n_total, loss);
    count_launch();
    return cudaGetLastError();
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
