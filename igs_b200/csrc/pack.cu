// Per-gaussian prologue kernel: one thread per gaussian turns the caller's raw
// parameters into the geometry record (backward) and the forward records (one array per
// channel chunk), and measures how far the gaussian reaches.
//
// Reach.  With the exponent q = A dx^2 + B2 dx dy + Cq dy^2 in log2 units, the weight
// ex2.approx.ftz(q) is exactly zero once q < -126 (results below 2^-126 are flushed).  For a
// negative-definite form the set q >= -CULL_T is an ellipse whose bounding box has the
// half-widths hx = sqrt(r2 cov_xx), hy = sqrt(r2 cov_yy) with cov the covariance (the inverse
// of cov_inv) and r2 = CULL_T / (0.5 log2 e); a pixel outside that box receives exactly
// nothing from the gaussian, which is what lets the splat kernels skip (gaussian, pixel
// tile) combinations without changing a bit of the result.  An indefinite form has no such
// box: hx = hy = +inf.
#include "pack.cuh"

namespace igs {

__global__ void __launch_bounds__(256) pack_kernel(PackArgs a) {
    // `slot` is where the records go, `i` the gaussian they describe: the same unless the
    // caller asked for the forward records in a given order
    const long long slot = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    bool narrow = false;
    if (slot < a.M) {
        // (an entry that is no index is clamped: wrong output for a malformed order, never a stray read)
        const long long i = a.order ? slot / a.N * a.N + min(max(a.order[slot], 0), a.N - 1) : slot;
        const ParamLayout& L = a.lay;
        float px = a.pos[(long long)L.pos_s * i], py = a.pos[(long long)L.pos_s * i + 1];
        if (L.pos_off) {
            px += L.pos_off[2 * i];
            py += L.pos_off[2 * i + 1];
        }
        float c00, c01, c11;
        float hx = INFINITY, hy = INFINITY;
        // Reach: the ellipse d^T cov_inv d <= r2 (r2 = CULL_T / (0.5 log2 e)) has the bounding
        // box half-widths sqrt(r2 * cov_xx), sqrt(r2 * cov_yy).  A little wider than exact
        // (factor 1.001 on top of the 130-against-126 margin of CULL_T), so that fp32 rounding
        // here can never cull a non-zero weight.
        const float r2 = CULL_T / -EXP2_SCALE;
        if (a.kind == SHAPE_SCALE_ROT) {
            float sx = a.shape0[(long long)L.s0_s * i], sy = a.shape0[(long long)L.s0_s * i + 1];
            if (L.log_scale) {
                sx = expf(sx) + a.eps;
                sy = expf(sy) + a.eps;
            }
            const CovInv ci = cov_inv_from_scale_rot(sx, sy, a.shape1[(long long)L.s1_s * i], a.eps);
            c00 = ci.c00;
            c01 = ci.c01;
            c11 = ci.c11;
            // the covariance itself is at hand (sums of squares: nothing cancels, however
            // anisotropic or rotated the gaussian is)
            hx = 1.001f * sqrtf(r2 * ci.a);
            hy = 1.001f * sqrtf(r2 * ci.d);
        } else {
            c00 = a.shape0[i];
            c01 = a.shape1[i];
            c11 = a.shape2[i];
            // cov = inverse of the caller's matrix: its determinant cancels for strongly
            // anisotropic rotated gaussians, so it is formed in double, and a form that is
            // not safely positive definite gets no box at all
            const double d00 = c00, d01 = c01, d11 = c11;
            const double det = d00 * d11 - d01 * d01;
            if (d00 > 0.0 && d11 > 0.0 && det > 1e-6 * d00 * d11) {
                hx = 1.001f * (float)sqrt((double)r2 * d11 / det);
                hy = 1.001f * (float)sqrt((double)r2 * d00 / det);
            }
        }
        if (!(hx == hx) || !(hy == hy)) hx = hy = INFINITY;
        const float A = EXP2_SCALE * c00, B2 = 2.0f * EXP2_SCALE * c01, Cq = EXP2_SCALE * c11;
        const float al = a.alpha ? a.alpha[i] : 1.0f;

        // 0 * NaN is NaN: a gaussian with a non-finite parameter must reach every pixel, as in
        // the reference (its weights, or their products with alpha and the colours, are NaN)
        bool finite = isfinite(px) && isfinite(py) && isfinite(A) && isfinite(B2) && isfinite(Cq) && isfinite(al);
        for (int c = 0; c < a.C; ++c) finite = finite && isfinite(a.colors[i * L.col_s + c]);
        if (!finite) hx = hy = INFINITY;
        if (a.narrow_count && a.x && a.W > 1 && a.H > 1) {
            // "narrow" = the box covers less than three quarters of the sampled extent in x or y
            const long long b = i / a.N;
            const float x0 = a.x[b * a.xs_b], x1 = a.x[b * a.xs_b + (long long)(a.W - 1) * a.xs_w];
            const float y0 = a.y[b * a.ys_b], y1 = a.y[b * a.ys_b + (long long)(a.H - 1) * a.ys_h];
            narrow = (2.f * hx < 0.75f * fabsf(x1 - x0)) || (2.f * hy < 0.75f * fabsf(y1 - y0));
        }

        if (a.geo) {
            // (indexed by the gaussian, not by the slot: the backward kernels follow the order themselves)
            float4* g = reinterpret_cast<float4*>(a.geo + i * GEO_FLOATS);
            g[0] = make_float4(px, py, A, B2);
            g[1] = make_float4(Cq, al, hx, hy);
        }
        for (int k = 0; k < a.ch.n; ++k) {
            float* rec = a.frec[k];
            if (!rec) continue;
            const int ct = a.ch.ct[k], cr = a.ch.cr[k], c0 = a.ch.c0[k];
            const int rs = fwd_rec_floats(ct);
            float* r = rec + slot * rs;
            r[0] = px; r[1] = py; r[2] = A; r[3] = B2; r[4] = Cq; r[5] = al;
            // colours pre-multiplied by alpha: numerator += e * (alpha * colour)
            for (int c = 0; c < ct; ++c) r[6 + c] = (c < cr) ? al * a.colors[i * L.col_s + c0 + c] : 0.f;
            r[6 + ct] = hx;
            r[7 + ct] = hy;
            for (int c = 8 + ct; c < rs; ++c) r[c] = 0.f;
        }
    }
    if (a.narrow_count) {
        const int n = __syncthreads_count(narrow);
        if (threadIdx.x == 0 && n) atomicAdd(a.narrow_count, n);
    }
    // Are the first row of x and the first column of y non-decreasing?  (The separable
    // backward kernel takes the ends of a run of columns as its x range when it skips.)
    if (a.grid_flag && a.x) {
        bool bad = false;
        const long long per_b = (long long)a.W + a.H, total = a.B * per_b;
        for (long long j = slot; j < total; j += (long long)gridDim.x * blockDim.x) {
            const long long b = j / per_b, k = j - b * per_b;
            if (k < a.W - 1) {
                const float* p = a.x + b * a.xs_b + k * a.xs_w;
                bad |= !(p[0] <= p[a.xs_w]);
            } else if (k >= a.W && k - a.W < a.H - 1) {
                const float* p = a.y + b * a.ys_b + (k - a.W) * a.ys_h;
                bad |= !(p[0] <= p[a.ys_h]);
            }
        }
        if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(a.grid_flag, GRID_NOT_MONOTONE);
    }
}

// Box {x0, x1, y0, y1} around the zero-weight boxes of the gaussians of one forward stage
// (chunk_g consecutive records), read back from the records pack_kernel wrote.
__global__ void __launch_bounds__(128) stage_box_kernel(PackArgs a, int n_stages) {
    __shared__ float s_box[4][4];
    const int b = blockIdx.y, stage = blockIdx.x;
    const int ct = a.ch.ct[0], rs = fwd_rec_floats(ct);
    float u[4] = {INFINITY, -INFINITY, INFINITY, -INFINITY};
    for (int k = threadIdx.x; k < a.chunk_g; k += blockDim.x) {
        const int slot = stage * a.chunk_g + k;
        if (slot >= a.N) break;
        const float* r = a.frec[0] + ((long long)b * a.N + slot) * rs;
        const float gx = r[0], gy = r[1], hx = r[6 + ct], hy = r[7 + ct];
        // a NaN anywhere makes the box NaN-free but infinite: such a stage is never skipped
        const bool bad = !(gx == gx) || !(gy == gy) || !(hx == hx) || !(hy == hy);
        u[0] = fminf(u[0], bad ? -INFINITY : gx - hx);
        u[1] = fmaxf(u[1], bad ? INFINITY : gx + hx);
        u[2] = fminf(u[2], bad ? -INFINITY : gy - hy);
        u[3] = fmaxf(u[3], bad ? INFINITY : gy + hy);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        u[0] = fminf(u[0], __shfl_xor_sync(0xffffffffu, u[0], d));
        u[1] = fmaxf(u[1], __shfl_xor_sync(0xffffffffu, u[1], d));
        u[2] = fminf(u[2], __shfl_xor_sync(0xffffffffu, u[2], d));
        u[3] = fmaxf(u[3], __shfl_xor_sync(0xffffffffu, u[3], d));
    }
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) s_box[threadIdx.x >> 5][k] = u[k];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 4; ++w) {
            u[0] = fminf(u[0], s_box[w][0]);
            u[1] = fmaxf(u[1], s_box[w][1]);
            u[2] = fminf(u[2], s_box[w][2]);
            u[3] = fmaxf(u[3], s_box[w][3]);
        }
        reinterpret_cast<float4*>(a.cbox)[(long long)b * n_stages + stage] = make_float4(u[0], u[1], u[2], u[3]);
    }
}

cudaError_t launch_stage_boxes(const PackArgs& a, cudaStream_t s) {
    if (!a.cbox || !a.frec[0] || a.chunk_g <= 0 || a.N <= 0 || a.B <= 0) return cudaSuccess;
    const int n_stages = (a.N + a.chunk_g - 1) / a.chunk_g;
    stage_box_kernel<<<dim3((unsigned)n_stages, (unsigned)a.B), 128, 0, s>>>(a, n_stages);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_pack(const PackArgs& a, cudaStream_t s) {
    if (a.M <= 0) return cudaSuccess;
    const int threads = 256;
    const long long blocks = (a.M + threads - 1) / threads;
    // (a.narrow_count and a.grid_flag are words of the status area, which the caller cleared)
    {
        KernelTimer timer(K_PACK, s);
        pack_kernel<<<(unsigned)blocks, threads, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace igs
