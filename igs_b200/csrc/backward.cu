// Backward splat kernels (sm_100a).
//
// The weights are recomputed, never cached.  The roles of the forward kernel are
// swapped: one THREAD owns one gaussian (parameters and all of its gradient sums live
// in registers), one CTA owns a group of gaussians and a slab of pixels, and the
// per-pixel upstream terms stream through shared memory as pair records
//   {x0,x1, y0,y1, gS0,gS1, gn_c0,gn_c1 ...}
// filled by 1-D bulk (TMA) copies.  Every lane reads the same record (broadcast), so
// the reduction over pixels needs no shuffles and no atomics: it is a register
// accumulation, folded per stage into a second-level accumulator, and one partial per
// (slab, gaussian) that finalize_kernel adds in slab order.
//
// Per gaussian x pixel, with h = G*e and G = gS + sum_c gn_c*colour_c:
//   M0 += h; Mx += h*dx; My += h*dy; Mxx += h*dx*dx; Mxy += h*dx*dy; Myy += h*dy*dy;
//   E_c += gn_c*e
// 22 FMA-pipe instructions and one MUFU at C = 3, all f32x2 over the two pixels of a
// pair.  finalize_kernel turns the sums into the reference's gradients:
//   d_alpha = M0                    d_colour_c = alpha*E_c
//   d_c00 = -alpha/2*Mxx   d_c11 = -alpha/2*Myy   d_c01 = -alpha*Mxy
//   d_px = alpha*(c00*Mx + c01*My)  d_py = alpha*(c11*My + c01*Mx)
// and, for the scale/rotation entry, chains d_c** through the closed-form inverse.
#include "backward.cuh"

namespace igs {

// ---------------------------------------------------------------------------
// per-pixel upstream terms
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pixel_terms_kernel(PixelTermArgs a) {
    if (a.grid_sel && !(*a.grid_sel & GRID_NOT_SEPARABLE)) return;  // separable grid: the block-record kernel runs
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over B*npairs
    if (i >= (long long)a.B * a.npairs) return;
    const long long b = i / a.npairs, pair = i - b * a.npairs;
    const long long HW = (long long)a.H * a.W;
    float xv[2], yv[2], inv_ok[2], Sp[2], gS[2] = {0.f, 0.f};
    long long pp[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        long long p = pair * 2 + k;
        inv_ok[k] = 1.f;
        if (p >= HW) {  // odd pixel count: repeat the last pixel with zero upstream terms
            p = HW - 1;
            inv_ok[k] = 0.f;
        }
        pp[k] = p;
        const long long h = p / a.W, w = p - h * a.W;
        xv[k] = a.x[b * a.xs_b + h * a.xs_h + w * a.xs_w];
        yv[k] = a.y[b * a.ys_b + h * a.ys_h + w * a.ys_w];
        Sp[k] = a.wsum[b * HW + p] + a.eps;
    }
    // gS, summed over ALL channels (first chunk carries it)
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        float acc = 0.f;
        for (int c = 0; c < a.C; ++c) {
            const float g = a.gout[(b * a.C + c) * HW + pp[k]];
            if (a.mode == IGS_GRAD_REFERENCE)
                acc += g * g;
            else
                acc += (g / Sp[k]) * a.out[(b * a.C + c) * HW + pp[k]];
        }
        gS[k] = (a.mode == IGS_GRAD_REFERENCE) ? -acc / (Sp[k] * Sp[k]) : -acc;
        gS[k] *= inv_ok[k];
    }
    for (int q = 0; q < a.ch.n; ++q) {
        const int ct = a.ch.ct[q], cr = a.ch.cr[q], c0 = a.ch.c0[q];
        const int rs = bwd_rec_floats(ct);
        float* r = a.prec[q] + i * rs;
        r[0] = xv[0];
        r[1] = xv[1];
        r[2] = yv[0];
        r[3] = yv[1];
        r[4] = q == 0 ? gS[0] : 0.f;
        r[5] = q == 0 ? gS[1] : 0.f;
        for (int c = 0; c < rs / 2 - 3; ++c) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                float v = 0.f;
                if (c < cr) v = inv_ok[k] * (a.gout[(b * a.C + c0 + c) * HW + pp[k]] / Sp[k]);
                r[6 + 2 * c + k] = v;
            }
        }
    }
}

cudaError_t launch_pixel_terms(const PixelTermArgs& a, bool separable, cudaStream_t s) {
    if (separable) return a.axes ? launch_pixel_terms_row(a, s) : launch_pixel_terms_sep(a, s);
    const long long n = (long long)a.B * a.npairs;
    if (n <= 0) return cudaSuccess;
    {
        KernelTimer timer(K_PIXEL_TERMS, s);
        pixel_terms_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// main backward kernel
// ---------------------------------------------------------------------------
// GPT = gaussians per thread.  A pair record costs one shared-memory read per thread
// whatever GPT is, and a 16-byte broadcast read occupies the shared-memory return path
// for four cycles per warp, so with GPT = 1 the 3 reads per pixel pair (C = 3) need
// more return-path cycles than the 22 f32x2 instructions need FMA-pipe cycles; GPT = 2
// halves the reads per evaluation and makes the FMA pipe the limiter again.
constexpr int BWD_GPT = 2;
// gaussians per thread in the 16-channel instantiation (165 registers, 12 warps per SM:
// 248.8 ms against 254.7 ms with one, B=8 N=65536 512x512)
constexpr int BWD_GPT_16 = 2;

template <int CT, int GPT>
struct BwdCfg {
    static constexpr int THREADS = 128;
    static constexpr int GAUSS_PER_CTA = THREADS * GPT;
    static constexpr int CHUNK_PAIRS = CT <= 4 ? 256 : 128;
    static constexpr int STAGES = 2;
    static constexpr int MIN_CTAS = CT <= 4 ? 5 : (CT <= 8 ? 4 : 3);
    static constexpr int UNROLL = CT > 4 ? (GPT >= 2 ? 1 : 2) : (GPT >= 2 ? 4 : 2);
    static constexpr bool TWO_LEVEL = (CT <= 4 && GPT == 1);
    static constexpr int RS = bwd_rec_floats(CT);
    static constexpr int NACC = N_MOMENTS + CT;
    static constexpr size_t SMEM = (size_t)STAGES * CHUNK_PAIRS * RS * sizeof(float) + STAGES * sizeof(uint64_t) + 16;
};

template <int CT, int GPT>
__global__ void __launch_bounds__(BwdCfg<CT, GPT>::THREADS, BwdCfg<CT, GPT>::MIN_CTAS)
    splat_backward_kernel(BwdArgs a) {
    using Cfg = BwdCfg<CT, GPT>;
    constexpr int T = Cfg::THREADS, PC = Cfg::CHUNK_PAIRS, NS = Cfg::STAGES, RS = Cfg::RS, NACC = Cfg::NACC;

    if (a.grid_sel && !(*a.grid_sel & GRID_NOT_SEPARABLE)) return;  // separable grid: splat_backward_sep_kernel runs

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage_base = reinterpret_cast<float*>(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NS * PC * RS * sizeof(float));
    int* s_failed = reinterpret_cast<int*>(bars + NS);

    const int tid = threadIdx.x;
    const int b = blockIdx.z, slab = blockIdx.y;

    // ---- this thread's gaussians ----
    int n[GPT];
    f2 px[GPT], py[GPT], A[GPT], B2[GPT], Cq[GPT], col[GPT][CT];
#pragma unroll
    for (int g = 0; g < GPT; ++g) {
        // slot in processing order -> gaussian index (a caller-supplied spatial order puts
        // neighbours into the same warp; without one the order is the identity)
        const int slot = a.order ? blockIdx.x * Cfg::GAUSS_PER_CTA + tid * GPT + g
                                 : blockIdx.x * Cfg::GAUSS_PER_CTA + g * T + tid;
        n[g] = slot < a.N ? (a.order ? a.order[(long long)b * a.N + slot] : slot) : a.N;
        if ((unsigned)n[g] > (unsigned)a.N) n[g] = a.N;  // an entry that is no index: the slot stays empty
        const int nn = n[g] < a.N ? n[g] : a.N - 1;
        const float4* gp = reinterpret_cast<const float4*>(a.geo + ((long long)b * a.N + nn) * GEO_FLOATS);
        const float4 g0 = gp[0], g1 = gp[1];
        px[g] = pk(g0.x, g0.x);
        py[g] = pk(g0.y, g0.y);
        A[g] = pk(g0.z, g0.z);
        B2[g] = pk(g0.w, g0.w);
        Cq[g] = pk(g1.x, g1.x);
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const float v = (c < a.cr) ? a.colors[((long long)b * a.N + nn) * a.C + a.c0 + c] : 0.f;
            col[g][c] = pk(v, v);
        }
    }

    f2 tot[GPT][NACC];
#pragma unroll
    for (int g = 0; g < GPT; ++g)
#pragma unroll
        for (int k = 0; k < NACC; ++k) tot[g][k] = 0ull;

    // ---- pixel slab, streamed in stages ----
    const long long pair_begin = (long long)slab * a.pairs_per_slab;
    const long long pair_end = min(a.npairs, pair_begin + a.pairs_per_slab);
    const int n_total = (int)max(0ll, pair_end - pair_begin);
    const int n_chunks = (n_total + PC - 1) / PC;
    const float* src = a.prec + ((long long)b * a.npairs + pair_begin) * RS;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
        *s_failed = 0;
        mbar_init_fence();
    }
    __syncthreads();

    auto issue = [&](int chunk) {
        const int st = chunk % NS;
        const int cnt = min(PC, n_total - chunk * PC);
        const uint32_t bytes = (uint32_t)cnt * RS * sizeof(float);
        mbar_expect_tx(&bars[st], bytes);
        bulk_g2s(stage_base + (size_t)st * PC * RS, src + (long long)chunk * PC * RS, bytes, &bars[st]);
    };
    if (tid == 0) {
        for (int c = 0; c < NS && c < n_chunks; ++c) issue(c);
    }

    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        const int st = chunk % NS;
        const uint32_t parity = (chunk / NS) & 1;
        if (!mbar_wait_bounded(&bars[st], parity)) *s_failed = 1;
        __syncthreads();
        if (*s_failed) {
            if (tid == 0) {
                for (int c = chunk + 1; c < n_chunks && c < chunk + NS; ++c)
                    mbar_wait_bounded(&bars[c % NS], (c / NS) & 1);
                atomicOr(a.status, STATUS_WAIT_TIMEOUT);
            }
            return;
        }
        const int cnt = min(PC, n_total - chunk * PC);
        const ulonglong2* rec = reinterpret_cast<const ulonglong2*>(stage_base + (size_t)st * PC * RS);

        f2 acc[GPT][NACC];
#pragma unroll
        for (int g = 0; g < GPT; ++g)
#pragma unroll
            for (int k = 0; k < NACC; ++k) acc[g][k] = Cfg::TWO_LEVEL ? 0ull : tot[g][k];

#pragma unroll(Cfg::UNROLL)
        for (int i = 0; i < cnt; ++i) {
            const ulonglong2* r = rec + (size_t)i * (RS / 4);
            const ulonglong2 r0 = r[0];  // {x0,x1},{y0,y1}
            f2 gterm[CT + 2];            // gS, gn_0 .. gn_{CT-1} (+ pad)
#pragma unroll
            for (int c = 0; c < (CT + 2) / 2; ++c) {
                const ulonglong2 rc = r[1 + c];
                gterm[2 * c] = rc.x;
                gterm[2 * c + 1] = rc.y;
            }
#pragma unroll
            for (int g = 0; g < GPT; ++g) {
                const f2 dx = sub2(r0.x, px[g]);
                const f2 dy = sub2(r0.y, py[g]);
                const f2 t = fma2(A[g], dx, mul2(B2[g], dy));
                const f2 v = mul2(mul2(Cq[g], dy), dy);
                const f2 e = ex2_2(fma2(dx, t, v));
                f2 G = gterm[0];
#pragma unroll
                for (int c = 0; c < CT; ++c) G = fma2(gterm[1 + c], col[g][c], G);
                const f2 h = mul2(G, e);
                acc[g][0] = add2(acc[g][0], h);
                const f2 hx = mul2(h, dx), hy = mul2(h, dy);
                acc[g][1] = add2(acc[g][1], hx);
                acc[g][2] = add2(acc[g][2], hy);
                acc[g][3] = fma2(hx, dx, acc[g][3]);
                acc[g][4] = fma2(hx, dy, acc[g][4]);
                acc[g][5] = fma2(hy, dy, acc[g][5]);
#pragma unroll
                for (int c = 0; c < CT; ++c) acc[g][N_MOMENTS + c] = fma2(gterm[1 + c], e, acc[g][N_MOMENTS + c]);
            }
        }
#pragma unroll
        for (int g = 0; g < GPT; ++g)
#pragma unroll
            for (int k = 0; k < NACC; ++k) tot[g][k] = Cfg::TWO_LEVEL ? add2(tot[g][k], acc[g][k]) : acc[g][k];
        __syncthreads();
        if (tid == 0 && chunk + NS < n_chunks) issue(chunk + NS);
    }

#pragma unroll
    for (int g = 0; g < GPT; ++g) {
        if (n[g] >= a.N) continue;
        // (the partial sums are laid out by slot, not by gaussian: recomputed here, not kept)
        const int slot = a.order ? blockIdx.x * Cfg::GAUSS_PER_CTA + tid * GPT + g
                                 : blockIdx.x * Cfg::GAUSS_PER_CTA + g * T + tid;
        float* dst = a.part + ((long long)slab * a.B + b) * a.planes * (long long)a.N + slot;
#pragma unroll
        for (int k = 0; k < N_MOMENTS; ++k) {
            float lo, hi;
            upk(tot[g][k], lo, hi);
            dst[(long long)(a.moment_plane0 + k) * a.N] = lo + hi;
        }
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            if (c < a.cr) {
                float lo, hi;
                upk(tot[g][N_MOMENTS + c], lo, hi);
                dst[(long long)(a.color_plane0 + a.c0 + c) * a.N] = lo + hi;
            }
        }
    }
}

template <int CT, int GPT>
static cudaError_t launch_one(const BwdArgs& a, const BwdPlan& p, cudaStream_t s) {
    using Cfg = BwdCfg<CT, GPT>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(splat_backward_kernel<CT, GPT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    dim3 grid((unsigned)((a.N + Cfg::GAUSS_PER_CTA - 1) / Cfg::GAUSS_PER_CTA), (unsigned)p.n_slab, (unsigned)a.B);
    {
        KernelTimer timer(K_BACKWARD, s);
        splat_backward_kernel<CT, GPT><<<grid, Cfg::THREADS, Cfg::SMEM, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_backward_chunk(int ct, bool separable, bool culling, const BwdArgs& a, const BwdPlan& p,
                                  cudaStream_t s) {
    if (separable)
        return p.row_kernel ? launch_backward_row_chunk(ct, culling, a, p, s) : launch_backward_sep_chunk(ct, culling, a, p, s);
    const bool two = p.gauss_per_thread >= 2;
    switch (ct) {
        case 1: return two ? launch_one<1, BWD_GPT>(a, p, s) : launch_one<1, 1>(a, p, s);
        case 2: return two ? launch_one<2, BWD_GPT>(a, p, s) : launch_one<2, 1>(a, p, s);
        case 3: return two ? launch_one<3, BWD_GPT>(a, p, s) : launch_one<3, 1>(a, p, s);
        case 4: return two ? launch_one<4, BWD_GPT>(a, p, s) : launch_one<4, 1>(a, p, s);
        case 8: return launch_one<8, 1>(a, p, s);
        case 16: return launch_one<16, BWD_GPT_16>(a, p, s);
    }
    return cudaErrorInvalidValue;
}

template <int CT, int GPT>
static int occ(int device) {
    using Cfg = BwdCfg<CT, GPT>;
    static int cached[64];
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    cudaFuncSetAttribute(splat_backward_kernel<CT, GPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, splat_backward_kernel<CT, GPT>, Cfg::THREADS, Cfg::SMEM) !=
            cudaSuccess ||
        n <= 0) {
        cudaGetLastError();
        n = Cfg::MIN_CTAS;
    }
    if (device >= 0 && device < 64) cached[device] = n;
    return n;
}

// two gaussians per thread where the registers allow it (up to 4 channels per chunk)
int backward_gauss_per_thread(int ct) { return ct > 8 ? BWD_GPT_16 : (ct > 4 ? 1 : BWD_GPT); }

int backward_ctas_per_sm(int ct, int device) {
    const bool two = backward_gauss_per_thread(ct) >= 2;
    switch (ct) {
        case 1: return two ? occ<1, BWD_GPT>(device) : occ<1, 1>(device);
        case 2: return two ? occ<2, BWD_GPT>(device) : occ<2, 1>(device);
        case 3: return two ? occ<3, BWD_GPT>(device) : occ<3, 1>(device);
        case 4: return two ? occ<4, BWD_GPT>(device) : occ<4, 1>(device);
        case 8: return occ<8, 1>(device);
        default: return occ<16, BWD_GPT_16>(device);
    }
}
int backward_threads(int) { return 128; }
int backward_chunk_pairs(int ct) { return ct <= 4 ? 256 : 128; }

// ---------------------------------------------------------------------------
// per-gaussian epilogue: slab partials -> gradients
// ---------------------------------------------------------------------------
// One CTA finalises FIN_G consecutive gaussians.  First every warp adds up the slab partials
// of some of the planes (in slab order; a warp's loads are 32 consecutive gaussians of one
// plane, and the eight warps keep eight planes' worth of loads in flight), then the first
// warp turns the sums into gradients, one gaussian per lane.
constexpr int FIN_G = 32, FIN_THREADS = 256;

// RANGED: per-slot slab ranges (a.slab_range); ORDERED: a.order maps slots to gaussians.  Separate
// instantiations: with both decided at run time the plain case ran 10 us longer.
template <bool RANGED, bool ORDERED>
__global__ void __launch_bounds__(FIN_THREADS) finalize_kernel(FinalizeArgs a) {
    extern __shared__ float s_sum[];  // [planes][FIN_G]
    const int lane = threadIdx.x & 31, wq = threadIdx.x >> 5;
    const long long total = (long long)a.B * a.N;
    // The partial sums are laid out by processing slot (coalesced for the kernels that wrote
    // them and for the loads below); the order maps a slot to its gaussian.
    const long long t_raw = (long long)blockIdx.x * FIN_G + lane;  // over B*N slots
    const long long t = t_raw < total ? t_raw : total - 1;
    const long long b = t / a.N, slot = t - b * a.N;
    const long long plane = a.N;
    const long long slab_stride = (long long)a.B * a.planes * plane;
    // the slabs that hold sums of this slot: all of them, or (ordered skipping path) the
    // range its group had tasks for; the others were never written and stand for exact zeros
    if constexpr (RANGED) {
        const int r = a.slab_range[t];
        const int s_lo = min(r & 0xffff, a.n_slab), s_hi = min(r >> 16, a.n_slab);
        for (int p = wq; p < a.planes; p += FIN_THREADS / 32) {
            const float* src = a.part + (b * a.planes + p) * plane + slot;
            float acc = 0.f;
#pragma unroll 4
            for (int s = s_lo; s < s_hi; ++s) acc += src[(long long)s * slab_stride];
            s_sum[p * FIN_G + lane] = acc;
        }
    } else {
        for (int p = wq; p < a.planes; p += FIN_THREADS / 32) {
            const float* src = a.part + (b * a.planes + p) * plane + slot;
            float acc = 0.f;
#pragma unroll 8
            for (int s = 0; s < a.n_slab; ++s) acc += src[(long long)s * slab_stride];
            s_sum[p * FIN_G + lane] = acc;
        }
    }
    __syncthreads();
    long long n = slot;
    if constexpr (ORDERED) n = a.order[t];
    if (wq != 0 || t_raw >= total || n < 0 || n >= a.N) return;  // (an entry that is no index: nothing to write)
    const long long i = b * a.N + n;
    float M[N_MOMENTS] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < a.n_chunks; ++q)
#pragma unroll
        for (int k = 0; k < N_MOMENTS; ++k) M[k] += s_sum[(q * N_MOMENTS + k) * FIN_G + lane];
    const ParamLayout& L = a.lay;
    const float al = a.alpha ? a.alpha[i] : 1.0f;
    for (int c = 0; c < a.C; ++c) a.d_colors[i * L.col_s + c] = al * s_sum[(a.n_chunks * N_MOMENTS + c) * FIN_G + lane];
    float c00, c01, c11;
    CovInv ci;
    float sx = 0.f, sy = 0.f, ex = 1.f, ey = 1.f;  // ex, ey: d scale / d (what the caller stores)
    if (a.kind == SHAPE_SCALE_ROT) {
        sx = a.shape0[(long long)L.s0_s * i];
        sy = a.shape0[(long long)L.s0_s * i + 1];
        if (L.log_scale) {
            ex = expf(sx);
            ey = expf(sy);
            sx = ex + a.eps;
            sy = ey + a.eps;
        }
        ci = cov_inv_from_scale_rot(sx, sy, a.shape1[(long long)L.s1_s * i], a.eps);
        c00 = ci.c00;
        c01 = ci.c01;
        c11 = ci.c11;
    } else {
        c00 = a.shape0[i];
        c01 = a.shape1[i];
        c11 = a.shape2[i];
    }
    if (a.d_alpha) a.d_alpha[i] = M[0];
    if (L.d_unused) L.d_unused[(long long)L.pos_s * i] = 0.f;
    a.d_pos[(long long)L.pos_s * i] = al * (c00 * M[1] + c01 * M[2]);
    a.d_pos[(long long)L.pos_s * i + 1] = al * (c11 * M[2] + c01 * M[1]);
    const float g00 = -0.5f * al * M[3], g01 = -al * M[4], g11 = -0.5f * al * M[5];
    if (a.kind == SHAPE_COV_INV) {
        a.d_shape0[i] = g00;
        a.d_shape1[i] = g01;
        a.d_shape2[i] = g11;
    } else {
        // c00 = d/det, c01 = -b/det, c11 = a/det with det = a*d - b^2
        const float id = 1.0f / ci.det, id2 = id * id;
        const float A_ = ci.a, B_ = ci.b, D_ = ci.d;
        const float ga = g00 * (-D_ * D_ * id2) + g01 * (B_ * D_ * id2) + g11 * (id - A_ * D_ * id2);
        const float gd = g00 * (id - A_ * D_ * id2) + g01 * (A_ * B_ * id2) + g11 * (-A_ * A_ * id2);
        const float gb = g00 * (2.f * B_ * D_ * id2) + g01 * (-id - 2.f * B_ * B_ * id2) + g11 * (2.f * A_ * B_ * id2);
        const float cs = ci.cs, sn = ci.sn;
        a.d_shape0[(long long)L.s0_s * i] = ex * (2.f * sx * (ga * cs * cs + gb * cs * sn + gd * sn * sn));
        a.d_shape0[(long long)L.s0_s * i + 1] = ey * (2.f * sy * (ga * sn * sn - gb * cs * sn + gd * cs * cs));
        a.d_shape1[(long long)L.s1_s * i] = -2.f * B_ * ga + (cs * cs - sn * sn) * (sx * sx - sy * sy) * gb + 2.f * B_ * gd;
    }
}

cudaError_t launch_finalize(const FinalizeArgs& a, cudaStream_t s) {
    const long long n = (long long)a.B * a.N;
    if (n <= 0) return cudaSuccess;
    {
        KernelTimer timer(K_FINALIZE, s);
        // (planes <= 6 * 16 + 256: at most 45 KB, within the default dynamic limit)
        const unsigned blocks = (unsigned)((n + FIN_G - 1) / FIN_G);
        const size_t smem = (size_t)a.planes * FIN_G * sizeof(float);
        if (a.slab_range && a.order)
            finalize_kernel<true, true><<<blocks, FIN_THREADS, smem, s>>>(a);
        else if (a.slab_range)
            finalize_kernel<true, false><<<blocks, FIN_THREADS, smem, s>>>(a);
        else if (a.order)
            finalize_kernel<false, true><<<blocks, FIN_THREADS, smem, s>>>(a);
        else
            finalize_kernel<false, false><<<blocks, FIN_THREADS, smem, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// coordinate gradients d_x, d_y (pixel-owner pass; only on request)
//   d_x = sum_n cf*(2 c00 dx + 2 c01 dy) = -sum_n alpha*h*(c00 dx + c01 dy), likewise d_y
// with the coefficients recovered from the pre-scaled geometry record.
// ---------------------------------------------------------------------------
constexpr int CG_THREADS = 128;
constexpr int CG_CHUNK = 128;
constexpr int CG_CMAX = 16;

__global__ void __launch_bounds__(CG_THREADS) coord_grad_kernel(CoordGradArgs a) {
    __shared__ float s_geo[CG_CHUNK][GEO_FLOATS];
    __shared__ float s_col[CG_CHUNK][CG_CMAX];
    const long long HW = (long long)a.H * a.W;
    const int b = blockIdx.y;
    const long long p = (long long)blockIdx.x * CG_THREADS + threadIdx.x;
    const bool valid = p < HW;
    const long long pc = valid ? p : HW - 1;
    const long long h_ = pc / a.W, w_ = pc - h_ * a.W;
    const float xv = a.x[b * a.xs_b + h_ * a.xs_h + w_ * a.xs_w];
    const float yv = a.y[b * a.ys_b + h_ * a.ys_h + w_ * a.ys_w];
    const float Sp = a.wsum[b * HW + pc] + a.eps;
    float gS = 0.f;
    for (int c = 0; c < a.C; ++c) {
        const float g = a.gout[((long long)b * a.C + c) * HW + pc];
        gS += (a.mode == IGS_GRAD_REFERENCE) ? g * g : (g / Sp) * a.out[((long long)b * a.C + c) * HW + pc];
    }
    gS = (a.mode == IGS_GRAD_REFERENCE) ? -gS / (Sp * Sp) : -gS;
    float gxa = 0.f, gya = 0.f;
    const float inv_k = 1.0f / EXP2_SCALE;
    for (int c0 = 0; c0 < max(a.C, 1); c0 += CG_CMAX) {
        const int cr = min(CG_CMAX, a.C - c0);
        float gn[CG_CMAX];
#pragma unroll
        for (int c = 0; c < CG_CMAX; ++c)
            gn[c] = (c < cr) ? a.gout[((long long)b * a.C + c0 + c) * HW + pc] / Sp : 0.f;
        const float gS_pass = (c0 == 0) ? gS : 0.f;
        for (int n0 = 0; n0 < a.N; n0 += CG_CHUNK) {
            const int cnt = min(CG_CHUNK, a.N - n0);
            __syncthreads();
            for (int i = threadIdx.x; i < cnt * GEO_FLOATS; i += CG_THREADS)
                s_geo[i / GEO_FLOATS][i % GEO_FLOATS] = a.geo[((long long)b * a.N + n0) * GEO_FLOATS + i];
            for (int i = threadIdx.x; i < cnt * CG_CMAX; i += CG_THREADS) {
                const int g = i / CG_CMAX, c = i % CG_CMAX;
                s_col[g][c] = (c < cr) ? a.colors[((long long)b * a.N + n0 + g) * a.C + c0 + c] : 0.f;
            }
            __syncthreads();
            for (int g = 0; g < cnt; ++g) {
                const float dx = xv - s_geo[g][0], dy = yv - s_geo[g][1];
                const float A = s_geo[g][2], B2 = s_geo[g][3], Cq = s_geo[g][4], al = s_geo[g][5];
                const float e = ex2f(dx * (A * dx + B2 * dy) + (Cq * dy) * dy);
                float G = gS_pass;
#pragma unroll
                for (int c = 0; c < CG_CMAX; ++c) G = fmaf(gn[c], s_col[g][c], G);
                const float hw = -(G * e) * al;
                // c00 = A/k, c01 = B2/(2k), c11 = Cq/k
                gxa = fmaf(hw, (A * dx + 0.5f * B2 * dy) * inv_k, gxa);
                gya = fmaf(hw, (Cq * dy + 0.5f * B2 * dx) * inv_k, gya);
            }
        }
    }
    if (valid) {
        a.d_x[b * HW + p] = gxa;
        a.d_y[b * HW + p] = gya;
    }
}

cudaError_t launch_coord_grad(const CoordGradArgs& a, cudaStream_t s) {
    const long long HW = (long long)a.H * a.W;
    if (HW <= 0 || a.B <= 0) return cudaSuccess;
    dim3 grid((unsigned)((HW + CG_THREADS - 1) / CG_THREADS), (unsigned)a.B);
    {
        KernelTimer timer(K_COORD_GRAD, s);
        coord_grad_kernel<<<grid, CG_THREADS, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace igs
