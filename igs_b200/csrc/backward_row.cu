// Backward splat kernel for separable grids and MANY channels (chunks of 8 and 16).
//
// The separable kernel for up to 4 channels (backward_sep.cu) packs two PIXELS into every
// f32x2 operand, which makes every per-gaussian quantity (centre, exponent coefficients,
// colours, all gradient sums) cost two registers per gaussian twice over.  At 16 channels that
// does not fit a thread any more.  Here the two lanes of an f32x2 are two GAUSSIANS instead:
// a thread owns one pair, its constants and sums take one register pair each, and the pixels
// stream by one at a time, row after row, their upstream terms broadcast into both lanes.
// 114 registers of per-gaussian state at C = 16 instead of 228.
//
// The grid factorises as in backward_sep.cu (x by column, y by row): with h = G*e,
//   M0 = sum_rows hs_r       Mx  = sum_rows hxs_r       Mxx = sum h*dx*dx
//   My = sum_rows dy_r*hs_r  Mxy = sum_rows dy_r*hxs_r  Myy = sum_rows dy_r^2*hs_r
//   hs_r = sum_cols h,  hxs_r = sum_cols h*dx
// and per pixel the exponent is two FMAs on top of dx, because B2*dy and Cq*dy^2 are per-row
// constants:  s = A*dx + bd;  q = dx*s + cd.  Per gaussian x pixel, 8 + 2C FMA-pipe
// instructions (40 at C = 16; the general kernel issues 48):
//   dx = x - px; s; q                    3      G = gS + sum_c gn_c*col_c     C
//   h = G*e; hs += h; hx = h*dx; hxs += hx; Mxx += hx*dx   5      E_c += gn_c*e    C
//
// Pixel records (pixel_terms_row_kernel): [B, H, W, PF] floats {x, gS, gn_0 .. gn_{CT-1}, pad},
// streamed through shared memory by 1-D bulk copies in stages of up to SEG pixels; the row
// coordinates y[b, h] sit in a small array of their own.
//
// Skipping (CULL = true; the same rules as in backward_sep.cu, so that skipping changes no
// bit): the CTA streams only the rectangle of pixels that the box around all its gaussians
// meets, and inside it each warp votes on runs of RUN pixels.  Needs non-decreasing axes and a
// finite upstream gradient (else the plain instantiation runs).
#include "backward.cuh"

namespace igs {

// floats per pixel record of the row layout
__host__ __device__ constexpr int bwd_row_rec_floats(int ct) { return (2 + ct + 3) / 4 * 4; }

// ---------------------------------------------------------------------------
// per-pixel upstream terms, row layout
// ---------------------------------------------------------------------------
template <int CT>
__global__ void __launch_bounds__(256) pixel_terms_row_kernel(PixelTermArgs a) {
    constexpr int PF = bwd_row_rec_floats(CT);
    if (a.grid_sel && (*a.grid_sel & GRID_NOT_SEPARABLE)) return;
    const long long HW = (long long)a.H * a.W;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over B*H*W
    bool bad = false;
    if (i < (long long)a.B * HW) {
        const long long b = i / HW, p = i - b * HW;
        const int h = (int)(p / a.W), w = (int)(p - (long long)h * a.W);
        const int cr = a.ch.cr[0];
        // separable grid: row 0 holds every row's x, column 0 every column's y
        if (w == 0) a.axes[b * a.H + h] = a.y[b * a.ys_b + (long long)h * a.ys_h];
        const float Sp = a.wsum[b * HW + p] + a.eps;
        float v[PF];
#pragma unroll
        for (int k = 0; k < PF; ++k) v[k] = 0.f;
        v[0] = a.x[b * a.xs_b + (long long)w * a.xs_w];
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            if (c < cr) {
                const float g = a.gout[(b * a.C + c) * HW + p];
                if (a.mode == IGS_GRAD_REFERENCE)
                    acc += g * g;
                else
                    acc += (g / Sp) * a.out[(b * a.C + c) * HW + p];
                v[2 + c] = g / Sp;
                bad |= !isfinite(v[2 + c]);
            }
        }
        v[1] = (a.mode == IGS_GRAD_REFERENCE) ? -acc / (Sp * Sp) : -acc;
        bad |= !isfinite(v[1]);
        float4* rec = reinterpret_cast<float4*>(a.prec[0] + i * PF);
#pragma unroll
        for (int q = 0; q < PF / 4; ++q) rec[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
    if (a.flags && __syncthreads_or(bad) && threadIdx.x == 0) atomicOr(a.flags, UPSTREAM_NOT_FINITE);
}

cudaError_t launch_pixel_terms_row(const PixelTermArgs& a, cudaStream_t s) {
    const long long n = (long long)a.B * a.H * a.W;
    if (n <= 0) return cudaSuccess;
    if (a.ch.n != 1 || !a.axes) return cudaErrorInvalidValue;
    {
        KernelTimer timer(K_PIXEL_TERMS, s);
        const unsigned blocks = (unsigned)((n + 255) / 256);
        if (a.ch.ct[0] == 8)
            pixel_terms_row_kernel<8><<<blocks, 256, 0, s>>>(a);
        else if (a.ch.ct[0] == 16)
            pixel_terms_row_kernel<16><<<blocks, 256, 0, s>>>(a);
        else
            return cudaErrorInvalidValue;
    }
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------
template <int CT>
struct BwdRowCfg {
    static constexpr int THREADS = 128;
    static constexpr int GAUSS_PER_CTA = THREADS * 2;  // one pair per thread
    static constexpr int SEG = 128;                    // pixels per shared-memory stage
    static constexpr int STAGES = 2;
    static constexpr int RUN = 32;                     // pixels per skip decision
    // measured on an inner-loop model of this kernel: 8 channels 4 CTAs per SM (110 registers),
    // 16 channels 3 CTAs (152 registers) with the pixel loop unrolled twice
    static constexpr int MIN_CTAS = CT <= 8 ? 4 : 3;
    static constexpr int UNROLL = 2;
    static constexpr int PF = bwd_row_rec_floats(CT);
    static constexpr size_t SMEM = (size_t)STAGES * SEG * PF * sizeof(float) + STAGES * sizeof(uint64_t) + 16 + 128;
};

template <int CT, bool CULL>
__global__ void __launch_bounds__(BwdRowCfg<CT>::THREADS, BwdRowCfg<CT>::MIN_CTAS) splat_backward_row_kernel(BwdArgs a) {
    using Cfg = BwdRowCfg<CT>;
    constexpr int T = Cfg::THREADS, SEG = Cfg::SEG, NS = Cfg::STAGES, PF = Cfg::PF, RUN = Cfg::RUN;

    if (a.grid_sel && (*a.grid_sel & GRID_NOT_SEPARABLE)) return;  // not a separable grid: the general kernel runs
    if (a.cull_sel && ((!(*a.grid_word & NO_BACKWARD_SKIPPING) &&
                        (long long)(*a.cull_sel) * 8 >= (long long)a.B * a.N) != CULL))
        return;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage_base = reinterpret_cast<float*>(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NS * SEG * PF * sizeof(float));
    int* s_failed = reinterpret_cast<int*>(bars + NS);

    const int tid = threadIdx.x;
    const int b = blockIdx.z, slab = blockIdx.y;

    // ---- this thread's two gaussians (lanes lo, hi of every f32x2) ----
    int n[2];
    const int slot0 = blockIdx.x * Cfg::GAUSS_PER_CTA + tid * 2;  // the partial sums are laid out by slot
    float gv[2][8], cv[2][CT];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const int slot = slot0 + g;
        n[g] = slot < a.N ? (a.order ? a.order[(long long)b * a.N + slot] : slot) : a.N;
        if ((unsigned)n[g] > (unsigned)a.N) n[g] = a.N;  // an entry that is no index: the slot stays empty
        const int nn = n[g] < a.N ? n[g] : a.N - 1;
        const float4* gp = reinterpret_cast<const float4*>(a.geo + ((long long)b * a.N + nn) * GEO_FLOATS);
        const float4 g0 = gp[0], g1 = gp[1];
        gv[g][0] = g0.x; gv[g][1] = g0.y; gv[g][2] = g0.z; gv[g][3] = g0.w;
        gv[g][4] = g1.x; gv[g][5] = g1.y; gv[g][6] = g1.z; gv[g][7] = g1.w;
#pragma unroll
        for (int c = 0; c < CT; ++c)
            cv[g][c] = (c < a.cr) ? a.colors[((long long)b * a.N + nn) * a.C + a.c0 + c] : 0.f;
    }
    const f2 px = pk(gv[0][0], gv[1][0]), py = pk(gv[0][1], gv[1][1]);
    const f2 A = pk(gv[0][2], gv[1][2]), B2 = pk(gv[0][3], gv[1][3]), Cq = pk(gv[0][4], gv[1][4]);
    f2 col[CT];
#pragma unroll
    for (int c = 0; c < CT; ++c) col[c] = pk(cv[0][c], cv[1][c]);
    // the box outside which both gaussians' weights are exactly zero (pack.cu); an empty slot
    // reaches nothing
    float box_x0 = INFINITY, box_x1 = -INFINITY, box_y0 = INFINITY, box_y1 = -INFINITY;
    bool open_box = false;  // a NaN or infinite box: no restriction
    if constexpr (CULL) {
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            if (n[g] >= a.N) continue;
            const float x0 = gv[g][0] - gv[g][6], x1 = gv[g][0] + gv[g][6];
            const float y0 = gv[g][1] - gv[g][7], y1 = gv[g][1] + gv[g][7];
            open_box |= !(x1 - x0 < INFINITY) || !(y1 - y0 < INFINITY);
            box_x0 = fminf(box_x0, x0);
            box_x1 = fmaxf(box_x1, x1);
            box_y0 = fminf(box_y0, y0);
            box_y1 = fmaxf(box_y1, y1);
        }
        if (open_box) {
            box_x0 = box_y0 = -INFINITY;
            box_x1 = box_y1 = INFINITY;
        }
    }

    f2 M[N_MOMENTS], E[CT];
#pragma unroll
    for (int k = 0; k < N_MOMENTS; ++k) M[k] = 0ull;
#pragma unroll
    for (int c = 0; c < CT; ++c) E[c] = 0ull;

    // ---- this slab's rows ----
    const int n_rows_img = a.nrp;  // (rows of the image; see launch_backward_row_chunk)
    const int W = a.ncb;           // (pixels per row)
    const int r_begin = min(n_rows_img, slab * a.rp_per_slab);
    const int r_end = min(n_rows_img, r_begin + a.rp_per_slab);
    const float* ys = a.axes + (long long)b * n_rows_img;
    // The stream is rows [r0, r0 + n_r) x pixels [c0, c0 + seg) of the records: everything in
    // the plain kernel; in the skipping kernel only the rectangle the box around ALL of this
    // CTA's gaussians meets.  The slabs stay fixed ranges of rows whatever the gaussians.
    int r0 = r_begin, n_r = r_end - r_begin, c0 = 0, seg = W;
    if constexpr (CULL) {
        float* s_box = reinterpret_cast<float*>(s_failed + 4);  // [4 warps][4], then 4 ints
        int* s_rng = reinterpret_cast<int*>(s_box + 16);
        float u[4] = {box_x0, box_x1, box_y0, box_y1};
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            u[0] = fminf(u[0], __shfl_xor_sync(0xffffffffu, u[0], d));
            u[1] = fmaxf(u[1], __shfl_xor_sync(0xffffffffu, u[1], d));
            u[2] = fminf(u[2], __shfl_xor_sync(0xffffffffu, u[2], d));
            u[3] = fmaxf(u[3], __shfl_xor_sync(0xffffffffu, u[3], d));
        }
        if ((tid & 31) == 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) s_box[(tid >> 5) * 4 + k] = u[k];
        }
        if (tid < 4) s_rng[tid] = (tid & 1) ? -1 : 0x7fffffff;  // lo row, hi row, lo column, hi column
        __syncthreads();
#pragma unroll
        for (int w = 0; w < T / 32; ++w) {
            u[0] = fminf(u[0], s_box[w * 4 + 0]);
            u[1] = fmaxf(u[1], s_box[w * 4 + 1]);
            u[2] = fminf(u[2], s_box[w * 4 + 2]);
            u[3] = fmaxf(u[3], s_box[w * 4 + 3]);
        }
        if (u[1] - u[0] < INFINITY && u[3] - u[2] < INFINITY) {
            const float* rec0 = a.prec + (long long)b * n_rows_img * W * PF;  // row 0: every column's x
            int lo = 0x7fffffff, hi = -1;
            for (int r = r_begin + tid; r < r_end; r += T) {
                const float yv = ys[r];
                if (!(u[3] < yv || u[2] > yv)) {
                    lo = min(lo, r);
                    hi = max(hi, r);
                }
            }
            int clo = 0x7fffffff, chi = -1;
            for (int c = tid; c < W; c += T) {
                const float xv = rec0[(long long)c * PF];
                if (!(u[1] < xv || u[0] > xv)) {
                    clo = min(clo, c);
                    chi = max(chi, c);
                }
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, d));
                hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, d));
                clo = min(clo, __shfl_xor_sync(0xffffffffu, clo, d));
                chi = max(chi, __shfl_xor_sync(0xffffffffu, chi, d));
            }
            if ((tid & 31) == 0) {
                atomicMin(&s_rng[0], lo);
                atomicMax(&s_rng[1], hi);
                atomicMin(&s_rng[2], clo);
                atomicMax(&s_rng[3], chi);
            }
            __syncthreads();
            lo = s_rng[0], hi = s_rng[1], clo = s_rng[2], chi = s_rng[3];
            if (hi < lo || chi < clo) {
                n_r = 0;  // nothing of this slab is reached: the sums stay zero
            } else {
                r0 = lo;
                n_r = hi - lo + 1;
                c0 = clo;
                seg = chi - clo + 1;
            }
        }
    }
    const int n_total = n_r * seg;  // pixels in the stream (a slab is far below 2^31 pixels)
    const int n_chunks = (n_total + SEG - 1) / SEG;
    const float* src = a.prec + (((long long)b * n_rows_img + r0) * W + c0) * PF;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
        *s_failed = 0;
        mbar_init_fence();
    }
    __syncthreads();

    auto issue = [&](int chunk) {
        const int st = chunk % NS;
        const int cnt = min(SEG, n_total - chunk * SEG);
        mbar_expect_tx(&bars[st], (uint32_t)cnt * PF * sizeof(float));
        // the chunk is a run of the virtual stream: one copy per row it touches
        float* dstp = stage_base + (size_t)st * SEG * PF;
        int v = chunk * SEG, left = cnt;
        while (left > 0) {
            const int r = v / seg, c = v - r * seg;
            const int len = min(left, seg - c);
            bulk_g2s(dstp, src + ((long long)r * W + c) * PF, (uint32_t)len * PF * sizeof(float), &bars[st]);
            dstp += (size_t)len * PF;
            v += len;
            left -= len;
        }
    };
    if (tid == 0) {
        for (int c = 0; c < NS && c < n_chunks; ++c) issue(c);
    }

    // row state: dy, B2*dy, Cq*dy^2 and the row sums hs, hxs
    f2 dyd = 0ull, bd = 0ull, cd = 0ull, hs = 0ull, hxs = 0ull;
    float row_y = 0.f;
    int cb = 0, row = r0;  // pixel position inside the current row of the stream; the row itself
    int must = 0;          // pixels of the current run still to be processed without voting again
    int visited = 0;       // pixels this warp did not skip (counted by the skipping kernel only)
    auto fold_row = [&]() {
        M[0] = add2(M[0], hs);
        M[1] = add2(M[1], hxs);
        M[2] = fma2(dyd, hs, M[2]);
        M[4] = fma2(dyd, hxs, M[4]);
        M[5] = fma2(mul2(dyd, dyd), hs, M[5]);
    };

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
        const int cnt = min(SEG, n_total - chunk * SEG);
        const float4* rec = reinterpret_cast<const float4*>(stage_base + (size_t)st * SEG * PF);

        int i = 0;
        while (i < cnt) {
            if (cb == 0) {
                // new row: row terms of the exponent, fresh row sums
                row_y = ys[row];
                const f2 dyr = sub2(pk(row_y, row_y), py);
                dyd = dyr;
                bd = mul2(B2, dyr);
                cd = mul2(mul2(Cq, dyr), dyr);
                hs = 0ull;
                hxs = 0ull;
            }
            // pixels of this row that are in this stage
            int len = min(cnt - i, seg - cb);
            if constexpr (CULL) {
                if (must == 0) {
                    const int run = min(RUN, len);
                    const float run_x0 = rec[(size_t)i * (PF / 4)].x, run_x1 = rec[(size_t)(i + run - 1) * (PF / 4)].x;
                    const bool need = !(box_x1 < run_x0 || box_x0 > run_x1 || box_y1 < row_y || box_y0 > row_y);
                    if (!__any_sync(0xffffffffu, need)) {
                        i += run;
                        cb += run;
                        if (cb == seg) {
                            cb = 0;
                            ++row;
                            fold_row();
                        }
                        continue;
                    }
                    must = run;
                }
                len = min(len, must);
                must -= len;
                visited += len;
            }
            const float4* r = rec + (size_t)i * (PF / 4);
#pragma unroll(Cfg::UNROLL)
            for (int k = 0; k < len; ++k, r += PF / 4) {
                float gt[PF];
#pragma unroll
                for (int q = 0; q < PF / 4; ++q) {
                    const float4 t4 = r[q];
                    gt[4 * q] = t4.x; gt[4 * q + 1] = t4.y; gt[4 * q + 2] = t4.z; gt[4 * q + 3] = t4.w;
                }
                const f2 dx = sub2(pk(gt[0], gt[0]), px);
                const f2 e = ex2_2(fma2(dx, fma2(A, dx, bd), cd));
                f2 G = pk(gt[1], gt[1]);
                f2 gn[CT];
#pragma unroll
                for (int c = 0; c < CT; ++c) {
                    gn[c] = pk(gt[2 + c], gt[2 + c]);
                    G = fma2(gn[c], col[c], G);
                }
                const f2 h = mul2(G, e);
                hs = add2(hs, h);
                const f2 hx = mul2(h, dx);
                hxs = add2(hxs, hx);
                M[3] = fma2(hx, dx, M[3]);
#pragma unroll
                for (int c = 0; c < CT; ++c) E[c] = fma2(gn[c], e, E[c]);
            }
            i += len;
            cb += len;
            if (cb == seg) {
                cb = 0;
                ++row;
                fold_row();
            }
        }
        __syncthreads();
        if (tid == 0 && chunk + NS < n_chunks) issue(chunk + NS);
    }

    if constexpr (CULL) {
        // a visited pixel is evaluated against the two gaussians of each of the warp's 32 lanes
        if ((tid & 31) == 0 && a.exec_count) atomicAdd(a.exec_count, (unsigned long long)visited * 64);
    }

    float* dst = a.part + ((long long)slab * a.B + b) * a.planes * (long long)a.N;
#pragma unroll
    for (int k = 0; k < N_MOMENTS; ++k) {
        float lo, hi;
        upk(M[k], lo, hi);
        if (n[0] < a.N) dst[(long long)(a.moment_plane0 + k) * a.N + slot0] = lo;
        if (n[1] < a.N) dst[(long long)(a.moment_plane0 + k) * a.N + slot0 + 1] = hi;
    }
#pragma unroll
    for (int c = 0; c < CT; ++c) {
        if (c < a.cr) {
            float lo, hi;
            upk(E[c], lo, hi);
            if (n[0] < a.N) dst[(long long)(a.color_plane0 + a.c0 + c) * a.N + slot0] = lo;
            if (n[1] < a.N) dst[(long long)(a.color_plane0 + a.c0 + c) * a.N + slot0 + 1] = hi;
        }
    }
}

template <int CT, bool CULL>
static cudaError_t launch_row_one(const BwdArgs& a_in, const BwdPlan& p, cudaStream_t s) {
    using Cfg = BwdRowCfg<CT>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(splat_backward_row_kernel<CT, CULL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    // this kernel counts rows and pixels, not row pairs and 4-column blocks: the fields of the
    // argument block are reused with that meaning
    BwdArgs a = a_in;
    a.nrp = p.rows;
    a.ncb = p.cols;
    a.rp_per_slab = 2 * p.rp_per_slab;
    dim3 grid((unsigned)((a.N + Cfg::GAUSS_PER_CTA - 1) / Cfg::GAUSS_PER_CTA), (unsigned)p.n_slab, (unsigned)a.B);
    {
        KernelTimer timer(K_BACKWARD, s);
        splat_backward_row_kernel<CT, CULL><<<grid, Cfg::THREADS, Cfg::SMEM, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

template <int CT>
static int row_occ(int device) {
    using Cfg = BwdRowCfg<CT>;
    static int cached[64];
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    cudaFuncSetAttribute(splat_backward_row_kernel<CT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Cfg::SMEM);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, splat_backward_row_kernel<CT, false>, Cfg::THREADS,
                                                      Cfg::SMEM) != cudaSuccess ||
        n <= 0) {
        cudaGetLastError();
        n = Cfg::MIN_CTAS;
    }
    if (device >= 0 && device < 64) cached[device] = n;
    return n;
}

bool backward_has_row_kernel(int ct) { return ct == 8 || ct == 16; }

int backward_row_ctas_per_sm(int ct, int device) { return ct == 8 ? row_occ<8>(device) : row_occ<16>(device); }

int backward_row_record_floats(int ct) { return bwd_row_rec_floats(ct); }

cudaError_t launch_backward_row_chunk(int ct, bool culling, const BwdArgs& a, const BwdPlan& p, cudaStream_t s) {
    switch (ct) {
        case 8: return culling ? launch_row_one<8, true>(a, p, s) : launch_row_one<8, false>(a, p, s);
        case 16: return culling ? launch_row_one<16, true>(a, p, s) : launch_row_one<16, false>(a, p, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace igs
