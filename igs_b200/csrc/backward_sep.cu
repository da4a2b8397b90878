// Backward splat kernel for separable grids (x by column, y by row; what xy_grid makes).
//
// Same ownership as the general backward kernel (a thread owns gaussians, pixels stream
// through shared memory by bulk copies) but the pixels arrive as 2-row x 4-column
// blocks, row pair after row pair, and a slab is a range of whole row pairs.  With
// h = G*e as before, the six moments factor along a row of constant dy:
//   M0 = sum_rows hs_r              Mx  = sum_rows hxs_r
//   My = sum_rows dy_r*hs_r         Mxy = sum_rows dy_r*hxs_r        Myy = sum_rows dy_r^2*hs_r
//   Mxx = sum h*dx*dx               with  hs_r = sum_cols h,  hxs_r = sum_cols h*dx
// so per pixel only hs, hxs and Mxx are updated, and the row-level products are formed
// once per row pair.  The exponent shares its terms the same way as in the separable
// forward (dx, dx^2 per column pair; B2*dy, Cq*dy^2 per row).  Per gaussian x pixel that
// is 12 FMA-pipe instructions + 1 per pixel of column terms instead of 22, at C = 3:
//   s = A*dx + B2*dy; q = dx*s + Cq*dy^2  (two FMAs)  2      G = gS + sum_c gn_c*col_c   3
//   h = G*e; hs += h; hxs += h*dx; Mxx += h*dx^2      4      E_c += gn_c*e               3
// (dx^2 once per column pair and row pair costs half an instruction per pixel and saves one:
// measured 4.41 -> 4.27 ms at B=16, N=8192, 256 x 256; forming A*dx + B2*dy as one FMA per pixel
// instead of a shared A*dx plus an add per pixel saves another half and eight registers, at
// the same time).
#include "backward.cuh"

namespace igs {

// ---------------------------------------------------------------------------
// per-pixel upstream terms, block records
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) pixel_terms_sep_kernel(PixelTermArgs a) {
    if (a.grid_sel && (*a.grid_sel & GRID_NOT_SEPARABLE)) return;
    const long long per_b = (long long)a.nrp * a.ncb;
    // Records are built in shared memory and written out by the whole CTA in consecutive
    // 16-byte pieces: a thread storing its own 160-byte record leaves every store instruction
    // of the warp scattered over 32 half-used sectors.
    extern __shared__ __align__(16) float s_rec[];  // [blockDim.x][record floats]
    const long long total = (long long)a.B * per_b;
    const long long i_raw = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over B*nrp*ncb
    const bool in_range = i_raw < total;
    const long long i = in_range ? i_raw : total - 1;  // threads past the end redo the last block, and store nothing
    const long long b = i / per_b, blk = i - b * per_b;
    const int rp = (int)(blk / a.ncb), cbk = (int)(blk - (long long)rp * a.ncb);
    const long long HW = (long long)a.H * a.W;
    const int h0 = rp * 2, w0 = cbk * 4;

    float xv[4], yv[2];
#pragma unroll
    for (int k = 0; k < 4; ++k) xv[k] = a.x[b * a.xs_b + (long long)min(w0 + k, a.W - 1) * a.xs_w];
#pragma unroll
    for (int k = 0; k < 2; ++k) yv[k] = a.y[b * a.ys_b + (long long)min(h0 + k, a.H - 1) * a.ys_h];

    // pixel (r, k): valid flag, flat index, S + eps, gS over ALL channels
    bool bad = false;  // a non-finite upstream term: the skipping kernels must not run
    float ok[2][4], Sp[2][4], gS[2][4];
    long long pp[2][4];
    // a full block of an image whose rows are a multiple of 4 wide: rows of 4 pixels are
    // single 16-byte loads (the planes are contiguous, so every such row is aligned)
    const bool full = (h0 + 1 < a.H) && (w0 + 3 < a.W) && (a.W % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(a.wsum) | reinterpret_cast<uintptr_t>(a.gout) |
                        reinterpret_cast<uintptr_t>(a.out)) & 15) == 0;
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const bool valid = (h0 + r < a.H) && (w0 + k < a.W);
            ok[r][k] = valid ? 1.f : 0.f;
            pp[r][k] = (long long)min(h0 + r, a.H - 1) * a.W + min(w0 + k, a.W - 1);
        }
    auto row4 = [&](const float* plane, int r, float v[4]) {  // plane: [HW] of this batch element / channel
        if (full) {
            const float4 t = *reinterpret_cast<const float4*>(plane + pp[r][0]);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = plane[pp[r][k]];
        }
    };
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sv[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
        row4(a.wsum + b * HW, r, sv);
#pragma unroll
        for (int k = 0; k < 4; ++k) Sp[r][k] = sv[k] + a.eps;
        for (int c = 0; c < a.C; ++c) {
            float g[4], o[4];
            row4(a.gout + (b * a.C + c) * HW, r, g);
            if (a.mode == IGS_GRAD_REFERENCE) {
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] += g[k] * g[k];
            } else {
                row4(a.out + (b * a.C + c) * HW, r, o);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] += (g[k] / Sp[r][k]) * o[k];
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            gS[r][k] = ok[r][k] * ((a.mode == IGS_GRAD_REFERENCE) ? -acc[k] / (Sp[r][k] * Sp[r][k]) : -acc[k]);
            bad |= !isfinite(gS[r][k]);
        }
    }

    for (int q = 0; q < a.ch.n; ++q) {
        const int ct = a.ch.ct[q], cr = a.ch.cr[q], c0 = a.ch.c0[q];
        const int pf = bwd_sep_pair_floats(ct);
        const int rs = bwd_sep_rec_floats(ct);
        float* rec = s_rec + (size_t)threadIdx.x * rs;
        reinterpret_cast<float4*>(rec)[0] = make_float4(xv[0], xv[1], xv[2], xv[3]);
        reinterpret_cast<float4*>(rec)[1] = make_float4(yv[0], yv[1], 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float* pr0 = rec + 8 + (r * 2) * pf;  // pixel pairs (columns 0,1) and (2,3) of this row
            float* pr1 = pr0 + pf;
            pr0[0] = q == 0 ? gS[r][0] : 0.f;
            pr0[1] = q == 0 ? gS[r][1] : 0.f;
            pr1[0] = q == 0 ? gS[r][2] : 0.f;
            pr1[1] = q == 0 ? gS[r][3] : 0.f;
            for (int c = 0; c < pf / 2 - 1; ++c) {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (c < cr) {
                    float g[4];
                    row4(a.gout + (b * a.C + c0 + c) * HW, r, g);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        v[k] = ok[r][k] * (g[k] / Sp[r][k]);
                        bad |= !isfinite(v[k]);
                    }
                }
                pr0[2 + 2 * c] = v[0];
                pr0[3 + 2 * c] = v[1];
                pr1[2 + 2 * c] = v[2];
                pr1[3 + 2 * c] = v[3];
            }
        }
        __syncthreads();
        {
            const long long first = (long long)blockIdx.x * blockDim.x;
            const long long n_here = total - first < (long long)blockDim.x ? total - first : (long long)blockDim.x;
            float4* dst = reinterpret_cast<float4*>(a.prec[q] + first * rs);
            const float4* src4 = reinterpret_cast<const float4*>(s_rec);
            for (long long j = threadIdx.x; j < n_here * (rs / 4); j += blockDim.x) dst[j] = src4[j];
        }
        __syncthreads();
    }
    if (bad && a.flags) atomicOr(a.flags, UPSTREAM_NOT_FINITE);
}

cudaError_t launch_pixel_terms_sep(const PixelTermArgs& a, cudaStream_t s) {
    const long long n = (long long)a.B * a.nrp * a.ncb;
    if (n <= 0) return cudaSuccess;
    {
        KernelTimer timer(K_PIXEL_TERMS, s);
        int max_rs = 0;
        for (int q = 0; q < a.ch.n; ++q) max_rs = max(max_rs, bwd_sep_rec_floats(a.ch.ct[q]));
        pixel_terms_sep_kernel<<<(unsigned)((n + 127) / 128), 128, (size_t)128 * max_rs * sizeof(float), s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------
template <int CT>
struct BwdSepCfg {
    static constexpr int THREADS = 128;
    static constexpr int GPT = 2;  // gaussians per thread
    static constexpr int GAUSS_PER_CTA = THREADS * GPT;
    static constexpr int CHUNK_BLOCKS = 64;  // 2x4-pixel blocks per shared-memory stage
    static constexpr int STAGES = 2;
    static constexpr int MIN_CTAS = CT <= 3 ? 4 : 3;
    static constexpr int UNROLL = 1;
    static constexpr int RS = bwd_sep_rec_floats(CT);
    static constexpr int PF = bwd_sep_pair_floats(CT);
    static constexpr int SKIP_RUN = 8;  // blocks (32 columns) per skip decision
    static constexpr int CULL_LESS = 1;  // resident CTAs per SM the skipping kernel gives up for registers (no spills)
    // stages, their barriers, the failure flag, and 32 words for the CTA-wide box reduction
    static constexpr size_t SMEM = (size_t)STAGES * CHUNK_BLOCKS * RS * sizeof(float) + STAGES * sizeof(uint64_t) + 16 + 128;
};

template <int CT, bool CULL>
__global__ void __launch_bounds__(BwdSepCfg<CT>::THREADS, BwdSepCfg<CT>::MIN_CTAS - (CULL ? BwdSepCfg<CT>::CULL_LESS : 0))
    splat_backward_sep_kernel(BwdArgs a) {
    using Cfg = BwdSepCfg<CT>;
    constexpr int T = Cfg::THREADS, GPT = Cfg::GPT, PCB = Cfg::CHUNK_BLOCKS, NS = Cfg::STAGES, RS = Cfg::RS, PF = Cfg::PF;
    constexpr int SKIP_RUN = Cfg::SKIP_RUN;

    if (a.grid_sel && (*a.grid_sel & GRID_NOT_SEPARABLE)) return;  // not a separable grid: the general kernel runs
    // of the skipping / plain pair, the one the gaussians' reach and the axes call for
    if (a.cull_sel && ((!(*a.grid_word & NO_BACKWARD_SKIPPING) &&
                        (long long)(*a.cull_sel) * 8 >= (long long)a.B * a.N) != CULL))
        return;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage_base = reinterpret_cast<float*>(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NS * PCB * RS * sizeof(float));
    int* s_failed = reinterpret_cast<int*>(bars + NS);

    const int tid = threadIdx.x;
    const int b = blockIdx.z, slab = blockIdx.y;

    // ---- this thread's gaussians ----
    int n[GPT];
    f2 px[GPT], py[GPT], A[GPT], B2[GPT], Cq[GPT], col[GPT][CT];
    float box_x0[GPT], box_x1[GPT], box_y0[GPT], box_y1[GPT];
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
        // the box outside which this gaussian's weight is exactly zero (pack.cu)
        box_x0[g] = g0.x - g1.z;
        box_x1[g] = g0.x + g1.z;
        box_y0[g] = g0.y - g1.w;
        box_y1[g] = g0.y + g1.w;
        if (CULL && n[g] >= a.N) {  // an empty slot reaches nothing
            box_x0[g] = box_y0[g] = INFINITY;
            box_x1[g] = box_y1[g] = -INFINITY;
        }
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const float v = (c < a.cr) ? a.colors[((long long)b * a.N + nn) * a.C + a.c0 + c] : 0.f;
            col[g][c] = pk(v, v);
        }
    }
    // Skipping: a run of up to SKIP_RUN blocks of a row pair is passed over when no lane
    // of the warp owns a gaussian whose box meets the run's pixels (every term would be an
    // exact zero).  Needs non-decreasing axes (the run's x range is taken from its two ends)
    // and is only tried when enough gaussians are narrow for it to pay.
    constexpr bool cull = CULL;
    float strip_y0 = 0.f, strip_y1 = 0.f;
    int must = 0;  // blocks of the current run still to be processed without voting again
    int visited = 0;  // blocks this warp did not skip (counted by the skipping kernel only)

    // totals: M0, Mx, My, Mxx, Mxy, Myy, E_c;  row-pair state: per row r of the pair
    f2 M[GPT][N_MOMENTS], E[GPT][CT];
    f2 dyd[GPT][2], bd[GPT][2], cd[GPT][2], hs[GPT][2], hxs[GPT][2];
#pragma unroll
    for (int g = 0; g < GPT; ++g) {
#pragma unroll
        for (int k = 0; k < N_MOMENTS; ++k) M[g][k] = 0ull;
#pragma unroll
        for (int c = 0; c < CT; ++c) E[g][c] = 0ull;
#pragma unroll
        for (int r = 0; r < 2; ++r) dyd[g][r] = bd[g][r] = cd[g][r] = hs[g][r] = hxs[g][r] = 0ull;
    }

    // ---- this slab's row pairs, as a stream of blocks ----
    const int rp_begin = min(a.nrp, slab * a.rp_per_slab);
    const int rp_end = min(a.nrp, rp_begin + a.rp_per_slab);
    // The stream is rows [rp0, rp0 + n_rp) x column blocks [cb0, cb0 + seg) of the block
    // records: everything in the plain kernel; in the skipping kernel only the rectangle of
    // blocks the box around ALL of this CTA's gaussians meets (non-decreasing axes make it a
    // rectangle), so a CTA of neighbouring gaussians neither loads nor visits the rest.  The
    // slabs stay fixed ranges of rows whatever the gaussians: which pixels a partial sum
    // covers, and with it every bit of the result, depends on the shape alone.
    int rp0 = rp_begin, n_rp = rp_end - rp_begin, cb0 = 0, seg_c = a.ncb;
    if constexpr (CULL) {
        float* s_box = reinterpret_cast<float*>(s_failed + 4);  // [4 warps][4], then 4 ints
        int* s_rng = reinterpret_cast<int*>(s_box + 16);
        float u[4] = {INFINITY, -INFINITY, INFINITY, -INFINITY};  // x0, x1, y0, y1 of the union
        bool open_box = false;  // a NaN or infinite box: no restriction
#pragma unroll
        for (int g = 0; g < GPT; ++g) {
            if (n[g] >= a.N) continue;
            open_box |= !(box_x1[g] - box_x0[g] < INFINITY) || !(box_y1[g] - box_y0[g] < INFINITY);
            u[0] = fminf(u[0], box_x0[g]);
            u[1] = fmaxf(u[1], box_x1[g]);
            u[2] = fminf(u[2], box_y0[g]);
            u[3] = fmaxf(u[3], box_y1[g]);
        }
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
        const bool any_open = __syncthreads_or(open_box);
#pragma unroll
        for (int w = 0; w < T / 32; ++w) {
            u[0] = fminf(u[0], s_box[w * 4 + 0]);
            u[1] = fmaxf(u[1], s_box[w * 4 + 1]);
            u[2] = fminf(u[2], s_box[w * 4 + 2]);
            u[3] = fmaxf(u[3], s_box[w * 4 + 3]);
        }
        if (!any_open) {
            const float* rec0 = a.prec + (long long)b * a.nrp * a.ncb * RS;
            int lo = 0x7fffffff, hi = -1;
            for (int rp = rp_begin + tid; rp < rp_end; rp += T) {
                const float4 yr = reinterpret_cast<const float4*>(rec0 + (long long)rp * a.ncb * RS)[1];
                if (!(u[3] < fminf(yr.x, yr.y) || u[2] > fmaxf(yr.x, yr.y))) {
                    lo = min(lo, rp);
                    hi = max(hi, rp);
                }
            }
            int clo = 0x7fffffff, chi = -1;
            for (int cb = tid; cb < a.ncb; cb += T) {
                const float4 xc = reinterpret_cast<const float4*>(rec0 + (long long)cb * RS)[0];
                if (!(u[1] < xc.x || u[0] > xc.w)) {
                    clo = min(clo, cb);
                    chi = max(chi, cb);
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
                n_rp = 0;  // nothing of this slab is reached: the sums stay zero
            } else {
                rp0 = lo;
                n_rp = hi - lo + 1;
                cb0 = clo;
                seg_c = chi - clo + 1;
            }
        }
    }
    const int seg = CULL ? seg_c : a.ncb;  // column blocks per row pair in the stream
    const long long blk_begin = CULL ? (long long)rp0 * a.ncb + cb0 : (long long)rp_begin * a.ncb;
    const int n_total = CULL ? n_rp * seg : (rp_end - rp_begin) * a.ncb;
    const int n_chunks = (n_total + PCB - 1) / PCB;
    const float* src = a.prec + ((long long)b * a.nrp * a.ncb + blk_begin) * RS;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
        *s_failed = 0;
        mbar_init_fence();
    }
    __syncthreads();

    auto issue = [&](int chunk) {
        const int st = chunk % NS;
        const int cnt = min(PCB, n_total - chunk * PCB);
        const uint32_t bytes = (uint32_t)cnt * RS * sizeof(float);
        mbar_expect_tx(&bars[st], bytes);
        if constexpr (!CULL) {
            bulk_g2s(stage_base + (size_t)st * PCB * RS, src + (long long)chunk * PCB * RS, bytes, &bars[st]);
        } else {
            // the chunk is a run of the virtual stream: one copy per row pair it touches
            float* dstp = stage_base + (size_t)st * PCB * RS;
            int v = chunk * PCB, left = cnt;
            while (left > 0) {
                const int r = v / seg, c = v - r * seg;
                const int len = min(left, seg - c);
                bulk_g2s(dstp, src + ((long long)r * a.ncb + c) * RS, (uint32_t)len * RS * sizeof(float), &bars[st]);
                dstp += (size_t)len * RS;
                v += len;
                left -= len;
            }
        }
    };
    if (tid == 0) {
        for (int c = 0; c < NS && c < n_chunks; ++c) issue(c);
    }

    int cb = 0;  // block position inside the current row pair (uniform over the CTA)
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
        const int cnt = min(PCB, n_total - chunk * PCB);
        const float4* rec = reinterpret_cast<const float4*>(stage_base + (size_t)st * PCB * RS);

        auto fold_row_pair = [&]() {
            // row pair complete: fold its row sums into the moments
#pragma unroll
            for (int g = 0; g < GPT; ++g)
#pragma unroll
                for (int row = 0; row < 2; ++row) {
                    M[g][0] = add2(M[g][0], hs[g][row]);
                    M[g][1] = add2(M[g][1], hxs[g][row]);
                    M[g][2] = fma2(dyd[g][row], hs[g][row], M[g][2]);
                    M[g][4] = fma2(dyd[g][row], hxs[g][row], M[g][4]);
                    M[g][5] = fma2(mul2(dyd[g][row], dyd[g][row]), hs[g][row], M[g][5]);
                }
        };
#pragma unroll(Cfg::UNROLL)
        for (int i = 0; i < cnt;) {
            const float4* r = rec + (size_t)i * (RS / 4);
            const float4 xc = r[0];
            const f2 xcp[2] = {pk(xc.x, xc.y), pk(xc.z, xc.w)};
            if (cb == 0) {
                // new row pair: row terms of the exponent, fresh row sums
                const float4 yr = r[1];
                const f2 yy = pk(yr.x, yr.y);
                strip_y0 = fminf(yr.x, yr.y);
                strip_y1 = fmaxf(yr.x, yr.y);
#pragma unroll
                for (int g = 0; g < GPT; ++g) {
                    const f2 dyr = sub2(yy, py[g]);
                    float d0, d1, b0, b1, c0, c1;
                    upk(dyr, d0, d1);
                    upk(mul2(B2[g], dyr), b0, b1);
                    upk(mul2(mul2(Cq[g], dyr), dyr), c0, c1);
                    dyd[g][0] = pk(d0, d0); dyd[g][1] = pk(d1, d1);
                    bd[g][0] = pk(b0, b0);  bd[g][1] = pk(b1, b1);
                    cd[g][0] = pk(c0, c0);  cd[g][1] = pk(c1, c1);
                    hs[g][0] = hs[g][1] = hxs[g][0] = hxs[g][1] = 0ull;
                }
            }
            if (cull && must == 0) {
                const int run = min(min(SKIP_RUN, cnt - i), seg - cb);
                const float run_x0 = xc.x, run_x1 = rec[(size_t)(i + run - 1) * (RS / 4)].w;
                bool need = false;
#pragma unroll
                for (int g = 0; g < GPT; ++g)
                    need |= !(box_x1[g] < run_x0 || box_x0[g] > run_x1 || box_y1[g] < strip_y0 || box_y0[g] > strip_y1);
                if (!__any_sync(0xffffffffu, need)) {
                    i += run;
                    cb += run;
                    if (cb == seg) {
                        cb = 0;
                        fold_row_pair();
                    }
                    continue;
                }
                must = run;
            }
            if (cull) {
                --must;
                ++visited;
            }
            f2 dxc[GPT][2], dxx[GPT][2];
#pragma unroll
            for (int g = 0; g < GPT; ++g)
#pragma unroll
                for (int cp = 0; cp < 2; ++cp) {
                    dxc[g][cp] = sub2(xcp[cp], px[g]);
                    dxx[g][cp] = mul2(dxc[g][cp], dxc[g][cp]);
                }
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // j = 2*row + column pair
                const ulonglong2* pr = reinterpret_cast<const ulonglong2*>(r + 2 + j * (PF / 4));
                f2 gterm[PF / 2];  // gS, gn_0 .. gn_{CT-1} (+ pad)
#pragma unroll
                for (int c = 0; c < PF / 4; ++c) {
                    const ulonglong2 rc = pr[c];
                    gterm[2 * c] = rc.x;
                    gterm[2 * c + 1] = rc.y;
                }
                const int row = j >> 1, cp = j & 1;
#pragma unroll
                for (int g = 0; g < GPT; ++g) {
                    const f2 dx = dxc[g][cp];
                    const f2 e = ex2_2(fma2(dx, fma2(A[g], dx, bd[g][row]), cd[g][row]));
                    f2 G = gterm[0];
#pragma unroll
                    for (int c = 0; c < CT; ++c) G = fma2(gterm[1 + c], col[g][c], G);
                    const f2 h = mul2(G, e);
                    hs[g][row] = add2(hs[g][row], h);
                    hxs[g][row] = fma2(h, dx, hxs[g][row]);
                    M[g][3] = fma2(h, dxx[g][cp], M[g][3]);
#pragma unroll
                    for (int c = 0; c < CT; ++c) E[g][c] = fma2(gterm[1 + c], e, E[g][c]);
                }
            }
            ++i;
            if (++cb == seg) {
                cb = 0;
                fold_row_pair();
            }
        }
        __syncthreads();
        if (tid == 0 && chunk + NS < n_chunks) issue(chunk + NS);
    }

    if constexpr (CULL) {
        // a visited block is 8 pixels against the GPT gaussians of each of the warp's 32 lanes
        if ((tid & 31) == 0 && a.exec_count) atomicAdd(a.exec_count, (unsigned long long)visited * (8 * 32 * GPT));
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
            upk(M[g][k], lo, hi);
            dst[(long long)(a.moment_plane0 + k) * a.N] = lo + hi;
        }
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            if (c < a.cr) {
                float lo, hi;
                upk(E[g][c], lo, hi);
                dst[(long long)(a.color_plane0 + a.c0 + c) * a.N] = lo + hi;
            }
        }
    }
}

template <int CT, bool CULL>
static cudaError_t launch_sep_one(const BwdArgs& a, const BwdPlan& p, cudaStream_t s) {
    using Cfg = BwdSepCfg<CT>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(splat_backward_sep_kernel<CT, CULL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    dim3 grid((unsigned)((a.N + Cfg::GAUSS_PER_CTA - 1) / Cfg::GAUSS_PER_CTA), (unsigned)p.n_slab, (unsigned)a.B);
    {
        KernelTimer timer(K_BACKWARD, s);
        splat_backward_sep_kernel<CT, CULL><<<grid, Cfg::THREADS, Cfg::SMEM, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

template <int CT>
static int sep_occ(int device) {
    using Cfg = BwdSepCfg<CT>;
    static int cached[64];
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    cudaFuncSetAttribute(splat_backward_sep_kernel<CT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Cfg::SMEM);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, splat_backward_sep_kernel<CT, false>, Cfg::THREADS,
                                                      Cfg::SMEM) != cudaSuccess ||
        n <= 0) {
        cudaGetLastError();
        n = Cfg::MIN_CTAS;
    }
    if (device >= 0 && device < 64) cached[device] = n;
    return n;
}

// CTAs of the plain separable kernel an SM holds (the plan sizes its slab count by it)
int backward_sep_ctas_per_sm(int ct, int device) {
    switch (ct) {
        case 1: return sep_occ<1>(device);
        case 2: return sep_occ<2>(device);
        case 3: return sep_occ<3>(device);
        case 4: return sep_occ<4>(device);
    }
    return 0;
}

// instantiations exist for single-chunk channel counts up to 4, two gaussians per thread
bool backward_has_separable(int ct) { return ct <= 4 && backward_gauss_per_thread(ct) == BwdSepCfg<3>::GPT; }

cudaError_t launch_backward_sep_chunk(int ct, bool culling, const BwdArgs& a, const BwdPlan& p, cudaStream_t s) {
    switch (ct) {
        case 1: return culling ? launch_sep_one<1, true>(a, p, s) : launch_sep_one<1, false>(a, p, s);
        case 2: return culling ? launch_sep_one<2, true>(a, p, s) : launch_sep_one<2, false>(a, p, s);
        case 3: return culling ? launch_sep_one<3, true>(a, p, s) : launch_sep_one<3, false>(a, p, s);
        case 4: return culling ? launch_sep_one<4, true>(a, p, s) : launch_sep_one<4, false>(a, p, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace igs
