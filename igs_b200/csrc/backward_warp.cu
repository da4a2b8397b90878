// Backward splat kernel for narrow gaussians taken in a spatial order (separable grids).
//
// Same arithmetic, per gaussian and pixel block, as splat_backward_sep_kernel (see
// backward_sep.cu for the factorisation into row sums): the 2 x 4-pixel block records
// stream through shared memory, the moments accumulate in registers.  What differs is who
// decides what to visit.  There, the four warps of a CTA share one stream and meet at a
// barrier after every stage, so a stage costs the time of the warp that skipped least.
// Here every warp is on its own: a thread owns ONE gaussian, the warp forms the box around
// its 32 gaussians (neighbours, thanks to the caller's order), finds the rectangle of
// blocks that box meets inside the slab's rows, and streams just that rectangle through
// two private stages with private mbarriers.  No CTA-wide barrier, no work for a warp
// whose gaussians miss the slab, and no further test inside the rectangle: measured, a
// vote on runs of 8 blocks skipped 3 % more and cost more than that.
// Measured on 16384 gaussians of scale 0.004-0.012 at 1024 x 1024: 0.53 ms against 0.73 ms
// for per-CTA skipping and 8.8 ms for the dense kernel; two gaussians per thread (fewer
// shared-memory reads per evaluation, but 160 registers, 12 warps per SM) took 0.66 ms.
//
// Every gaussian's sums run over the slab's pixels in the same sequence as in the other
// two separable kernels, and the skipped terms are exact zeros, so the partial sums are
// the same bits.
#include "backward.cuh"

namespace igs {

#ifndef IGS_BWDW_GPT
#define IGS_BWDW_GPT 1
#endif
#ifndef IGS_BWDW_THREADS
#define IGS_BWDW_THREADS 64
#endif
#ifndef IGS_BWDW_MINCTAS
#define IGS_BWDW_MINCTAS 10
#endif
#ifndef IGS_BWDW_STAGE
#define IGS_BWDW_STAGE 16
#endif

template <int CT>
struct BwdWarpCfg {
    static constexpr int THREADS = IGS_BWDW_THREADS;
    static constexpr int WARPS = THREADS / 32;
    static constexpr int GPT = IGS_BWDW_GPT;  // gaussians per thread
    static constexpr int GAUSS_PER_CTA = THREADS * GPT;
    static constexpr int STAGE_BLOCKS = IGS_BWDW_STAGE;  // 2x4-pixel blocks per warp-private stage
    static constexpr int STAGES = 2;
    static constexpr int MIN_CTAS = IGS_BWDW_MINCTAS;
    static constexpr int RS = bwd_sep_rec_floats(CT);
    static constexpr int PF = bwd_sep_pair_floats(CT);
    static constexpr size_t SMEM =
        (size_t)WARPS * STAGES * STAGE_BLOCKS * RS * sizeof(float) + (size_t)WARPS * STAGES * sizeof(uint64_t);
};

template <int CT>
__global__ void __launch_bounds__(BwdWarpCfg<CT>::THREADS, BwdWarpCfg<CT>::MIN_CTAS) splat_backward_warp_kernel(BwdArgs a) {
    using Cfg = BwdWarpCfg<CT>;
    constexpr int GPT = Cfg::GPT, PCB = Cfg::STAGE_BLOCKS, NS = Cfg::STAGES, RS = Cfg::RS, PF = Cfg::PF;
    constexpr unsigned FULL = 0xffffffffu;

    // runs instead of the other separable kernels when the grid is separable with
    // non-decreasing axes and at least one gaussian in eight is narrow
    if (a.grid_sel && (*a.grid_sel & GRID_NOT_SEPARABLE)) return;
    if ((*a.grid_word & NO_BACKWARD_SKIPPING) || (long long)(*a.cull_sel) * 8 < (long long)a.B * a.N) return;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.z, slab = blockIdx.y;
    float* stage_base = reinterpret_cast<float*>(smem_raw) + (size_t)warp * NS * PCB * RS;
    uint64_t* bars =
        reinterpret_cast<uint64_t*>(smem_raw + (size_t)Cfg::WARPS * NS * PCB * RS * sizeof(float)) + warp * NS;

    // ---- this thread's gaussians (slot -> gaussian through the caller's order) ----
    int n[GPT];
    f2 px[GPT], py[GPT], A[GPT], B2[GPT], Cq[GPT], col[GPT][CT];
    float box_x0[GPT], box_x1[GPT], box_y0[GPT], box_y1[GPT];
#pragma unroll
    for (int g = 0; g < GPT; ++g) {
        const int slot = blockIdx.x * Cfg::GAUSS_PER_CTA + tid * GPT + g;
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
        box_x0[g] = g0.x - g1.z;
        box_x1[g] = g0.x + g1.z;
        box_y0[g] = g0.y - g1.w;
        box_y1[g] = g0.y + g1.w;
        if (n[g] >= a.N) {  // an empty slot reaches nothing
            box_x0[g] = box_y0[g] = INFINITY;
            box_x1[g] = box_y1[g] = -INFINITY;
        }
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const float v = (c < a.cr) ? a.colors[((long long)b * a.N + nn) * a.C + a.c0 + c] : 0.f;
            col[g][c] = pk(v, v);
        }
    }

    // ---- the warp's rectangle of blocks inside this slab ----
    const int rp_begin = min(a.nrp, slab * a.rp_per_slab);
    const int rp_end = min(a.nrp, rp_begin + a.rp_per_slab);
    int rp0 = rp_begin, n_rp = rp_end - rp_begin, cb0 = 0, seg = a.ncb;
    {
        float u[4] = {INFINITY, -INFINITY, INFINITY, -INFINITY};  // x0, x1, y0, y1 of the union
        bool open_box = false;                                    // a NaN or infinite box: no restriction
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
            u[0] = fminf(u[0], __shfl_xor_sync(FULL, u[0], d));
            u[1] = fmaxf(u[1], __shfl_xor_sync(FULL, u[1], d));
            u[2] = fminf(u[2], __shfl_xor_sync(FULL, u[2], d));
            u[3] = fmaxf(u[3], __shfl_xor_sync(FULL, u[3], d));
        }
        if (!__any_sync(FULL, open_box)) {
            const float* rec0 = a.prec + (long long)b * a.nrp * a.ncb * RS;
            int lo = 0x7fffffff, hi = -1, clo = 0x7fffffff, chi = -1;
            for (int rp = rp_begin + lane; rp < rp_end; rp += 32) {
                const float4 yr = reinterpret_cast<const float4*>(rec0 + (long long)rp * a.ncb * RS)[1];
                if (!(u[3] < fminf(yr.x, yr.y) || u[2] > fmaxf(yr.x, yr.y))) {
                    lo = min(lo, rp);
                    hi = max(hi, rp);
                }
            }
            for (int cb = lane; cb < a.ncb; cb += 32) {
                const float4 xc = reinterpret_cast<const float4*>(rec0 + (long long)cb * RS)[0];
                if (!(u[1] < xc.x || u[0] > xc.w)) {
                    clo = min(clo, cb);
                    chi = max(chi, cb);
                }
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                lo = min(lo, __shfl_xor_sync(FULL, lo, d));
                hi = max(hi, __shfl_xor_sync(FULL, hi, d));
                clo = min(clo, __shfl_xor_sync(FULL, clo, d));
                chi = max(chi, __shfl_xor_sync(FULL, chi, d));
            }
            if (hi < lo || chi < clo) {
                n_rp = 0;  // nothing of this slab is reached: the sums stay zero
            } else {
                rp0 = lo;
                n_rp = hi - lo + 1;
                cb0 = clo;
                seg = chi - clo + 1;
            }
        }
    }
    const int n_total = n_rp * seg;
    const int n_chunks = (n_total + PCB - 1) / PCB;
    const float* src = a.prec + (((long long)b * a.nrp + rp0) * a.ncb + cb0) * RS;

    // moments M0, Mx, My, Mxx, Mxy, Myy and colour sums E_c; per-row state of the current row pair
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

    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
        mbar_init_fence();
    }
    __syncwarp();

    // a stage is a run of the virtual stream (rows of the rectangle, one after another):
    // one bulk copy per row pair it touches
    auto issue = [&](int chunk) {
        const int st = chunk % NS;
        const int cnt = min(PCB, n_total - chunk * PCB);
        mbar_expect_tx(&bars[st], (uint32_t)cnt * RS * sizeof(float));
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
    };
    if (lane == 0) {
        for (int c = 0; c < NS && c < n_chunks; ++c) issue(c);
    }

    int visited = 0;  // blocks evaluated
    int cb = 0;       // block position inside the current row of the rectangle
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        const int st = chunk % NS;
        const bool ok = mbar_wait_bounded(&bars[st], (chunk / NS) & 1);
        if (!__all_sync(FULL, ok)) {
            // give the copies still in flight a bounded chance to land before the CTA's
            // shared memory can go away, report, and leave; the other warps carry on
            if (lane == 0) {
                for (int c = chunk + 1; c < n_chunks && c < chunk + NS; ++c)
                    mbar_wait_bounded(&bars[c % NS], (c / NS) & 1);
                atomicOr(a.status, STATUS_WAIT_TIMEOUT);
            }
            return;
        }
        const int cnt = min(PCB, n_total - chunk * PCB);
        const float4* rec = reinterpret_cast<const float4*>(stage_base + (size_t)st * PCB * RS);

        auto fold_row_pair = [&]() {
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
        for (int i = 0; i < cnt;) {
            const float4* r = rec + (size_t)i * (RS / 4);
            const float4 xc = r[0];
            const f2 xcp[2] = {pk(xc.x, xc.y), pk(xc.z, xc.w)};
            if (cb == 0) {
                // new row pair: row terms of the exponent, fresh row sums
                const float4 yr = r[1];
                const f2 yy = pk(yr.x, yr.y);
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
            ++visited;
            f2 dxc[GPT][2], adx[GPT][2];
#pragma unroll
            for (int g = 0; g < GPT; ++g)
#pragma unroll
                for (int cp = 0; cp < 2; ++cp) {
                    dxc[g][cp] = sub2(xcp[cp], px[g]);
                    adx[g][cp] = mul2(A[g], dxc[g][cp]);
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
                    const f2 e = ex2_2(fma2(dx, add2(adx[g][cp], bd[g][row]), cd[g][row]));
                    f2 G = gterm[0];
#pragma unroll
                    for (int c = 0; c < CT; ++c) G = fma2(gterm[1 + c], col[g][c], G);
                    const f2 h = mul2(G, e);
                    hs[g][row] = add2(hs[g][row], h);
                    const f2 hx = mul2(h, dx);
                    hxs[g][row] = add2(hxs[g][row], hx);
                    M[g][3] = fma2(hx, dx, M[g][3]);
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
        __syncwarp();  // every lane is done with this stage
        if (lane == 0 && chunk + NS < n_chunks) issue(chunk + NS);
    }

    if (lane == 0 && a.exec_count) atomicAdd(a.exec_count, (unsigned long long)visited * (8 * 32 * GPT));

#pragma unroll
    for (int g = 0; g < GPT; ++g) {
        if (n[g] >= a.N) continue;
        float* dst = a.part + ((long long)slab * a.B + b) * a.planes * (long long)a.N + n[g];
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

template <int CT>
static cudaError_t launch_warp_one(const BwdArgs& a, const BwdPlan& p, cudaStream_t s) {
    using Cfg = BwdWarpCfg<CT>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(splat_backward_warp_kernel<CT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    dim3 grid((unsigned)((a.N + Cfg::GAUSS_PER_CTA - 1) / Cfg::GAUSS_PER_CTA), (unsigned)p.n_slab, (unsigned)a.B);
    {
        KernelTimer timer(K_BACKWARD, s);
        splat_backward_warp_kernel<CT><<<grid, Cfg::THREADS, Cfg::SMEM, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

// the skipping kernel for calls that pass a processing order (needs a.cull_sel and a.grid_word)
cudaError_t launch_backward_warp_chunk(int ct, const BwdArgs& a, const BwdPlan& p, cudaStream_t s) {
    if (!a.cull_sel || !a.grid_word) return cudaErrorInvalidValue;
    switch (ct) {
        case 1: return launch_warp_one<1>(a, p, s);
        case 2: return launch_warp_one<2>(a, p, s);
        case 3: return launch_warp_one<3>(a, p, s);
        case 4: return launch_warp_one<4>(a, p, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace igs
