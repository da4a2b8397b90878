// Backward splat for narrow gaussians taken in a spatial order (separable grids).
//
// Same arithmetic, per gaussian and pixel block, as splat_backward_sep_kernel (see
// backward_sep.cu for the factorisation into row sums): the 2 x 4-pixel block records
// stream through shared memory, the moments accumulate in registers.  What differs is who
// decides what to visit, and how the work is handed out.
//
// A task is (32 consecutive gaussians of the caller's order, one slab of rows).  A thread
// owns ONE gaussian; the warp forms the box around its 32 gaussians (neighbours, thanks to
// the order), and the task covers the rectangle of blocks that box meets inside the slab.
//   warp_task_kernel   one warp per group of 32 gaussians: box -> rows and columns it meets
//                      -> one task per slab those rows touch, appended to a list in the
//                      workspace (the slot comes from an integer atomicAdd; the order of
//                      the list does not matter, every task writes its own partial sums)
//   splat_backward_queue_kernel   as many warps as the GPU holds, each taking the next task
//                      off the list until it is empty: streams the task's rectangle through
//                      two private stages with private mbarriers and writes the partial
//                      sums of its 32 gaussians for that slab
// (Group, slab) pairs that are not on the list contribute exact zeros and their partial sums
// are never written: warp_task_kernel leaves, per slot, the range of slabs its group has
// tasks for, and finalize_kernel adds up those only (the sums that are left out are exact
// zeros, so the result's bits do not change).
//
// Why a list: with one CTA per (group, slab) pair four fifths of the CTAs found nothing to
// do, and an SM held 12.8 of its 20 possible warps on average; a warp that pulls tasks
// stays busy until the list is empty.  Why warps and not CTAs: warps of one CTA that share
// a stream meet at a barrier after every stage, so a stage costs the time of the warp that
// skipped least.  Two gaussians per thread (fewer shared-memory reads per evaluation, but
// 160 registers, 12 warps per SM) were slower than one; so was a vote on runs of 8 blocks
// inside the rectangle (it skipped 3 % more and cost more than that).
//
// Every gaussian's sums run over the slab's pixels in the same sequence as in the other
// separable kernels, and the skipped terms are exact zeros, so the partial sums are the
// same bits -- whatever the order of the task list.
#include "backward.cuh"

namespace igs {

constexpr int BWDW_THREADS = 64;
constexpr int BWDW_MINCTAS = 8;  // 16 warps per SM at 126 registers (10: 96 registers and a spill, slower)
constexpr int BWDW_STAGE = 32;

template <int CT>
struct BwdWarpCfg {
    static constexpr int THREADS = BWDW_THREADS;
    static constexpr int WARPS = THREADS / 32;
    static constexpr int STAGE_BLOCKS = BWDW_STAGE;  // 2x4-pixel blocks per warp-private stage
    static constexpr int STAGES = 2;
    static constexpr int MIN_CTAS = BWDW_MINCTAS;
    static constexpr int RS = bwd_sep_rec_floats(CT);
    static constexpr int PF = bwd_sep_pair_floats(CT);
    static constexpr size_t SMEM =
        (size_t)WARPS * STAGES * STAGE_BLOCKS * RS * sizeof(float) + (size_t)WARPS * STAGES * sizeof(uint64_t);
};

// the kernels of this file run when the grid is separable with non-decreasing axes, the
// upstream values are finite and at least one gaussian in eight is narrow
__device__ __forceinline__ bool warp_path_selected(const BwdArgs& a) {
    if (a.grid_sel && (*a.grid_sel & GRID_NOT_SEPARABLE)) return false;
    return !(*a.grid_word & NO_BACKWARD_SKIPPING) && (long long)(*a.cull_sel) * 8 >= (long long)a.B * a.N;
}

// ---------------------------------------------------------------------------
// task list
// ---------------------------------------------------------------------------
// One warp per group: group g of batch element b holds the slots 32 g .. 32 g + 31.
__global__ void __launch_bounds__(128) warp_task_kernel(BwdArgs a, int rs) {
    constexpr unsigned FULL = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int group = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), b = blockIdx.y;
    const int n_groups = (a.N + 31) / 32;
    if (group >= n_groups) return;

    const int slot = group * 32 + lane;
    int n = slot < a.N ? (a.order ? a.order[(long long)b * a.N + slot] : slot) : a.N;
    if ((unsigned)n > (unsigned)a.N) n = a.N;
    if (!warp_path_selected(a)) {
        // another kernel does the work and fills every slab
        if (slot < a.N) a.slab_range[(long long)b * a.N + slot] = a.n_slab << 16;
        return;
    }
    float u[4] = {INFINITY, -INFINITY, INFINITY, -INFINITY};  // x0, x1, y0, y1 of the group's box
    bool open_box = false;                                    // a NaN or infinite box: no restriction
    if (n < a.N) {
        const float4* gp = reinterpret_cast<const float4*>(a.geo + ((long long)b * a.N + n) * GEO_FLOATS);
        const float4 g0 = gp[0], g1 = gp[1];
        u[0] = g0.x - g1.z;
        u[1] = g0.x + g1.z;
        u[2] = g0.y - g1.w;
        u[3] = g0.y + g1.w;
        open_box = !(u[1] - u[0] < INFINITY) || !(u[3] - u[2] < INFINITY);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        u[0] = fminf(u[0], __shfl_xor_sync(FULL, u[0], d));
        u[1] = fmaxf(u[1], __shfl_xor_sync(FULL, u[1], d));
        u[2] = fminf(u[2], __shfl_xor_sync(FULL, u[2], d));
        u[3] = fmaxf(u[3], __shfl_xor_sync(FULL, u[3], d));
    }
    int lo = 0, hi = a.nrp - 1, clo = 0, chi = a.ncb - 1;
    if (!__any_sync(FULL, open_box)) {
        // rows and columns of blocks the box meets (non-decreasing axes: contiguous ranges)
        const float* rec0 = a.prec + (long long)b * a.nrp * a.ncb * rs;
        lo = 0x7fffffff, hi = -1, clo = 0x7fffffff, chi = -1;
        for (int rp = lane; rp < a.nrp; rp += 32) {
            const float4 yr = reinterpret_cast<const float4*>(rec0 + (long long)rp * a.ncb * rs)[1];
            if (!(u[3] < fminf(yr.x, yr.y) || u[2] > fmaxf(yr.x, yr.y))) {
                lo = min(lo, rp);
                hi = max(hi, rp);
            }
        }
        for (int cb = lane; cb < a.ncb; cb += 32) {
            const float4 xc = reinterpret_cast<const float4*>(rec0 + (long long)cb * rs)[0];
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
    }
    if (hi < lo || chi < clo) {  // the group reaches no pixel: no task, no slab to add up
        if (slot < a.N) a.slab_range[(long long)b * a.N + slot] = 0;
        return;
    }
    const int s0 = lo / a.rp_per_slab, s1 = hi / a.rp_per_slab;
    if (slot < a.N) a.slab_range[(long long)b * a.N + slot] = s0 | ((s1 + 1) << 16);
    int base = 0;
    if (lane == 0) {
        a.group_rect[(long long)b * n_groups + group] = make_int4(lo, hi, clo, chi);
        base = atomicAdd(a.task_count, s1 - s0 + 1);
    }
    base = __shfl_sync(FULL, base, 0);
    for (int s = s0 + lane; s <= s1; s += 32) {
        const int t = base + (s - s0);
        if (t < a.task_capacity) a.tasks[t] = make_int4(b, group, s, 0);
    }
}

// ---------------------------------------------------------------------------
// task queue
// ---------------------------------------------------------------------------
template <int CT>
__global__ void __launch_bounds__(BwdWarpCfg<CT>::THREADS, BwdWarpCfg<CT>::MIN_CTAS) splat_backward_queue_kernel(BwdArgs a) {
    using Cfg = BwdWarpCfg<CT>;
    constexpr int PCB = Cfg::STAGE_BLOCKS, NS = Cfg::STAGES, RS = Cfg::RS, PF = Cfg::PF;
    constexpr unsigned FULL = 0xffffffffu;
    if (!warp_path_selected(a)) return;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* stage_base = reinterpret_cast<float*>(smem_raw) + (size_t)warp * NS * PCB * RS;
    uint64_t* bars =
        reinterpret_cast<uint64_t*>(smem_raw + (size_t)Cfg::WARPS * NS * PCB * RS * sizeof(float)) + warp * NS;
    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
        mbar_init_fence();
    }
    __syncwarp();

    const int n_groups = (a.N + 31) / 32;
    const int n_tasks = min(*a.task_count, a.task_capacity);
    unsigned it = 0;        // stages this warp has consumed so far: stage and parity of the next one
    long long visited = 0;  // blocks evaluated

    for (;;) {
        int t = 0;
        if (lane == 0) t = atomicAdd(a.task_next, 1);
        t = __shfl_sync(FULL, t, 0);
        if (t >= n_tasks) break;
        const int4 task = a.tasks[t];
        const int b = task.x, group = task.y, slab = task.z;
        const int4 rect = a.group_rect[(long long)b * n_groups + group];  // rows lo..hi, columns clo..chi

        // ---- this thread's gaussian (slot -> gaussian through the caller's order) ----
        const int slot = group * 32 + lane;
        int n = slot < a.N ? (a.order ? a.order[(long long)b * a.N + slot] : slot) : a.N;
        if ((unsigned)n > (unsigned)a.N) n = a.N;  // an entry that is no index: the slot stays empty
        const int nn = n < a.N ? n : a.N - 1;
        const float4* gp = reinterpret_cast<const float4*>(a.geo + ((long long)b * a.N + nn) * GEO_FLOATS);
        const float4 g0 = gp[0], g1 = gp[1];
        const f2 px = pk(g0.x, g0.x), py = pk(g0.y, g0.y), A = pk(g0.z, g0.z), B2 = pk(g0.w, g0.w), Cq = pk(g1.x, g1.x);
        f2 col[CT];
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const float v = (c < a.cr) ? a.colors[((long long)b * a.N + nn) * a.C + a.c0 + c] : 0.f;
            col[c] = pk(v, v);
        }

        // ---- the task's rectangle: the group's rows inside this slab, the group's columns ----
        const int rp_begin = min(a.nrp, slab * a.rp_per_slab);
        const int rp_end = min(a.nrp, rp_begin + a.rp_per_slab);
        const int rp0 = max(rp_begin, rect.x);
        const int n_rp = max(0, min(rp_end, rect.y + 1) - rp0);
        const int cb0 = rect.z, seg = rect.w - rect.z + 1;
        const int n_total = n_rp * seg;
        const int n_chunks = (n_total + PCB - 1) / PCB;
        const float* src = a.prec + (((long long)b * a.nrp + rp0) * a.ncb + cb0) * RS;

        // moments M0, Mx, My, Mxx, Mxy, Myy and colour sums E_c; per-row state of the current row pair
        f2 M[N_MOMENTS], E[CT];
        f2 dyd[2], bd[2], cd[2], hs[2], hxs[2];
#pragma unroll
        for (int k = 0; k < N_MOMENTS; ++k) M[k] = 0ull;
#pragma unroll
        for (int c = 0; c < CT; ++c) E[c] = 0ull;
#pragma unroll
        for (int r = 0; r < 2; ++r) dyd[r] = bd[r] = cd[r] = hs[r] = hxs[r] = 0ull;

        // a stage is a run of the virtual stream (rows of the rectangle, one after another):
        // one bulk copy per row pair it touches
        auto issue = [&](int chunk) {
            const int st = (it + chunk) % NS;
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

        int cb = 0;  // block position inside the current row of the rectangle
        for (int chunk = 0; chunk < n_chunks; ++chunk) {
            const unsigned use = it + chunk;
            const int st = use % NS;
            const bool ok = mbar_wait_bounded(&bars[st], (use / NS) & 1);
            if (!__all_sync(FULL, ok)) {
                // give the copies still in flight a bounded chance to land before the CTA's
                // shared memory can go away, report, and leave; the other warps carry on
                if (lane == 0) {
                    for (int c = chunk + 1; c < n_chunks && c < chunk + NS; ++c)
                        mbar_wait_bounded(&bars[(it + c) % NS], ((it + c) / NS) & 1);
                    atomicOr(a.status, STATUS_WAIT_TIMEOUT);
                }
                return;
            }
            const int cnt = min(PCB, n_total - chunk * PCB);
            const float4* rec = reinterpret_cast<const float4*>(stage_base + (size_t)st * PCB * RS);

            auto fold_row_pair = [&]() {
#pragma unroll
                for (int row = 0; row < 2; ++row) {
                    M[0] = add2(M[0], hs[row]);
                    M[1] = add2(M[1], hxs[row]);
                    M[2] = fma2(dyd[row], hs[row], M[2]);
                    M[4] = fma2(dyd[row], hxs[row], M[4]);
                    M[5] = fma2(mul2(dyd[row], dyd[row]), hs[row], M[5]);
                }
            };
            for (int i = 0; i < cnt; ++i) {
                const float4* r = rec + (size_t)i * (RS / 4);
                const float4 xc = r[0];
                const f2 xcp[2] = {pk(xc.x, xc.y), pk(xc.z, xc.w)};
                if (cb == 0) {
                    // new row pair: row terms of the exponent, fresh row sums
                    const float4 yr = r[1];
                    const f2 dyr = sub2(pk(yr.x, yr.y), py);
                    float d0, d1, b0, b1, c0, c1;
                    upk(dyr, d0, d1);
                    upk(mul2(B2, dyr), b0, b1);
                    upk(mul2(mul2(Cq, dyr), dyr), c0, c1);
                    dyd[0] = pk(d0, d0); dyd[1] = pk(d1, d1);
                    bd[0] = pk(b0, b0);  bd[1] = pk(b1, b1);
                    cd[0] = pk(c0, c0);  cd[1] = pk(c1, c1);
                    hs[0] = hs[1] = hxs[0] = hxs[1] = 0ull;
                }
                f2 dxc[2], dxx[2];
#pragma unroll
                for (int cp = 0; cp < 2; ++cp) {
                    dxc[cp] = sub2(xcp[cp], px);
                    dxx[cp] = mul2(dxc[cp], dxc[cp]);
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
                    const f2 dx = dxc[cp];
                    const f2 e = ex2_2(fma2(dx, fma2(A, dx, bd[row]), cd[row]));
                    f2 G = gterm[0];
#pragma unroll
                    for (int c = 0; c < CT; ++c) G = fma2(gterm[1 + c], col[c], G);
                    const f2 h = mul2(G, e);
                    hs[row] = add2(hs[row], h);
                    hxs[row] = fma2(h, dx, hxs[row]);
                    M[3] = fma2(h, dxx[cp], M[3]);
#pragma unroll
                    for (int c = 0; c < CT; ++c) E[c] = fma2(gterm[1 + c], e, E[c]);
                }
                if (++cb == seg) {
                    cb = 0;
                    fold_row_pair();
                }
            }
            visited += cnt;
            __syncwarp();  // every lane is done with this stage
            if (lane == 0 && chunk + NS < n_chunks) issue(chunk + NS);
        }
        it += (unsigned)n_chunks;

        if (n < a.N) {
            float* dst = a.part + ((long long)slab * a.B + b) * a.planes * (long long)a.N + slot;  // by slot
#pragma unroll
            for (int k = 0; k < N_MOMENTS; ++k) {
                float lo, hi;
                upk(M[k], lo, hi);
                dst[(long long)(a.moment_plane0 + k) * a.N] = lo + hi;
            }
#pragma unroll
            for (int c = 0; c < CT; ++c) {
                if (c < a.cr) {
                    float lo, hi;
                    upk(E[c], lo, hi);
                    dst[(long long)(a.color_plane0 + a.c0 + c) * a.N] = lo + hi;
                }
            }
        }
    }
    if (lane == 0 && a.exec_count && visited) atomicAdd(a.exec_count, (unsigned long long)visited * (8 * 32));
}

template <int CT>
static cudaError_t launch_queue_one(const BwdArgs& a, int n_ctas, cudaStream_t s) {
    using Cfg = BwdWarpCfg<CT>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(splat_backward_queue_kernel<CT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    {
        KernelTimer timer(K_BACKWARD, s);
        splat_backward_queue_kernel<CT><<<(unsigned)n_ctas, Cfg::THREADS, Cfg::SMEM, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

// The skipping backward for calls that pass a processing order (needs a.cull_sel, a.grid_word,
// a.tasks, a.group_rect, a.task_count, a.task_next, a.slab_range).
cudaError_t launch_backward_warp_chunk(int ct, const BwdArgs& a, const BwdPlan& p, int sm_count, cudaStream_t s) {
    if (!a.cull_sel || !a.grid_word || !a.tasks || !a.group_rect || !a.task_count || !a.task_next || !a.slab_range)
        return cudaErrorInvalidValue;
    (void)p;
    const int n_groups = (a.N + 31) / 32;
    if (n_groups <= 0 || a.B <= 0) return cudaSuccess;
    {
        KernelTimer timer(K_BACKWARD, s);
        warp_task_kernel<<<dim3((unsigned)((n_groups + 3) / 4), (unsigned)a.B), 128, 0, s>>>(a, bwd_sep_rec_floats(ct));
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int n_ctas = sm_count * BWDW_MINCTAS;  // as many warps as stay resident; each pulls tasks until none is left
    switch (ct) {
        case 1: return launch_queue_one<1>(a, n_ctas, s);
        case 2: return launch_queue_one<2>(a, n_ctas, s);
        case 3: return launch_queue_one<3>(a, n_ctas, s);
        case 4: return launch_queue_one<4>(a, n_ctas, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace igs
