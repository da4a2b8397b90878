// Forward splat kernel (sm_100a).
//
// One CTA owns a tile of pixels of one batch element and one range ("split") of
// gaussians.  Each thread keeps PX pixels in registers as PX/2 packed pairs:
// coordinates, the weight sum and CT colour numerators, all fp32.  Gaussian records
// stream through shared memory in stages filled by 1-D bulk (TMA) copies that
// complete on an mbarrier; every lane reads the same record, so the shared-memory
// reads are broadcasts and the arithmetic is f32x2 throughout:
//   dx = x - px, dy = y - py
//   q  = dx*(A*dx + B2*dy) + (Cq*dy)*dy            (pre-scaled by -0.5*log2 e)
//   e  = ex2(q);  S += e*alpha;  num_c += e*(alpha*colour_c)
// i.e. 11 FMA-pipe instructions and one MUFU per gaussian x pixel at C = 3.
//
// Two instantiations per channel count:
//   general (SEP = false): any sample coordinates x[b,h,w], y[b,h,w]; a thread's pixels
//     are consecutive pairs of the flattened image;
//   separable (SEP = true): x depends on the column only and y on the row only (what
//     xy_grid produces).  A thread owns a 2-row x 4-column patch, so dx is computed once
//     per column pair and dy, B2*dy, Cq*dy^2 once per row, and the exponent is two FMAs:
//     7.5 instead of 11 FMA-pipe instructions per evaluation.
// Which one applies is a property of the data; grid_check_kernel (grid.cu) decides it on
// the device and both instantiations are launched, the one whose mode does not match
// the flag returning at once (no host synchronisation).
//
// Epilogue: with a single split the CTA divides by (S + eps) itself, otherwise it
// stores un-normalised partial sums that reduce_normalize_kernel adds in split order
// (deterministic; no atomics anywhere).
#include "forward.cuh"

namespace igs {

// PX = pixels per thread.  A forward record costs 3 sixteen-byte broadcast reads per
// thread whatever PX is (12 cycles of the shared-memory return path per warp), against
// 11 f32x2 instructions per pixel pair; more pixels per thread move the balance from
// the return path to the FMA pipe at the price of registers (occupancy).  Measured at
// C = 3: PX = 8 with 4 CTAs/SM and the gaussian loop unrolled 4x is the fastest.
template <int CT, int PX_>
struct FwdCfg {
    static constexpr int THREADS = 128;
    static constexpr int PX = PX_;
    static constexpr int CHUNK_G = 128;  // gaussians per stage
    static constexpr int STAGES = 2;
    static constexpr int MIN_CTAS = (PX_ * (CT + 3) >= 128) ? 2 : ((PX_ * (CT + 3) >= 64) ? 3 : 4);
    static constexpr int UNROLL = CT <= 3 ? 4 : 2;
    static constexpr int RS = fwd_rec_floats(CT);
    // The culling kernel spends little time per stage (most gaussians are skipped), so the
    // latency of a stage's copy shows unless more copies are in flight.
    static constexpr int STAGES_CULL = 4;
    static constexpr int LIST_CAP = 8192;  // stages a CTA can list (ordered calls): 2^20 gaussians per split
    // stages | mbarriers | flags (16 B) | surviving-gaussian list of the current stage | per-warp scratch |
    // list of the stages whose box meets the CTA's pixels
    static constexpr size_t smem_bytes(int stages, int list_cap) {
        return (size_t)stages * CHUNK_G * RS * sizeof(float) + stages * sizeof(uint64_t) + 16 +
               CHUNK_G * sizeof(unsigned short) + 8 * 4 * sizeof(float) + list_cap * sizeof(unsigned short);
    }
    static constexpr size_t SMEM = smem_bytes(STAGES, 1024);  // (the plain kernels never list)
    static constexpr size_t SMEM_CULL = smem_bytes(STAGES_CULL, LIST_CAP);
};

// Separable tiles: 16 rows x 64 columns per CTA, 2 rows x 4 columns per thread.
constexpr int SEP_TILE_H = 16, SEP_TILE_W = 64;

template <int CT, int PX_, bool SEP, bool CULL>
__global__ void __launch_bounds__(FwdCfg<CT, PX_>::THREADS, FwdCfg<CT, PX_>::MIN_CTAS)
    splat_forward_kernel(FwdArgs a) {
    using Cfg = FwdCfg<CT, PX_>;
    constexpr int T = Cfg::THREADS, NP = Cfg::PX / 2, G = Cfg::CHUNK_G, RS = Cfg::RS;
    constexpr int NS = CULL ? Cfg::STAGES_CULL : Cfg::STAGES;
    static_assert(!SEP || PX_ == 8, "the separable patch is 2 rows x 4 columns");

    // only the instantiation that matches the grid's kind does the work
    if (a.grid_sel && (((*a.grid_sel & GRID_NOT_SEPARABLE) != 0) == SEP)) return;
    // ... and, of the culling / non-culling pair, the one the gaussians' reach calls for:
    // culling pays when at least one gaussian in eight is narrow (counted by pack_kernel)
    if (a.cull_sel && (((long long)(*a.cull_sel) * 8 >= (long long)a.B * a.N) != CULL)) return;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage_base = reinterpret_cast<float*>(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NS * G * RS * sizeof(float));
    int* s_failed = reinterpret_cast<int*>(bars + NS);
    unsigned short* s_list = reinterpret_cast<unsigned short*>(s_failed + 4);
    float* s_warp = reinterpret_cast<float*>(s_list + G);  // [4 warps][4] bounding box partials, then counts
    unsigned short* s_stages = reinterpret_cast<unsigned short*>(s_warp + 32);  // [LIST_CAP]

    const int tid = threadIdx.x;
    const int b = blockIdx.z, split = blockIdx.y;
    const long long HW = (long long)a.H * a.W;

    // ---- this thread's pixels: pair j, lane k -> (row, column) ----
    // general: consecutive pairs of the flattened image, interleaved over the CTA's threads
    const long long tile_base = (long long)blockIdx.x * (T * Cfg::PX);
    // separable: rows h0, h0+1 and columns w0 .. w0+3
    const int tile_y = SEP ? (int)(blockIdx.x / a.tiles_x) : 0, tile_x = SEP ? (int)(blockIdx.x % a.tiles_x) : 0;
    const int h0 = tile_y * SEP_TILE_H + (tid >> 4) * 2, w0 = tile_x * SEP_TILE_W + (tid & 15) * 4;

    f2 xx[NP], yy[NP];  // general: per pair.  separable: xx[0..1] = column pairs, yy[0] = {row0,row1}
    if constexpr (SEP) {
        float xv[4], yv[2];
#pragma unroll
        for (int k = 0; k < 4; ++k) xv[k] = a.x[b * a.xs_b + (long long)min(w0 + k, a.W - 1) * a.xs_w];
#pragma unroll
        for (int k = 0; k < 2; ++k) yv[k] = a.y[b * a.ys_b + (long long)min(h0 + k, a.H - 1) * a.ys_h];
        xx[0] = pk(xv[0], xv[1]);
        xx[1] = pk(xv[2], xv[3]);
        yy[0] = pk(yv[0], yv[1]);
    } else {
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const long long p0 = tile_base + (long long)(j * T + tid) * 2;
            float xv[2], yv[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const long long p = p0 + k;
                if (p < HW) {
                    const long long h = p / a.W, w = p - h * a.W;
                    xv[k] = a.x[b * a.xs_b + h * a.xs_h + w * a.xs_w];
                    yv[k] = a.y[b * a.ys_b + h * a.ys_h + w * a.ys_w];
                } else {
                    xv[k] = 0.f;
                    yv[k] = 0.f;
                }
            }
            xx[j] = pk(xv[0], xv[1]);
            yy[j] = pk(yv[0], yv[1]);
        }
    }

    f2 S[NP], acc[NP][CT];
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        S[j] = 0ull;
#pragma unroll
        for (int c = 0; c < CT; ++c) acc[j][c] = 0ull;
    }

    // ---- culling: is it worth it, and what is this CTA's bounding box of sample points? ----
    // (gaussians whose zero-weight box misses the CTA's box contribute exactly 0 to every
    // pixel here and are skipped; decided per launch from the count of narrow gaussians)
    bool cull = CULL;
    float bx0 = 0.f, bx1 = 0.f, by0 = 0.f, by1 = 0.f;
    if constexpr (CULL) {
        float lo_x = INFINITY, hi_x = -INFINITY, lo_y = INFINITY, hi_y = -INFINITY;
        bool bad = false;
        constexpr int NX = SEP ? 2 : NP, NY = SEP ? 1 : NP;
#pragma unroll
        for (int j = 0; j < NX; ++j) {
            float v0, v1;
            upk(xx[j], v0, v1);
            lo_x = fminf(lo_x, fminf(v0, v1));
            hi_x = fmaxf(hi_x, fmaxf(v0, v1));
            bad |= !(v0 == v0) || !(v1 == v1);
        }
#pragma unroll
        for (int j = 0; j < NY; ++j) {
            float v0, v1;
            upk(yy[j], v0, v1);
            lo_y = fminf(lo_y, fminf(v0, v1));
            hi_y = fmaxf(hi_y, fmaxf(v0, v1));
            bad |= !(v0 == v0) || !(v1 == v1);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo_x = fminf(lo_x, __shfl_xor_sync(0xffffffffu, lo_x, o));
            hi_x = fmaxf(hi_x, __shfl_xor_sync(0xffffffffu, hi_x, o));
            lo_y = fminf(lo_y, __shfl_xor_sync(0xffffffffu, lo_y, o));
            hi_y = fmaxf(hi_y, __shfl_xor_sync(0xffffffffu, hi_y, o));
        }
        if ((tid & 31) == 0) {
            float* w = s_warp + (tid >> 5) * 4;
            w[0] = lo_x; w[1] = hi_x; w[2] = lo_y; w[3] = hi_y;
        }
        // a NaN coordinate anywhere in the tile: no culling here (its pixel must see every gaussian)
        bad = __syncthreads_or(bad);
        bx0 = fminf(fminf(s_warp[0], s_warp[4]), fminf(s_warp[8], s_warp[12]));
        bx1 = fmaxf(fmaxf(s_warp[1], s_warp[5]), fmaxf(s_warp[9], s_warp[13]));
        by0 = fminf(fminf(s_warp[2], s_warp[6]), fminf(s_warp[10], s_warp[14]));
        by1 = fmaxf(fmaxf(s_warp[3], s_warp[7]), fmaxf(s_warp[11], s_warp[15]));
        __syncthreads();  // s_warp is reused for the per-stage counts
        cull = !bad;
    }

    // ---- gaussian range of this split, streamed in stages ----
    const int n_begin = split * a.per_split;
    const int n_end = min(a.N, n_begin + a.per_split);
    const int n_total = max(0, n_end - n_begin);
    const int n_chunks = (n_total + G - 1) / G;
    const float* src = a.frec + ((long long)b * a.N + n_begin) * RS;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
        *s_failed = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // Which stages to stream: all of them, or -- culling kernel, records in a spatial order --
    // only those whose bounding box meets this CTA's pixels, listed in ascending order (so
    // the sums run in the same sequence, minus terms that are exact zeros).
    int n_list = n_chunks;
    bool use_list = false;
    if constexpr (CULL) {
        if (a.cbox && cull && n_chunks <= Cfg::LIST_CAP) {
            use_list = true;
            const float4* boxes = reinterpret_cast<const float4*>(a.cbox) + ((long long)b * a.chunks_per_b + n_begin / G);
            int* s_count = reinterpret_cast<int*>(s_warp);
            int total = 0;
            for (int base0 = 0; base0 < n_chunks; base0 += T) {
                const int c = base0 + tid;
                bool keep = false;
                if (c < n_chunks) {
                    const float4 q = boxes[c];  // x0, x1, y0, y1
                    keep = !(q.y < bx0 || q.x > bx1 || q.w < by0 || q.z > by1);
                }
                const unsigned ballot = __ballot_sync(0xffffffffu, keep);
                if ((tid & 31) == 0) s_count[tid >> 5] = __popc(ballot);
                __syncthreads();
                int before = 0, n_keep = 0;
#pragma unroll
                for (int w = 0; w < T / 32; ++w) {
                    if (w < (tid >> 5)) before += s_count[w];
                    n_keep += s_count[w];
                }
                if (keep) s_stages[total + before + __popc(ballot & ((1u << (tid & 31)) - 1u))] = (unsigned short)c;
                total += n_keep;
                __syncthreads();
            }
            n_list = total;
        }
    }
    auto stage_chunk = [&](int k) { return (CULL && use_list) ? (int)s_stages[k] : k; };

    auto issue = [&](int k) {
        const int st = k % NS;
        const int chunk = stage_chunk(k);
        const int cnt = min(G, n_total - chunk * G);
        const uint32_t bytes = (uint32_t)cnt * RS * sizeof(float);
        mbar_expect_tx(&bars[st], bytes);
        bulk_g2s(stage_base + (size_t)st * G * RS, src + (long long)chunk * G * RS, bytes, &bars[st]);
    };
    if (tid == 0) {
        for (int c = 0; c < NS && c < n_list; ++c) issue(c);
    }

    int evaluated = 0;  // gaussians this CTA did not skip (counted by the culling kernel only)
    for (int k = 0; k < n_list; ++k) {
        const int st = k % NS;
        const uint32_t parity = (k / NS) & 1;
        if (!mbar_wait_bounded(&bars[st], parity)) *s_failed = 1;
        __syncthreads();
        if (*s_failed) {
            // give copies still in flight a bounded chance to land before the CTA
            // (and its shared memory) goes away, then report and leave
            if (tid == 0) {
                for (int c = k + 1; c < n_list && c < k + NS; ++c)
                    mbar_wait_bounded(&bars[c % NS], (c / NS) & 1);
                atomicOr(a.status, STATUS_WAIT_TIMEOUT);
            }
            return;
        }
        const int cnt = min(G, n_total - stage_chunk(k) * G);
        const float4* rec = reinterpret_cast<const float4*>(stage_base + (size_t)st * G * RS);
        auto splat = [&](int g) {
            const float4* rf = rec + (size_t)g * (RS / 4);
            float vals[RS];
#pragma unroll
            for (int q = 0; q < RS / 4; ++q) {
                const float4 t4 = rf[q];
                vals[4 * q] = t4.x; vals[4 * q + 1] = t4.y; vals[4 * q + 2] = t4.z; vals[4 * q + 3] = t4.w;
            }
            const f2 px2 = pk(vals[0], vals[0]), py2 = pk(vals[1], vals[1]);
            const f2 A2 = pk(vals[2], vals[2]), B22 = pk(vals[3], vals[3]);
            const f2 Cq2 = pk(vals[4], vals[4]), al2 = pk(vals[5], vals[5]);
            f2 col[CT + 1];
#pragma unroll
            for (int c = 0; c < CT; ++c) col[c] = pk(vals[6 + c], vals[6 + c]);
            if constexpr (SEP) {
                // per column pair: dx;  per row (both rows in one f32x2): B2*dy, Cq*dy^2;
                // per pixel pair the exponent is then two FMAs: dx * (A*dx + B2*dy) + Cq*dy^2
                const f2 dxc[2] = {sub2(xx[0], px2), sub2(xx[1], px2)};
                const f2 dyr = sub2(yy[0], py2);
                float b0, b1, c0, c1;
                upk(mul2(B22, dyr), b0, b1);
                upk(mul2(mul2(Cq2, dyr), dyr), c0, c1);
                const f2 bd[2] = {pk(b0, b0), pk(b1, b1)}, cd[2] = {pk(c0, c0), pk(c1, c1)};
#pragma unroll
                for (int j = 0; j < NP; ++j) {  // j = 2*row + column pair
                    const f2 e = ex2_2(fma2(dxc[j & 1], fma2(A2, dxc[j & 1], bd[j >> 1]), cd[j >> 1]));
                    S[j] = fma2(e, al2, S[j]);
#pragma unroll
                    for (int c = 0; c < CT; ++c) acc[j][c] = fma2(e, col[c], acc[j][c]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    const f2 dx = sub2(xx[j], px2);
                    const f2 dy = sub2(yy[j], py2);
                    const f2 t = fma2(A2, dx, mul2(B22, dy));
                    const f2 v = mul2(mul2(Cq2, dy), dy);
                    const f2 e = ex2_2(fma2(dx, t, v));
                    S[j] = fma2(e, al2, S[j]);
#pragma unroll
                    for (int c = 0; c < CT; ++c) acc[j][c] = fma2(e, col[c], acc[j][c]);
                }
            }
        };
        if (!CULL || !cull) {
            if constexpr (CULL) evaluated += cnt;
#pragma unroll(Cfg::UNROLL)
            for (int g = 0; g < cnt; ++g) splat(g);
        } else {
            // ordered list of the stage's gaussians whose box meets this CTA's box
            bool keep = false;
            if (tid < cnt) {
                const float* rt = reinterpret_cast<const float*>(rec) + (size_t)tid * RS;
                const float gx = rt[0], gy = rt[1], hx = rt[6 + CT], hy = rt[7 + CT];  // centre and reach
                keep = !(gx + hx < bx0 || gx - hx > bx1 || gy + hy < by0 || gy - hy > by1);
            }
            const unsigned ballot = __ballot_sync(0xffffffffu, keep);
            int* s_count = reinterpret_cast<int*>(s_warp);
            if ((tid & 31) == 0) s_count[tid >> 5] = __popc(ballot);
            __syncthreads();
            int base = 0, n_keep = 0;
#pragma unroll
            for (int w = 0; w < T / 32; ++w) {
                if (w < (tid >> 5)) base += s_count[w];
                n_keep += s_count[w];
            }
            if (keep) s_list[base + __popc(ballot & ((1u << (tid & 31)) - 1u))] = (unsigned short)tid;
            __syncthreads();
            evaluated += n_keep;
#pragma unroll(Cfg::UNROLL)
            for (int i = 0; i < n_keep; ++i) splat(s_list[i]);
        }
        __syncthreads();  // every lane is done with this stage
        if (tid == 0 && k + NS < n_list) issue(k + NS);
    }

    if constexpr (CULL) {
        // every thread of the CTA evaluated its pixels (padding included) against each kept gaussian
        if (tid == 0 && a.exec_count) atomicAdd(a.exec_count, (unsigned long long)evaluated * (T * 2 * NP));
    }

    // ---- epilogue ----
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        float s0, s1;
        upk(S[j], s0, s1);
        const float sv[2] = {s0, s1};
        float num[CT][2];
#pragma unroll
        for (int c = 0; c < CT; ++c) upk(acc[j][c], num[c][0], num[c][1]);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            long long p;
            if constexpr (SEP) {
                const int h = h0 + (j >> 1), w = w0 + (j & 1) * 2 + k;
                if (h >= a.H || w >= a.W) continue;
                p = (long long)h * a.W + w;
            } else {
                p = tile_base + (long long)(j * T + tid) * 2 + k;
                if (p >= HW) continue;
            }
            if (a.in_kernel_normalize) {
                const float den = sv[k] + a.eps;
#pragma unroll
                for (int c = 0; c < CT; ++c)
                    if (c < a.cr) a.out[((long long)b * a.C + a.c0 + c) * HW + p] = num[c][k] / den;
                if (a.write_s) a.wsum[(long long)b * HW + p] = sv[k];
            } else {
                float* dst = a.partial + ((long long)split * a.B + b) * (a.C + 1) * HW;
#pragma unroll
                for (int c = 0; c < CT; ++c)
                    if (c < a.cr) dst[(long long)(a.c0 + c) * HW + p] = num[c][k];
                if (a.write_s) dst[(long long)a.C * HW + p] = sv[k];
            }
        }
    }
}

// Adds the per-split partial sums in split order and either divides (normalize) or
// hands back the raw sums [B, C+1, HW].  V = pixels per thread: 4 (one 16-byte load or store
// per plane; the planes must be a multiple of four pixels and start on 16-byte boundaries) or 1.
template <int V>
__global__ void __launch_bounds__(256) reduce_normalize_kernel(ReduceArgs a) {
    const long long HW = a.HW;
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;  // over B*HW
    if (i >= (long long)a.B * HW) return;
    const long long b = i / HW, p = i - b * HW;
    const long long plane = (long long)(a.C + 1) * HW;
    const long long split_stride = (long long)a.B * plane;
    auto load = [&](const float* src, float (&v)[V]) {
        if constexpr (V == 4) {
            const float4 t = *reinterpret_cast<const float4*>(src);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
            v[0] = *src;
        }
    };
    auto store = [&](float* dst, const float (&v)[V]) {
        if constexpr (V == 4)
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        else
            *dst = v[0];
    };
    // one plane of this thread's pixels summed over the splits (the loads of four splits are in
    // flight together; the additions keep the split order)
    auto sum_plane = [&](int c, float (&acc)[V]) {
        const float* src = a.partial + b * plane + (long long)c * HW + p;
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = 0.f;
#pragma unroll 4
        for (int k = 0; k < a.n_split; ++k) {
            float t[V];
            load(src + (long long)k * split_stride, t);
#pragma unroll
            for (int q = 0; q < V; ++q) acc[q] += t[q];
        }
    };
    float s[V], den[V];
    sum_plane(a.C, s);
    store(a.normalize ? a.wsum + b * HW + p : a.out + b * plane + (long long)a.C * HW + p, s);
#pragma unroll
    for (int q = 0; q < V; ++q) den[q] = s[q] + a.eps;
    for (int c = 0; c < a.C; ++c) {
        float v[V];
        sum_plane(c, v);
        if (a.normalize) {
#pragma unroll
            for (int q = 0; q < V; ++q) v[q] = v[q] / den[q];
            store(a.out + (b * a.C + c) * HW + p, v);
        } else {
            store(a.out + b * plane + (long long)c * HW + p, v);
        }
    }
}

template <int CT, int PX_, bool SEP, bool CULL>
static cudaError_t launch_one(const FwdArgs& a, const FwdPlan& p, cudaStream_t s) {
    using Cfg = FwdCfg<CT, PX_>;
    constexpr size_t smem = CULL ? Cfg::SMEM_CULL : Cfg::SMEM;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(splat_forward_kernel<CT, PX_, SEP, CULL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    dim3 grid((unsigned)(SEP ? p.tiles_sep : p.tiles), (unsigned)p.n_split, (unsigned)a.B);
    {
        KernelTimer timer(K_FORWARD, s);
        splat_forward_kernel<CT, PX_, SEP, CULL><<<grid, Cfg::THREADS, smem, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

// 8 pixels per thread at every channel count (4 for the 8- and 16-channel instantiations
// needs fewer registers but measured 6 % slower at C = 16)
int forward_px_per_thread(int) { return 8; }

// every channel count has a separable instantiation
bool forward_has_separable(int) { return true; }

cudaError_t launch_forward_chunk(int ct, bool separable, bool culling, const FwdArgs& a, const FwdPlan& p,
                                 cudaStream_t s) {
    if (separable && culling) {
        switch (ct) {
            case 1: return launch_one<1, 8, true, true>(a, p, s);
            case 2: return launch_one<2, 8, true, true>(a, p, s);
            case 3: return launch_one<3, 8, true, true>(a, p, s);
            case 4: return launch_one<4, 8, true, true>(a, p, s);
            case 8: return launch_one<8, 8, true, true>(a, p, s);
            case 16: return launch_one<16, 8, true, true>(a, p, s);
        }
        return cudaErrorInvalidValue;
    }
    if (separable) {
        switch (ct) {
            case 1: return launch_one<1, 8, true, false>(a, p, s);
            case 2: return launch_one<2, 8, true, false>(a, p, s);
            case 3: return launch_one<3, 8, true, false>(a, p, s);
            case 4: return launch_one<4, 8, true, false>(a, p, s);
            case 8: return launch_one<8, 8, true, false>(a, p, s);
            case 16: return launch_one<16, 8, true, false>(a, p, s);
        }
        return cudaErrorInvalidValue;
    }
    switch (ct) {
        case 1: return launch_one<1, 8, false, false>(a, p, s);
        case 2: return launch_one<2, 8, false, false>(a, p, s);
        case 3: return launch_one<3, 8, false, false>(a, p, s);
        case 4: return launch_one<4, 8, false, false>(a, p, s);
        case 8: return launch_one<8, 8, false, false>(a, p, s);
        case 16: return launch_one<16, 8, false, false>(a, p, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_reduce_normalize(const ReduceArgs& a, cudaStream_t s) {
    const long long n = (long long)a.B * a.HW;
    if (n <= 0) return cudaSuccess;
    auto aligned16 = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = a.HW % 4 == 0 && aligned16(a.partial) && aligned16(a.out) && aligned16(a.wsum);
    {
        KernelTimer timer(K_REDUCE, s);
        if (vec)
            reduce_normalize_kernel<4><<<(unsigned)((n / 4 + 255) / 256), 256, 0, s>>>(a);
        else
            reduce_normalize_kernel<1><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

template <int CT, int PX_>
static int occ(int device) {
    using Cfg = FwdCfg<CT, PX_>;
    static int cached[64];
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    cudaFuncSetAttribute(splat_forward_kernel<CT, PX_, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Cfg::SMEM);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, splat_forward_kernel<CT, PX_, false, false>, Cfg::THREADS,
                                                      Cfg::SMEM) != cudaSuccess ||
        n <= 0) {
        cudaGetLastError();
        n = Cfg::MIN_CTAS;
    }
    if (device >= 0 && device < 64) cached[device] = n;
    return n;
}

int forward_ctas_per_sm(int ct, int device) {
    switch (ct) {
        case 1: return occ<1, 8>(device);
        case 2: return occ<2, 8>(device);
        case 3: return occ<3, 8>(device);
        case 4: return occ<4, 8>(device);
        case 8: return occ<8, 8>(device);
        default: return occ<16, 8>(device);
    }
}
int forward_threads(int) { return 128; }
int forward_chunk_g(int) { return 128; }
int forward_sep_tile_h() { return SEP_TILE_H; }
int forward_sep_tile_w() { return SEP_TILE_W; }

}  // namespace igs
