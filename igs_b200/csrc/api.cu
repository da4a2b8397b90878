// extern "C" entry points, launch plans and workspace carving.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "backward.cuh"
#include "forward.cuh"
#include "grid.cuh"
#include "loss.cuh"
#include "pack.cuh"
#include "plan.cuh"

namespace igs {

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// ---- optional per-kernel timing (igs_profile_*) ----
static std::atomic<int> g_profile_on{0};
static std::mutex g_profile_mu;
struct EventPair {
    int id, dev;
    cudaEvent_t start, stop;
};
static std::vector<EventPair> g_pending;
// events that have been read are kept, per device, for the next timed launches: creating a
// pair per launch costs the host more than the launch itself
static std::vector<cudaEvent_t> g_free_events[64];
static double g_total_ms[K_COUNT];
static long long g_timed_launches[K_COUNT];

static cudaEvent_t take_event(int dev) {
    {
        std::lock_guard<std::mutex> lock(g_profile_mu);
        if (dev >= 0 && dev < 64 && !g_free_events[dev].empty()) {
            cudaEvent_t e = g_free_events[dev].back();
            g_free_events[dev].pop_back();
            return e;
        }
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return e;
}

KernelTimer::KernelTimer(int id_, cudaStream_t s) : id(id_), stream(s) {
    const int mode = g_profile_on.load(std::memory_order_relaxed);
    if (!mode || (mode == 2 && id_ != K_FORWARD && id_ != K_BACKWARD)) return;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    start = take_event(dev);
    stop = take_event(dev);
    if (!start || !stop) {
        if (start) cudaEventDestroy(start);
        if (stop) cudaEventDestroy(stop);
        start = stop = nullptr;
        return;
    }
    cudaEventRecord(start, stream);
}
KernelTimer::~KernelTimer() {
    if (!start || !stop) return;
    cudaEventRecord(stop, stream);
    std::lock_guard<std::mutex> lock(g_profile_mu);
    g_pending.push_back({id, dev, start, stop});
}

// waits for every pending pair and folds it into the totals
static cudaError_t profile_drain() {
    std::lock_guard<std::mutex> lock(g_profile_mu);
    cudaError_t first = cudaSuccess;
    for (const EventPair& p : g_pending) {
        cudaError_t e = cudaEventSynchronize(p.stop);
        float ms = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, p.start, p.stop);
        if (e == cudaSuccess) {
            g_total_ms[p.id] += ms;
            g_timed_launches[p.id] += 1;
        } else if (first == cudaSuccess) {
            first = e;
        }
        if (p.dev >= 0 && p.dev < 64 && g_free_events[p.dev].size() < 4096) {
            g_free_events[p.dev].push_back(p.start);
            g_free_events[p.dev].push_back(p.stop);
        } else {
            cudaEventDestroy(p.start);
            cudaEventDestroy(p.stop);
        }
    }
    g_pending.clear();
    return first;
}

int sm_count(int device) {
    static int cached[64];
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 148;
    }
    if (device >= 0 && device < 64) cached[device] = n;
    return n;
}

int make_chunks(int C, Chunks* out) {
    if (C < 1 || C > 16 * MAX_CHUNKS) return IGS_ERR_LIMIT;
    out->n = 0;
    int c = 0;
    while (c < C) {
        const int cr = (C - c) >= 16 ? 16 : (C - c);
        const int k = out->n++;
        out->c0[k] = c;
        out->cr[k] = cr;
        out->ct[k] = chunk_template(cr);
        c += cr;
    }
    return IGS_OK;
}

// How the streamed axis (gaussians in the forward, pixels in the backward) is cut into parts,
// one CTA per (part, everything else).  The axis comes in indivisible units (stages of 128
// gaussians, row pairs, chunks of pixel pairs); a part is `per` consecutive units.  The model:
// CTAs run in waves of `slots`, every CTA of a wave takes per + overhead (its prologue and
// epilogue, in units), so the kernel takes waves * (per + overhead); the partition with the
// least modelled time wins, a deeper one only if it is at least half a percent better (more
// parts mean more partial sums to write and add up).  CTAs do not finish in lockstep, so with
// one or two waves the slowest SM sets the time (measured on B=1, N=16384, 512 x 512, backward:
// 2.47 / 2.45 / 2.29 / 2.24 / 2.23 ms at 1 / 2 / 3 / 4 / 8 waves): fewer than three waves are
// charged 8 % extra.
struct Parts {
    long long per;  // units per part
    int n;          // parts
};
static Parts pick_parts(long long base_ctas, long long slots, long long units, double overhead, int max_parts,
                        long long min_units) {
    if (units < 1) units = 1;
    if (base_ctas < 1) base_ctas = 1;
    Parts best{units, 1};
    double best_t = -1.0;
    for (long long want = 1; want <= max_parts && want <= units; ++want) {
        const long long per = (units + want - 1) / want;  // the shortest parts that give this count
        if (want > 1 && per < min_units) break;
        const long long n = (units + per - 1) / per;
        const long long waves = (base_ctas * n + slots - 1) / slots;
        const double t = (double)waves * ((double)per + overhead) * (waves < 3 ? 1.08 : 1.0);
        if (best_t < 0.0 || t < best_t * 0.995) {
            best_t = t;
            best = Parts{per, (int)n};
        }
    }
    return best;
}

int plan_forward(int B, int N, int H, int W, int C, int device, FwdPlan* p) {
    if (B < 0 || N < 0 || H < 0 || W < 0) return IGS_ERR_ARG;
    if (B > 65535) return IGS_ERR_LIMIT;
    int rc = make_chunks(C, &p->ch);
    if (rc) return rc;
    const long long HW = (long long)H * W;
    const int ct = p->ch.ct[0];
    p->threads = forward_threads(ct);
    p->px_per_thread = forward_px_per_thread(ct);
    p->tile_px = p->threads * p->px_per_thread;
    const long long tiles = (HW + p->tile_px - 1) / p->tile_px;
    if (tiles > 0x7fffffffLL) return IGS_ERR_LIMIT;
    p->tiles = (int)tiles;
    // separable tiling (16 x 64 pixel tiles); the split count chosen below serves both
    p->tiles_x = (W + forward_sep_tile_w() - 1) / forward_sep_tile_w();
    const long long tiles_sep = (long long)p->tiles_x * ((H + forward_sep_tile_h() - 1) / forward_sep_tile_h());
    p->tiles_sep = (forward_has_separable(ct) && tiles_sep <= 0x7fffffffLL) ? (int)tiles_sep : 0;
    p->chunk_g = forward_chunk_g(ct);
    p->stages = 2;
    const long long slots = (long long)sm_count(device) * forward_ctas_per_sm(ct, device);
    const long long base = tiles * (B > 0 ? B : 1);
    // splits are whole stages (every bulk copy is a whole number of records); a CTA's epilogue
    // (its partial sums) costs about a third of a stage
    const long long stages_n = ((long long)N + p->chunk_g - 1) / p->chunk_g;
    const Parts split = pick_parts(base, slots, stages_n, 0.3, 64, 2);
    p->per_split = (int)(split.per * p->chunk_g);
    p->n_split = split.n;

    size_t off = STATUS_BYTES;
    const long long M = (long long)B * N;
    for (int k = 0; k < p->ch.n; ++k) {
        p->off_frec[k] = off;
        off = align_up(off + (size_t)M * fwd_rec_floats(p->ch.ct[k]) * sizeof(float), 256);
    }
    p->off_partial = off;
    off = align_up(off + (size_t)p->n_split * B * (C + 1) * HW * sizeof(float), 256);
    p->off_cbox = off;
    off = align_up(off + (size_t)B * ((N + p->chunk_g - 1) / p->chunk_g) * 4 * sizeof(float), 256);
    p->bytes = off;
    return IGS_OK;
}

int plan_backward(int B, int N, int H, int W, int C, int device, BwdPlan* p, bool fine_slabs, bool separable_grid) {
    if (B < 0 || N < 0 || H < 0 || W < 0) return IGS_ERR_ARG;
    if (B > 65535) return IGS_ERR_LIMIT;
    int rc = make_chunks(C, &p->ch);
    if (rc) return rc;
    const long long HW = (long long)H * W;
    const int ct = p->ch.ct[0];
    p->threads = backward_threads(ct);
    p->gauss_per_thread = backward_gauss_per_thread(ct);
    p->chunk_pairs = backward_chunk_pairs(ct);
    p->stages = 2;
    p->npairs = (HW + 1) / 2;
    p->nrp = (H + 1) / 2;
    p->ncb = (W + 3) / 4;
    p->rows = H;
    p->cols = W;
    p->row_kernel = (p->ch.n == 1 && backward_has_row_kernel(ct)) ? 1 : 0;
    p->sep_ok = (p->ch.n == 1 && (backward_has_separable(ct) || p->row_kernel)) ? 1 : 0;
    const long long per_cta = (long long)p->threads * p->gauss_per_thread;
    const long long groups = ((long long)N + per_cta - 1) / per_cta;
    const long long base = groups * (B > 0 ? B : 1);
    // (every separable kernel gives a CTA 256 gaussians)
    const long long base_sep = (((long long)N + 255) / 256) * (B > 0 ? B : 1);
    // The slab count is chosen for the general kernel's occupancy; when the separable kernel
    // will run (it holds fewer CTAs per SM: more registers) and would get fewer than four
    // waves, a deeper count is taken.  The workspace covers both.
    // general kernel: units are stages of pixel pairs; separable kernels: row pairs.  A CTA's
    // prologue and epilogue cost about what ten 2 x 4-pixel blocks cost.
    const long long slots_gen = (long long)sm_count(device) * backward_ctas_per_sm(ct, device);
    const long long chunks_n = (p->npairs + p->chunk_pairs - 1) / p->chunk_pairs;
    const int ns_gen = pick_parts(base, slots_gen, chunks_n, 40.0 / p->chunk_pairs, 256, 2).n;
    int ns_sep = ns_gen;
    long long rp_sep = 0;  // row pairs per slab the separable kernel's own partition takes
    if (p->sep_ok) {
        const int per_sm = p->row_kernel ? backward_row_ctas_per_sm(ct, device) : backward_sep_ctas_per_sm(ct, device);
        if (per_sm > 0) {
            const Parts rows = pick_parts(base_sep, (long long)sm_count(device) * per_sm, p->nrp,
                                          10.0 / (p->ncb > 0 ? p->ncb : 1), 256, 1);
            ns_sep = rows.n;
            rp_sep = rows.per;
        }
    }
    const int ns = (separable_grid && p->sep_ok) ? ns_sep : ns_gen;
    // Fine partition: slabs of 8 row pairs, at most 96 of them, never fewer than the plain
    // partition has.  A function of the shape alone, like the plain one, so the result's bits
    // depend on whether an order was passed but not on the order or on the gaussians.
    // (Group, slab) pairs without work cost nothing -- the ordered path hands out tasks from a
    // list -- so short slabs only add partial sums to add up.  Measured, narrow gaussians at
    // 1024 x 1024, skipping kernel: N = 16384: 0.43 / 0.44 / 0.50 ms for 4 / 8 / 16 row pairs;
    // N = 65536: 0.47 / 0.48 / 0.51 ms, the step as a whole being fastest at 8.
    int ns_fine = ns;
    if (p->sep_ok) {
        const int rp_fine = 8;
        const int want = (p->nrp + rp_fine - 1) / rp_fine;
        ns_fine = want < 96 ? want : 96;
        // the partial sums grow with slabs x gaussians: keep them under half a gigabyte
        const long long per_slab_bytes = (long long)(B > 0 ? B : 1) * (N_MOMENTS * p->ch.n + C) * (long long)N * 4;
        const long long fit = per_slab_bytes > 0 ? (512LL << 20) / per_slab_bytes : ns_fine;
        if (fit < ns_fine) ns_fine = (int)(fit > 1 ? fit : 1);
        if (ns_fine < ns) ns_fine = ns;
    }
    auto slabs_for = [&](int parts, long long* per_out) {
        long long per = (p->npairs + parts - 1) / parts;
        per = (per + p->chunk_pairs - 1) / p->chunk_pairs * p->chunk_pairs;
        if (per <= 0) per = p->chunk_pairs;
        *per_out = per;
        const int n = (int)((p->npairs + per - 1) / per);
        return n < 1 ? 1 : n;
    };
    long long per_plain = 0, per_fine = 0;
    const int n_plain = slabs_for(ns, &per_plain);
    // the fine count is kept as asked (slabs past the image's end are empty and write zeros)
    slabs_for(ns_fine, &per_fine);
    const bool fine = fine_slabs && ns_fine > n_plain;
    p->pairs_per_slab = fine ? per_fine : per_plain;
    p->n_slab = fine ? ns_fine : n_plain;
    // the most slabs any of the partitions can have, whichever kernel the grid selects: the
    // workspace size must not depend on that choice
    int n_slab_max = ns_gen > ns_sep ? ns_gen : ns_sep;
    if (ns_fine > n_slab_max) n_slab_max = ns_fine;
    p->planes = N_MOMENTS * p->ch.n + C;
    // separable variant: same slab count, slabs are ranges of whole row pairs
    if (!fine && separable_grid && p->sep_ok && rp_sep > 0) {
        p->n_slab = ns_sep;
        p->rp_per_slab = (int)rp_sep;
    } else {
        p->rp_per_slab = (p->nrp + p->n_slab - 1) / p->n_slab;
    }
    if (p->rp_per_slab < 1) p->rp_per_slab = 1;

    size_t off = STATUS_BYTES;
    const long long M = (long long)B * N;
    p->off_geo = off;
    off = align_up(off + (size_t)M * GEO_FLOATS * sizeof(float), 256);
    for (int k = 0; k < p->ch.n; ++k) {
        p->off_prec[k] = off;
        size_t rec_bytes = (size_t)B * p->npairs * bwd_rec_floats(p->ch.ct[k]) * sizeof(float);
        if (p->sep_ok) {
            const size_t sep_bytes =
                p->row_kernel ? (size_t)B * HW * backward_row_record_floats(p->ch.ct[k]) * sizeof(float)
                              : (size_t)B * p->nrp * p->ncb * bwd_sep_rec_floats(p->ch.ct[k]) * sizeof(float);
            if (sep_bytes > rec_bytes) rec_bytes = sep_bytes;
        }
        off = align_up(off + rec_bytes, 256);
    }
    p->off_axes = off;
    if (p->row_kernel) off = align_up(off + (size_t)B * H * sizeof(float), 256);
    p->off_part = off;
    off = align_up(off + (size_t)n_slab_max * B * p->planes * (size_t)N * sizeof(float), 256);
    p->off_tasks = off;
    p->task_capacity = 0;
    p->off_slab_range = 0;
    if (p->sep_ok && !p->row_kernel) {  // (the task-queue kernel exists for up to 4 channels)
        const long long groups32 = ((long long)N + 31) / 32;
        const long long cap = (long long)B * groups32 * n_slab_max;
        if (cap <= 0x7fffffffLL / 2) {
            p->task_capacity = (int)cap;
            off = align_up(off + (size_t)cap * sizeof(int4), 256);
            off = align_up(off + (size_t)B * groups32 * sizeof(int4), 256);
            p->off_slab_range = off;  // [B, N] int: the slabs that hold sums of a slot
            off = align_up(off + (size_t)B * N * sizeof(int), 256);
        }
    }
    p->bytes = off;
    return IGS_OK;
}

static int check_device(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return IGS_ERR_DEVICE;
    }
    return IGS_OK;
}

struct Strides {
    long long b, h, w;
};
static Strides get_strides(const int64_t* s, int H, int W) {
    if (!s) return {(long long)H * W, (long long)W, 1};
    return {(long long)s[0], (long long)s[1], (long long)s[2]};
}

// ---- lossless culling switch (igs_set_culling) ----
static std::atomic<int> g_culling{1};

// Classifies the sample grid (GridKind); launches the separability check when the strides do
// not settle the question.  The caller has cleared the status area (grid word included).
static cudaError_t prepare_grid(unsigned char* ws, const float* x, const float* y, const Strides& sx, const Strides& sy,
                                int B, int H, int W, bool separable_available, int hints, GridKind* kind,
                                cudaStream_t st) {
    int* flag = reinterpret_cast<int*>(ws) + GRID_FLAG_WORD;
    *kind = classify_grid(sx.h, sy.w, H, W, separable_available && !(hints & IGS_HINT_GENERAL_GRID));
    if (*kind != GRID_CHECK_ON_DEVICE) return cudaSuccess;
    GridCheckArgs ga;
    ga.x = x; ga.y = y;
    ga.xs_b = sx.b; ga.xs_h = sx.h; ga.xs_w = sx.w;
    ga.ys_b = sy.b; ga.ys_h = sy.h; ga.ys_w = sy.w;
    ga.flag = flag;
    ga.B = B; ga.H = H; ga.W = W;
    return launch_grid_check(ga, st);
}

// The part of the prologue's arguments that describes the sample grid (for the reach
// statistics and the axis-monotonicity bit the culling code relies on).
static void pack_grid_args(PackArgs* pa, unsigned char* ws, const float* x, const float* y, const Strides& sx,
                           const Strides& sy, int B, int N, int H, int W) {
    pa->x = x; pa->y = y;
    pa->xs_b = sx.b; pa->xs_w = sx.w;
    pa->ys_b = sy.b; pa->ys_h = sy.h;
    pa->narrow_count = reinterpret_cast<int*>(ws) + NARROW_COUNT_WORD;
    pa->grid_flag = reinterpret_cast<int*>(ws) + GRID_FLAG_WORD;
    pa->B = B; pa->N = N; pa->H = H; pa->W = W;
}

static ParamLayout layout_or_default(const ParamLayout* layout, int kind, int C) {
    if (layout) return *layout;
    ParamLayout l;
    std::memset(&l, 0, sizeof(l));
    l.pos_s = 2;
    l.s0_s = kind == SHAPE_SCALE_ROT ? 2 : 1;
    l.s1_s = 1;
    l.col_s = C;
    return l;
}

// One-split override for ordered calls.  A caller that passes an order expects narrow
// gaussians: a CTA then streams a few stages only, and splitting the gaussians over several
// CTAs per tile would just add partial sums to write and add up.  (A function of the shape and
// of whether an order was passed, like every other choice that affects the bits of the result.)
static void single_split_for_ordered_calls(FwdPlan* p, int B, int N, const int* order, bool culling_on, int device) {
    if (order && culling_on && p->tiles_sep > 0 && (long long)p->tiles_sep * B >= sm_count(device) &&
        (N + p->chunk_g - 1) / p->chunk_g <= 8192 /* what a CTA can list */) {
        p->n_split = 1;
        p->per_split = (N + p->chunk_g - 1) / p->chunk_g * p->chunk_g;
    }
}

int forward_impl(int kind, const float* pos, const float* s0, const float* s1, const float* s2, const float* alpha,
                 const float* colors, const float* x, const int64_t* xs, const float* y, const int64_t* ys, int B, int N,
                 int H, int W, int C, float eps, int normalize, float* out, float* wsum, void* workspace,
                 size_t workspace_bytes, int device, void* stream, const FwdPlan* use_plan, const ParamLayout* layout,
                 const int* order, int hints, const FwdExtras* extras) {
    if (B < 0 || N < 0 || H < 0 || W < 0 || C < 1) return IGS_ERR_ARG;
    if (hints & ~(IGS_HINT_WIDE_GAUSSIANS | IGS_HINT_GENERAL_GRID)) return IGS_ERR_ARG;
    if (!out || (normalize && !wsum)) return IGS_ERR_ARG;
    const long long HW = (long long)H * W;
    if (B == 0 || HW == 0) return IGS_OK;
    if (!x || !y) return IGS_ERR_ARG;
    // (only a caller-described layout may leave the opacities out: all ones)
    if (N > 0 && (!pos || !s0 || !s1 || (!alpha && !layout) || !colors || (kind == SHAPE_COV_INV && !s2)))
        return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    if (N == 0) {
        // no gaussians: every sum is zero (the reference's loop body never runs)
        cudaError_t e;
        if (normalize) {
            e = cudaMemsetAsync(out, 0, (size_t)B * C * HW * sizeof(float), st);
            if (e == cudaSuccess) e = cudaMemsetAsync(wsum, 0, (size_t)B * HW * sizeof(float), st);
        } else {
            e = cudaMemsetAsync(out, 0, (size_t)B * (C + 1) * HW * sizeof(float), st);
        }
        return (int)e;
    }

    FwdPlan p;
    if (use_plan) {
        p = *use_plan;
    } else {
        rc = plan_forward(B, N, H, W, C, device, &p);
        if (rc) return rc;
    }
    if (!workspace || workspace_bytes < p.bytes) return IGS_ERR_WORKSPACE;
    const bool culling_on = g_culling.load(std::memory_order_relaxed) && !(hints & IGS_HINT_WIDE_GAUSSIANS);
    if (!use_plan) single_split_for_ordered_calls(&p, B, N, order, culling_on, device);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    cudaError_t e = cudaMemsetAsync(ws, 0, 8 * sizeof(int), st);  // status word, flags, counters
    if (e != cudaSuccess) return (int)e;

    const Strides sx = get_strides(xs, H, W), sy = get_strides(ys, H, W);
    // separable grid (x by column, y by row)?  known from the strides, or checked on the device
    int* grid_flag = reinterpret_cast<int*>(ws) + GRID_FLAG_WORD;
    GridKind grid_kind;
    e = prepare_grid(ws, x, y, sx, sy, B, H, W, p.tiles_sep > 0, hints, &grid_kind, st);
    if (e != cudaSuccess) return (int)e;

    PackArgs pa;
    std::memset(&pa, 0, sizeof(pa));
    pa.pos = pos;
    pa.shape0 = s0;
    pa.shape1 = s1;
    pa.shape2 = s2;
    pa.alpha = alpha;
    pa.colors = colors;
    pa.geo = extras ? extras->geo_out : nullptr;  // (a fused forward + backward packs once for both)
    pa.lay = layout_or_default(layout, kind, C);
    pack_grid_args(&pa, ws, x, y, sx, sy, B, N, H, W);
    for (int k = 0; k < p.ch.n; ++k) pa.frec[k] = reinterpret_cast<float*>(ws + p.off_frec[k]);
    pa.ch = p.ch;
    pa.M = (long long)B * N;
    pa.C = C;
    pa.eps = eps;
    pa.kind = kind;
    // A caller's order: the records are written in that order, and the box around each
    // stage's gaussians lets the culling kernel pass over whole stages.
    const bool listed = order != nullptr && p.bytes > p.off_cbox && culling_on && p.per_split / p.chunk_g >= 8;
    pa.order = order;
    pa.chunk_g = p.chunk_g;
    pa.cbox = listed ? reinterpret_cast<float*>(ws + p.off_cbox) : nullptr;
    e = launch_pack(pa, st);
    if (e != cudaSuccess) return (int)e;
    e = launch_stage_boxes(pa, st);
    if (e != cudaSuccess) return (int)e;

    const bool in_kernel = normalize && p.n_split == 1;
    for (int k = 0; k < p.ch.n; ++k) {
        FwdArgs fa;
        std::memset(&fa, 0, sizeof(fa));
        fa.frec = pa.frec[k];
        fa.x = x;
        fa.y = y;
        fa.xs_b = sx.b; fa.xs_h = sx.h; fa.xs_w = sx.w;
        fa.ys_b = sy.b; fa.ys_h = sy.h; fa.ys_w = sy.w;
        fa.out = out;
        fa.wsum = wsum;
        // single split without normalisation: the "partial" array IS the caller's sums buffer
        // (unless the caller wants the per-split sums left where they are)
        const bool leave = extras && extras->leave_partials;
        fa.partial = (!normalize && p.n_split == 1 && !leave) ? out : reinterpret_cast<float*>(ws + p.off_partial);
        fa.status = reinterpret_cast<int*>(ws);
        fa.B = B; fa.N = N; fa.H = H; fa.W = W; fa.C = C;
        fa.c0 = p.ch.c0[k];
        fa.cr = p.ch.cr[k];
        fa.per_split = p.per_split;
        fa.in_kernel_normalize = in_kernel ? 1 : 0;
        fa.write_s = (k == 0) ? 1 : 0;
        fa.eps = eps;
        fa.tiles_x = p.tiles_x;
        const GridKind gk = forward_has_separable(p.ch.ct[k]) ? grid_kind : GRID_GENERAL;
        fa.grid_sel = (grid_kind == GRID_CHECK_ON_DEVICE) ? grid_flag : nullptr;
        if (gk != GRID_GENERAL) {
            // the separable kernel comes as a plain and a culling instantiation; both are
            // launched and the count of narrow gaussians picks one (the other returns at once)
            fa.cull_sel = culling_on ? pa.narrow_count : nullptr;
            fa.exec_count = reinterpret_cast<unsigned long long*>(ws) + EXEC_COUNT_WORD / 2;
            fa.cbox = pa.cbox;
            fa.chunks_per_b = (N + p.chunk_g - 1) / p.chunk_g;
            e = launch_forward_chunk(p.ch.ct[k], true, false, fa, p, st);
            if (e != cudaSuccess) return (int)e;
            if (fa.cull_sel) {
                e = launch_forward_chunk(p.ch.ct[k], true, true, fa, p, st);
                if (e != cudaSuccess) return (int)e;
            }
        }
        if (gk != GRID_SEPARABLE) {
            // a chunk without a separable instantiation runs whatever the flag says
            if (gk == GRID_GENERAL) fa.grid_sel = nullptr;
            fa.cull_sel = nullptr;
            e = launch_forward_chunk(p.ch.ct[k], false, false, fa, p, st);
            if (e != cudaSuccess) return (int)e;
        }
    }
    if (extras && extras->leave_partials) return IGS_OK;  // the caller adds the splits up itself
    if (p.n_split > 1) {
        ReduceArgs ra;
        ra.partial = reinterpret_cast<const float*>(ws + p.off_partial);
        ra.out = out;
        ra.wsum = wsum;
        ra.HW = HW;
        ra.B = B; ra.C = C; ra.n_split = p.n_split; ra.normalize = normalize ? 1 : 0;
        ra.eps = eps;
        e = launch_reduce_normalize(ra, st);
        if (e != cudaSuccess) return (int)e;
    }
    return IGS_OK;
}

static int backward_impl(int kind, const float* pos, const float* s0, const float* s1, const float* s2,
                         const float* alpha, const float* colors, const float* x, const int64_t* xs, const float* y,
                         const int64_t* ys, const float* wsum, const float* out, const float* gout, int B, int N,
                         int H, int W, int C, float eps, int mode, float* d_pos, float* d_s0, float* d_s1,
                         float* d_s2, float* d_alpha, float* d_colors, float* d_x, float* d_y, const int* order,
                         int hints, void* workspace, size_t workspace_bytes, int device, void* stream,
                         const ParamLayout* layout = nullptr, const BwdPrepared* prepared = nullptr) {
    if (B < 0 || N < 0 || H < 0 || W < 0 || C < 1) return IGS_ERR_ARG;
    if (mode != IGS_GRAD_REFERENCE && mode != IGS_GRAD_EXACT) return IGS_ERR_ARG;
    if (hints & ~(IGS_HINT_WIDE_GAUSSIANS | IGS_HINT_GENERAL_GRID)) return IGS_ERR_ARG;
    if (layout && (d_x || d_y)) return IGS_ERR_ARG;  // coordinate gradients: separate tensors only
    if ((d_x == nullptr) != (d_y == nullptr)) return IGS_ERR_ARG;
    const long long HW = (long long)H * W;
    if (B == 0) return IGS_OK;
    if (HW > 0 && !prepared && (!x || !y || !wsum || !gout || (mode == IGS_GRAD_EXACT && !out))) return IGS_ERR_ARG;
    if (N > 0 && (!pos || !s0 || !s1 || !colors || !d_pos || !d_s0 || !d_s1 || !d_colors ||
                  (!layout && (!alpha || !d_alpha)) || (kind == SHAPE_COV_INV && (!s2 || !d_s2))))
        return IGS_ERR_ARG;
    if (layout && (N == 0 || HW == 0)) return IGS_ERR_ARG;  // the feature-level wrapper handles these itself
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;

    if (N == 0 || HW == 0) {
        // nothing to sum over: every gradient is zero
        const size_t M = (size_t)B * N;
        e = cudaSuccess;
        if (M) {
            e = cudaMemsetAsync(d_pos, 0, M * 2 * sizeof(float), st);
            if (e == cudaSuccess) e = cudaMemsetAsync(d_s0, 0, M * (kind == SHAPE_SCALE_ROT ? 2 : 1) * sizeof(float), st);
            if (e == cudaSuccess) e = cudaMemsetAsync(d_s1, 0, M * sizeof(float), st);
            if (e == cudaSuccess && kind == SHAPE_COV_INV) e = cudaMemsetAsync(d_s2, 0, M * sizeof(float), st);
            if (e == cudaSuccess) e = cudaMemsetAsync(d_alpha, 0, M * sizeof(float), st);
            if (e == cudaSuccess) e = cudaMemsetAsync(d_colors, 0, M * C * sizeof(float), st);
        }
        if (e == cudaSuccess && d_x && HW) {
            e = cudaMemsetAsync(d_x, 0, (size_t)B * HW * sizeof(float), st);
            if (e == cudaSuccess) e = cudaMemsetAsync(d_y, 0, (size_t)B * HW * sizeof(float), st);
        }
        return (int)e;
    }

    // which kernel family will (probably) run is known from the strides, or assumed separable
    // when the data has to be checked on the device (a materialised xy_grid)
    const Strides sx = get_strides(xs, H, W), sy = get_strides(ys, H, W);
    // (not a matter of the hints: the partition, and with it the bits of the result, must be the same with and without them)
    const bool likely_separable = classify_grid(sx.h, sy.w, H, W, true) != GRID_GENERAL;
    BwdPlan p;
    rc = plan_backward(B, N, H, W, C, device, &p, order != nullptr, likely_separable);
    if (rc) return rc;
    if (!workspace || workspace_bytes < p.bytes) return IGS_ERR_WORKSPACE;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    // Prepared mode (the fused render + loss + gradient entry): a forward on the same data has
    // just filled a status area (narrow count, axis flags), packed the geometry records into
    // this workspace and written the pixel records; the grid is separable by its strides.
    // Nothing of that is redone: straight to the splat kernels.
    unsigned char* sa = prepared ? prepared->status : ws;  // status area
    if (!prepared) {
        e = cudaMemsetAsync(ws, 0, 8 * sizeof(int), st);  // status word, flags, counters
        if (e != cudaSuccess) return (int)e;
    }

    // separable grid?  (same decision procedure as the forward)
    int* grid_flag = reinterpret_cast<int*>(sa) + GRID_FLAG_WORD;
    GridKind grid_kind = GRID_SEPARABLE;
    if (!prepared) {
        e = prepare_grid(ws, x, y, sx, sy, B, H, W, p.sep_ok != 0, hints, &grid_kind, st);
        if (e != cudaSuccess) return (int)e;
    }

    PackArgs pa;
    std::memset(&pa, 0, sizeof(pa));
    pa.pos = pos;
    pa.shape0 = s0;
    pa.shape1 = s1;
    pa.shape2 = s2;
    pa.alpha = alpha;
    pa.colors = colors;
    pa.geo = reinterpret_cast<float*>(ws + p.off_geo);
    pa.lay = layout_or_default(layout, kind, C);
    pack_grid_args(&pa, sa, x, y, sx, sy, B, N, H, W);
    pa.ch = p.ch;
    pa.M = (long long)B * N;
    pa.C = C;
    pa.eps = eps;
    pa.kind = kind;
    if (!prepared) {
        e = launch_pack(pa, st);
        if (e != cudaSuccess) return (int)e;
    }

    PixelTermArgs ta;
    std::memset(&ta, 0, sizeof(ta));
    ta.x = x;
    ta.y = y;
    ta.xs_b = sx.b; ta.xs_h = sx.h; ta.xs_w = sx.w;
    ta.ys_b = sy.b; ta.ys_h = sy.h; ta.ys_w = sy.w;
    ta.wsum = wsum;
    ta.out = out;
    ta.gout = gout;
    for (int k = 0; k < p.ch.n; ++k) ta.prec[k] = reinterpret_cast<float*>(ws + p.off_prec[k]);
    ta.ch = p.ch;
    ta.npairs = p.npairs;
    ta.nrp = p.nrp;
    ta.ncb = p.ncb;
    ta.axes = p.row_kernel ? reinterpret_cast<float*>(ws + p.off_axes) : nullptr;
    ta.grid_sel = (grid_kind == GRID_CHECK_ON_DEVICE) ? grid_flag : nullptr;
    ta.flags = grid_flag;
    ta.B = B; ta.H = H; ta.W = W; ta.C = C;
    ta.mode = mode;
    ta.eps = eps;
    if (grid_kind != GRID_GENERAL && !prepared) {
        e = launch_pixel_terms(ta, true, st);
        if (e != cudaSuccess) return (int)e;
    }
    if (grid_kind != GRID_SEPARABLE) {
        e = launch_pixel_terms(ta, false, st);
        if (e != cudaSuccess) return (int)e;
    }

    const int* slab_range = nullptr;  // set by the ordered skipping path
    for (int k = 0; k < p.ch.n; ++k) {
        BwdArgs ba;
        std::memset(&ba, 0, sizeof(ba));
        ba.geo = pa.geo;
        ba.colors = colors;
        ba.prec = ta.prec[k];
        ba.order = order;
        ba.axes = ta.axes;
        ba.part = reinterpret_cast<float*>(ws + p.off_part);
        ba.status = reinterpret_cast<int*>(sa);
        ba.npairs = p.npairs;
        ba.nrp = p.nrp;
        ba.ncb = p.ncb;
        ba.rp_per_slab = p.rp_per_slab;
        ba.grid_sel = (grid_kind == GRID_CHECK_ON_DEVICE) ? grid_flag : nullptr;
        ba.grid_word = grid_flag;
        ba.cull_sel = (g_culling.load(std::memory_order_relaxed) && !(hints & IGS_HINT_WIDE_GAUSSIANS)) ? pa.narrow_count : nullptr;
        ba.exec_count = reinterpret_cast<unsigned long long*>(sa) + EXEC_COUNT_WORD / 2;
        ba.pairs_per_slab = p.pairs_per_slab;
        ba.B = B; ba.N = N;
        ba.C = pa.lay.col_s;  // the kernels use it as the colours' row stride only
        ba.c0 = p.ch.c0[k];
        ba.cr = p.ch.cr[k];
        ba.planes = p.planes;
        ba.n_slab = p.n_slab;
        ba.moment_plane0 = N_MOMENTS * k;
        ba.color_plane0 = N_MOMENTS * p.ch.n;
        if (grid_kind != GRID_GENERAL) {
            const bool queued = order && p.task_capacity > 0 && ba.cull_sel;
            if (queued) {
                // The ordered skipping path writes partial sums only for the (group, slab) pairs
                // that have a task and leaves, per gaussian, the range of slabs to add up
                // (all of them when the device selects another kernel).
                ba.slab_range = reinterpret_cast<int*>(ws + p.off_slab_range);
                slab_range = ba.slab_range;
            }
            e = launch_backward_chunk(p.ch.ct[k], true, false, ba, p, st);
            if (e != cudaSuccess) return (int)e;
            if (ba.cull_sel) {
                // the skipping kernel: with a processing order, the one whose warps each follow
                // their own gaussians' reach; without, the one that skips per CTA
                if (queued) {
                    ba.tasks = reinterpret_cast<int4*>(ws + p.off_tasks);
                    ba.group_rect = reinterpret_cast<int4*>(
                        ws + align_up(p.off_tasks + (size_t)p.task_capacity * sizeof(int4), 256));
                    ba.task_count = reinterpret_cast<int*>(sa) + TASK_COUNT_WORD;
                    ba.task_next = reinterpret_cast<int*>(sa) + TASK_NEXT_WORD;
                    ba.task_capacity = p.task_capacity;
                    e = launch_backward_warp_chunk(p.ch.ct[k], ba, p, sm_count(device), st);
                } else {
                    e = launch_backward_chunk(p.ch.ct[k], true, true, ba, p, st);
                }
                if (e != cudaSuccess) return (int)e;
            }
        }
        if (grid_kind != GRID_SEPARABLE) {
            e = launch_backward_chunk(p.ch.ct[k], false, false, ba, p, st);
            if (e != cudaSuccess) return (int)e;
        }
    }

    FinalizeArgs fa;
    std::memset(&fa, 0, sizeof(fa));
    fa.part = reinterpret_cast<const float*>(ws + p.off_part);
    fa.slab_range = slab_range;
    fa.order = order;
    fa.pos = pos;
    fa.shape0 = s0;
    fa.shape1 = s1;
    fa.shape2 = s2;
    fa.alpha = alpha;
    fa.d_pos = d_pos;
    fa.d_shape0 = d_s0;
    fa.d_shape1 = d_s1;
    fa.d_shape2 = d_s2;
    fa.d_alpha = d_alpha;
    fa.d_colors = d_colors;
    fa.lay = pa.lay;
    fa.B = B; fa.N = N; fa.C = C;
    fa.n_slab = p.n_slab;
    fa.planes = p.planes;
    fa.n_chunks = p.ch.n;
    fa.kind = kind;
    fa.eps = eps;
    e = launch_finalize(fa, st);
    if (e != cudaSuccess) return (int)e;

    if (d_x) {
        CoordGradArgs ca;
        std::memset(&ca, 0, sizeof(ca));
        ca.geo = pa.geo;
        ca.colors = colors;
        ca.x = x;
        ca.y = y;
        ca.xs_b = sx.b; ca.xs_h = sx.h; ca.xs_w = sx.w;
        ca.ys_b = sy.b; ca.ys_h = sy.h; ca.ys_w = sy.w;
        ca.wsum = wsum;
        ca.out = out;
        ca.gout = gout;
        ca.d_x = d_x;
        ca.d_y = d_y;
        ca.B = B; ca.N = N; ca.H = H; ca.W = W; ca.C = C;
        ca.mode = mode;
        ca.eps = eps;
        e = launch_coord_grad(ca, st);
        if (e != cudaSuccess) return (int)e;
    }
    return IGS_OK;
}

// normalisation split off for the gaussian-sharded multi-GPU path: same kernel as the
// split reduction, with the all-reduced sums as a single "split"
static int normalize_impl(const float* sums, int B, int H, int W, int C, float eps, float* out, float* wsum,
                          int device, void* stream) {
    if (B < 0 || H < 0 || W < 0 || C < 1) return IGS_ERR_ARG;
    const long long HW = (long long)H * W;
    if (B == 0 || HW == 0) return IGS_OK;
    if (!sums || !out || !wsum) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    ReduceArgs ra;
    ra.partial = sums;
    ra.out = out;
    ra.wsum = wsum;
    ra.HW = HW;
    ra.B = B; ra.C = C; ra.n_split = 1; ra.normalize = 1;
    ra.eps = eps;
    return (int)launch_reduce_normalize(ra, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// render + mean-squared-error loss + gradients in one call (igs_render_mse_sr)
// ---------------------------------------------------------------------------
struct RenderMsePlan {
    FwdPlan fp;
    BwdPlan bp;
    bool fused;          // separable grid by its strides, one channel chunk, a separable backward for it
    size_t off_bwd;      // the backward's workspace
    size_t off_loss;     // block partial sums of the loss
    size_t off_image;    // unfused path: image [B,C,HW] + weight sums [B,HW]
    size_t off_gout;     // unfused path: upstream gradient [B,C,HW]
    size_t bytes;
};

static int plan_render_mse(int B, int N, int H, int W, int C, int device, bool separable_by_strides, bool ordered,
                           bool culling_on, const int* order, RenderMsePlan* p) {
    int rc = plan_forward(B, N, H, W, C, device, &p->fp);
    if (rc) return rc;
    rc = plan_backward(B, N, H, W, C, device, &p->bp, ordered, separable_by_strides);
    if (rc) return rc;
    p->fused = separable_by_strides && p->bp.sep_ok && !p->bp.row_kernel && p->fp.tiles_sep > 0;
    if (p->fused) single_split_for_ordered_calls(&p->fp, B, N, order, culling_on, device);
    const long long HW = (long long)H * W;
    size_t off = align_up(p->fp.bytes, 256);
    p->off_bwd = off;
    off = align_up(off + p->bp.bytes, 256);
    p->off_loss = off;
    long long lb = loss_terms_blocks(B, p->bp.nrp, p->bp.ncb);
    if (lb < 1024) lb = 1024;  // (the unfused path's loss kernel uses up to 1024 blocks)
    off = align_up(off + (size_t)lb * sizeof(float), 256);
    p->off_image = off;
    off = align_up(off + (size_t)B * (C + 1) * HW * sizeof(float), 256);
    p->off_gout = off;
    off = align_up(off + (size_t)B * C * HW * sizeof(float), 256);
    p->bytes = off;
    return IGS_OK;
}

static int render_mse_impl(const float* pos, const float* scales, const float* rot, const float* alpha,
                           const float* colors, int log_scales, const float* x, const int64_t* xs, const float* y,
                           const int64_t* ys, const float* target, int B, int N, int H, int W, int C, float eps,
                           int mode, const float* upstream, float* loss, float* out, float* d_pos, float* d_scales,
                           float* d_rot, float* d_alpha, float* d_colors, const int* order, int hints, void* workspace,
                           size_t workspace_bytes, int device, void* stream) {
    if (B < 1 || N < 1 || H < 1 || W < 1 || C < 1) return IGS_ERR_ARG;
    if (mode != IGS_GRAD_REFERENCE && mode != IGS_GRAD_EXACT) return IGS_ERR_ARG;
    if (hints & ~(IGS_HINT_WIDE_GAUSSIANS | IGS_HINT_GENERAL_GRID)) return IGS_ERR_ARG;
    if (!pos || !scales || !rot || !colors || !x || !y || !target || !loss || !d_pos || !d_scales || !d_rot || !d_colors)
        return IGS_ERR_ARG;
    if ((alpha == nullptr) != (d_alpha == nullptr)) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long HW = (long long)H * W;
    const Strides sx = get_strides(xs, H, W), sy = get_strides(ys, H, W);
    const bool culling_on = g_culling.load(std::memory_order_relaxed) && !(hints & IGS_HINT_WIDE_GAUSSIANS);
    const bool by_strides =
        !(hints & IGS_HINT_GENERAL_GRID) && classify_grid(sx.h, sy.w, H, W, true) == GRID_SEPARABLE;
    RenderMsePlan p;
    rc = plan_render_mse(B, N, H, W, C, device, by_strides, order != nullptr, culling_on, order, &p);
    if (rc) return rc;
    if (!workspace || workspace_bytes < p.bytes) return IGS_ERR_WORKSPACE;
    unsigned char* ws = static_cast<unsigned char*>(workspace);

    // the parameter tensors as the caller holds them: separate arrays, scales possibly as logs,
    // opacities possibly absent (all ones)
    ParamLayout lay;
    std::memset(&lay, 0, sizeof(lay));
    lay.pos_s = 2;
    lay.s0_s = 2;
    lay.s1_s = 1;
    lay.col_s = C;
    lay.log_scale = log_scales ? 1 : 0;

    if (p.fused) {
        // forward: un-normalised sums per gaussian split, left in the forward's workspace; its
        // prologue also packs the backward's geometry records
        FwdExtras ex;
        ex.geo_out = reinterpret_cast<float*>(ws + p.off_bwd + p.bp.off_geo);
        ex.leave_partials = 1;
        float* partial = reinterpret_cast<float*>(ws + p.fp.off_partial);
        rc = forward_impl(SHAPE_SCALE_ROT, pos, scales, rot, nullptr, alpha, colors, x, xs, y, ys, B, N, H, W, C, eps, 0,
                          partial, nullptr, ws, p.fp.bytes, device, stream, &p.fp, &lay, order, hints, &ex);
        if (rc) return rc;
        LossTermArgs la;
        std::memset(&la, 0, sizeof(la));
        la.partial = partial;
        la.target = target;
        la.x = x;
        la.y = y;
        la.xs_b = sx.b; la.xs_w = sx.w; la.ys_b = sy.b; la.ys_h = sy.h;
        la.upstream = upstream;
        la.out = out;
        la.wsum = nullptr;
        la.prec = reinterpret_cast<float*>(ws + p.off_bwd + p.bp.off_prec[0]);
        la.loss_partial = reinterpret_cast<float*>(ws + p.off_loss);
        la.flags = reinterpret_cast<int*>(ws) + GRID_FLAG_WORD;
        la.n_total = (long long)B * C * HW;
        la.n_split = p.fp.n_split;
        la.B = B; la.H = H; la.W = W; la.C = C;
        la.nrp = p.bp.nrp; la.ncb = p.bp.ncb; la.ct = p.bp.ch.ct[0];
        la.mode = mode;
        la.eps = eps;
        cudaError_t e = launch_loss_terms_sep(la, loss, st);
        if (e != cudaSuccess) return (int)e;
        BwdPrepared prep;
        prep.status = ws;
        return backward_impl(SHAPE_SCALE_ROT, pos, scales, rot, nullptr, alpha, colors, x, xs, y, ys, nullptr, nullptr,
                             nullptr, B, N, H, W, C, eps, mode, d_pos, d_scales, d_rot, nullptr, d_alpha, d_colors,
                             nullptr, nullptr, order, hints, ws + p.off_bwd, p.bp.bytes, device, stream, &lay, &prep);
    }

    // any other grid or channel count: the same steps one after the other
    float* image = out ? out : reinterpret_cast<float*>(ws + p.off_image);
    float* wsum = reinterpret_cast<float*>(ws + p.off_image) + (size_t)B * C * HW;
    float* gout = reinterpret_cast<float*>(ws + p.off_gout);
    rc = forward_impl(SHAPE_SCALE_ROT, pos, scales, rot, nullptr, alpha, colors, x, xs, y, ys, B, N, H, W, C, eps, 1, image,
                      wsum, ws, p.fp.bytes, device, stream, nullptr, &lay, order, hints, nullptr);
    if (rc) return rc;
    const long long n = (long long)B * C * HW;
    rc = igs_mse_loss(image, target, n, loss, ws + p.off_loss, IGS_MSE_WORKSPACE_BYTES, device, stream);
    if (rc) return rc;
    rc = igs_mse_grad(image, target, n, upstream, gout, device, stream);
    if (rc) return rc;
    return backward_impl(SHAPE_SCALE_ROT, pos, scales, rot, nullptr, alpha, colors, x, xs, y, ys, wsum, image, gout, B, N,
                         H, W, C, eps, mode, d_pos, d_scales, d_rot, nullptr, d_alpha, d_colors, nullptr, nullptr, order,
                         hints, ws + p.off_bwd, p.bp.bytes, device, stream, &lay, nullptr);
}

}  // namespace igs

using namespace igs;

extern "C" {

int igs_version(void) { return 110; }

const char* igs_strerror(int code) {
    switch (code) {
        case IGS_OK: return "ok";
        case IGS_ERR_ARG: return "invalid argument (null pointer, negative size or unsupported value)";
        case IGS_ERR_WORKSPACE: return "workspace missing or smaller than igs_workspace_bytes reports";
        case IGS_ERR_LIMIT: return "size beyond a supported limit (B <= 65535, C <= 256, or the fixed scratch of a *_static entry point)";
        case IGS_ERR_DEVICE: return "CUDA device cannot be selected";
        case IGS_ERR_STATUS: return "a kernel gave up on a bounded wait (status word non-zero)";
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown igs_b200 error";
}

long long igs_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int igs_workspace_bytes(int B, int N, int H, int W, int C, int device, size_t* forward_bytes, size_t* backward_bytes) {
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    FwdPlan fp;
    BwdPlan bp;
    rc = plan_forward(B, N, H, W, C, device, &fp);
    if (rc) return rc;
    rc = plan_backward(B, N, H, W, C, device, &bp);
    if (rc) return rc;
    if (forward_bytes) *forward_bytes = fp.bytes;
    if (backward_bytes) *backward_bytes = bp.bytes;
    return IGS_OK;
}

int igs_describe_plan(int B, int N, int H, int W, int C, int device, int* fwd_tile_pixels, int* fwd_splits,
                      int* bwd_threads, int* bwd_slabs) {
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    FwdPlan fp;
    BwdPlan bp;
    rc = plan_forward(B, N, H, W, C, device, &fp);
    if (rc) return rc;
    rc = plan_backward(B, N, H, W, C, device, &bp);
    if (rc) return rc;
    if (fwd_tile_pixels) *fwd_tile_pixels = fp.tile_px;
    if (fwd_splits) *fwd_splits = fp.n_split;
    if (bwd_threads) *bwd_threads = bp.threads;
    if (bwd_slabs) *bwd_slabs = bp.n_slab;
    return IGS_OK;
}

int igs_describe_kernels(int C, int* forward_separable, int* backward_separable) {
    Chunks ch;
    int rc = make_chunks(C, &ch);
    if (rc) return rc;
    if (forward_separable) *forward_separable = forward_has_separable(ch.ct[0]) ? 1 : 0;
    if (backward_separable)
        *backward_separable = (ch.n == 1 && (backward_has_separable(ch.ct[0]) || backward_has_row_kernel(ch.ct[0]))) ? 1 : 0;
    return IGS_OK;
}

int igs_forward_sr(const float* positions, const float* scales, const float* rotations, const float* alphas,
                   const float* colors, const float* x, const int64_t* x_strides, const float* y,
                   const int64_t* y_strides, int B, int N, int H, int W, int C, float eps, int normalize, float* out,
                   float* wsum, const int* order, int hints, void* workspace, size_t workspace_bytes, int device,
                   void* stream) {
    return forward_impl(SHAPE_SCALE_ROT, positions, scales, rotations, nullptr, alphas, colors, x, x_strides, y,
                        y_strides, B, N, H, W, C, eps, normalize, out, wsum, workspace, workspace_bytes, device, stream,
                        nullptr, nullptr, order, hints);
}

int igs_forward_cov(const float* positions, const float* cov_inv_00, const float* cov_inv_01, const float* cov_inv_11,
                    const float* alphas, const float* colors, const float* x, const int64_t* x_strides, const float* y,
                    const int64_t* y_strides, int B, int N, int H, int W, int C, float eps, int normalize, float* out,
                    float* wsum, const int* order, int hints, void* workspace, size_t workspace_bytes, int device,
                    void* stream) {
    return forward_impl(SHAPE_COV_INV, positions, cov_inv_00, cov_inv_01, cov_inv_11, alphas, colors, x, x_strides, y,
                        y_strides, B, N, H, W, C, eps, normalize, out, wsum, workspace, workspace_bytes, device, stream,
                        nullptr, nullptr, order, hints);
}

int igs_normalize(const float* sums, int B, int H, int W, int C, float eps, float* out, float* wsum, int device,
                  void* stream) {
    return normalize_impl(sums, B, H, W, C, eps, out, wsum, device, stream);
}

int igs_backward_sr(const float* positions, const float* scales, const float* rotations, const float* alphas,
                    const float* colors, const float* x, const int64_t* x_strides, const float* y,
                    const int64_t* y_strides, const float* wsum, const float* out, const float* gout, int B, int N,
                    int H, int W, int C, float eps, int grad_mode, float* d_positions, float* d_scales,
                    float* d_rotations, float* d_alphas, float* d_colors, float* d_x, float* d_y, const int* order,
                    int hints, void* workspace, size_t workspace_bytes, int device, void* stream) {
    return backward_impl(SHAPE_SCALE_ROT, positions, scales, rotations, nullptr, alphas, colors, x, x_strides, y,
                         y_strides, wsum, out, gout, B, N, H, W, C, eps, grad_mode, d_positions, d_scales, d_rotations,
                         nullptr, d_alphas, d_colors, d_x, d_y, order, hints, workspace, workspace_bytes, device,
                         stream);
}

int igs_backward_cov(const float* positions, const float* cov_inv_00, const float* cov_inv_01,
                     const float* cov_inv_11, const float* alphas, const float* colors, const float* x,
                     const int64_t* x_strides, const float* y, const int64_t* y_strides, const float* wsum,
                     const float* out, const float* gout, int B, int N, int H, int W, int C, float eps, int grad_mode,
                     float* d_positions, float* d_cov_inv_00, float* d_cov_inv_01, float* d_cov_inv_11,
                     float* d_alphas, float* d_colors, float* d_x, float* d_y, const int* order, int hints,
                     void* workspace, size_t workspace_bytes, int device, void* stream) {
    return backward_impl(SHAPE_COV_INV, positions, cov_inv_00, cov_inv_01, cov_inv_11, alphas, colors, x, x_strides, y,
                         y_strides, wsum, out, gout, B, N, H, W, C, eps, grad_mode, d_positions, d_cov_inv_00,
                         d_cov_inv_01, d_cov_inv_11, d_alphas, d_colors, d_x, d_y, order, hints, workspace,
                         workspace_bytes, device, stream);
}

int igs_render_mse_workspace_bytes(int B, int N, int H, int W, int C, int device, size_t* bytes) {
    if (!bytes) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    // the largest of the layouts a call of this shape can choose (an order only shrinks the forward's)
    RenderMsePlan a, b;
    rc = plan_render_mse(B, N, H, W, C, device, true, true, false, nullptr, &a);
    if (rc) return rc;
    rc = plan_render_mse(B, N, H, W, C, device, false, false, false, nullptr, &b);
    if (rc) return rc;
    *bytes = a.bytes > b.bytes ? a.bytes : b.bytes;
    return IGS_OK;
}

int igs_render_mse_sr(const float* positions, const float* scales, const float* rotations, const float* alphas,
                      const float* colors, int log_scales, const float* x, const int64_t* x_strides, const float* y,
                      const int64_t* y_strides, const float* target, int B, int N, int H, int W, int C, float eps,
                      int grad_mode, const float* upstream, float* loss, float* out, float* d_positions,
                      float* d_scales, float* d_rotations, float* d_alphas, float* d_colors, const int* order,
                      int hints, void* workspace, size_t workspace_bytes, int device, void* stream) {
    return render_mse_impl(positions, scales, rotations, alphas, colors, log_scales, x, x_strides, y, y_strides, target,
                           B, N, H, W, C, eps, grad_mode, upstream, loss, out, d_positions, d_scales, d_rotations,
                           d_alphas, d_colors, order, hints, workspace, workspace_bytes, device, stream);
}

int igs_set_culling(int on) {
    g_culling.store(on ? 1 : 0, std::memory_order_relaxed);
    return IGS_OK;
}

int igs_profile_enable(int on) {
    g_profile_on.store(on == 2 ? 2 : (on ? 1 : 0), std::memory_order_relaxed);
    return IGS_OK;
}

int igs_profile_reset(void) {
    cudaError_t e = profile_drain();
    std::lock_guard<std::mutex> lock(g_profile_mu);
    for (int k = 0; k < K_COUNT; ++k) {
        g_total_ms[k] = 0.0;
        g_timed_launches[k] = 0;
    }
    return (int)e;
}

int igs_profile_read(int kernel_id, double* total_ms, long long* launches) {
    if (kernel_id < 0 || kernel_id >= K_COUNT) return IGS_ERR_ARG;
    cudaError_t e = profile_drain();
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lock(g_profile_mu);
    if (total_ms) *total_ms = g_total_ms[kernel_id];
    if (launches) *launches = g_timed_launches[kernel_id];
    return IGS_OK;
}

// The module's projection output as the parameter tensor: row = {x, y, log sx, log sy,
// rotation, (unused), colours}, opacities all ones.
static ParamLayout feature_layout(int C, const float* pos_offset, float* d_feature) {
    ParamLayout l;
    std::memset(&l, 0, sizeof(l));
    l.pos_s = l.s0_s = l.s1_s = l.col_s = 6 + C;
    l.log_scale = 1;
    l.pos_off = pos_offset;
    l.d_unused = d_feature ? d_feature + 5 : nullptr;
    return l;
}

int igs_forward_feature(const float* gs_feature, const float* pos_offset, const float* x, const int64_t* x_strides,
                        const float* y, const int64_t* y_strides, int B, int N, int H, int W, int C, float eps,
                        int normalize, float* out, float* wsum, const int* order, int hints, void* workspace,
                        size_t workspace_bytes, int device, void* stream) {
    if (C < 1) return IGS_ERR_ARG;
    const ParamLayout l = feature_layout(C, pos_offset, nullptr);
    return forward_impl(SHAPE_SCALE_ROT, gs_feature, gs_feature ? gs_feature + 2 : nullptr,
                        gs_feature ? gs_feature + 4 : nullptr, nullptr, nullptr, gs_feature ? gs_feature + 6 : nullptr, x,
                        x_strides, y, y_strides, B, N, H, W, C, eps, normalize, out, wsum, workspace, workspace_bytes,
                        device, stream, nullptr, &l, order, hints);
}

int igs_backward_feature(const float* gs_feature, const float* pos_offset, const float* x, const int64_t* x_strides,
                         const float* y, const int64_t* y_strides, const float* wsum, const float* out,
                         const float* gout, int B, int N, int H, int W, int C, float eps, int grad_mode,
                         float* d_feature, const int* order, int hints, void* workspace, size_t workspace_bytes,
                         int device, void* stream) {
    if (B < 0 || N < 0 || H < 0 || W < 0 || C < 1) return IGS_ERR_ARG;
    if (B == 0 || N == 0) return IGS_OK;
    if (!gs_feature || !d_feature) return IGS_ERR_ARG;
    if ((long long)H * W == 0) {  // nothing to sum over: every gradient is zero
        int rc = check_device(device);
        if (rc) return rc;
        DeviceGuard guard(device);
        if (!guard.ok) return IGS_ERR_DEVICE;
        return (int)cudaMemsetAsync(d_feature, 0, (size_t)B * N * (6 + C) * sizeof(float),
                                    static_cast<cudaStream_t>(stream));
    }
    const ParamLayout l = feature_layout(C, pos_offset, d_feature);
    return backward_impl(SHAPE_SCALE_ROT, gs_feature, gs_feature + 2, gs_feature + 4, nullptr, nullptr, gs_feature + 6, x,
                         x_strides, y, y_strides, wsum, out, gout, B, N, H, W, C, eps, grad_mode, d_feature,
                         d_feature + 2, d_feature + 4, nullptr, nullptr, d_feature + 6, nullptr, nullptr, order, hints,
                         workspace, workspace_bytes, device, stream, &l);
}

int igs_read_status(const void* workspace, int device, void* stream, int* host_status) {
    if (!workspace || !host_status) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(host_status, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    return *host_status ? IGS_ERR_STATUS : IGS_OK;
}

int igs_read_status_words(const void* workspace, int device, void* stream, int* host_words) {
    if (!workspace || !host_words) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    return (int)cudaMemcpyAsync(host_words, workspace, IGS_STATUS_WORDS * sizeof(int), cudaMemcpyDeviceToHost,
                                static_cast<cudaStream_t>(stream));
}

int igs_read_executed(const void* workspace, int device, void* stream, unsigned long long* host_count) {
    if (!workspace || !host_count) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(host_count, reinterpret_cast<const unsigned long long*>(workspace) + EXEC_COUNT_WORD / 2,
                                    sizeof(unsigned long long), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return (int)e;
}

int igs_read_narrow_count(const void* workspace, int device, void* stream, int* host_count) {
    if (!workspace || !host_count) return IGS_ERR_ARG;
    int rc = check_device(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    return (int)cudaMemcpyAsync(host_count, reinterpret_cast<const int*>(workspace) + NARROW_COUNT_WORD, sizeof(int),
                                cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
