// Launch plans: how a call of shape (B, N, H, W, C) is cut into channel chunks,
// pixel tiles x gaussian splits (forward) and gaussian groups x pixel slabs
// (backward), and where each scratch array sits in the caller's workspace.
#pragma once

#include "common.cuh"

namespace igs {

constexpr int MAX_CHUNKS = 16;   // channel chunks of up to 16 -> C <= 256
constexpr int STATUS_BYTES = 256;

struct Chunks {
    int n;
    int c0[MAX_CHUNKS];  // first channel of the chunk
    int cr[MAX_CHUNKS];  // real channels in the chunk
    int ct[MAX_CHUNKS];  // kernel instantiation used (>= cr)
};

struct FwdPlan {
    Chunks ch;
    int threads;        // threads per CTA
    int px_per_thread;  // pixels each thread owns (even)
    int tile_px;        // threads * px_per_thread
    int tiles;          // CTAs along the pixel axis, per batch element (general kernel)
    int tiles_sep;      // the same for the separable kernel (16 x 64 pixel tiles), 0 = not available
    int tiles_x;        // separable tiles per tile row
    int n_split;        // CTAs along the gaussian axis
    int per_split;      // gaussians per split
    int chunk_g;        // gaussians per shared-memory stage
    int stages;
    size_t off_frec[MAX_CHUNKS];
    size_t off_partial;  // [n_split][B][C+1][HW] when n_split > 1 or not normalising in-kernel
    size_t off_cbox;     // [B][ceil(N / chunk_g)][4]: bounding boxes of the stages' gaussians (ordered calls)
    size_t bytes;
};

struct BwdPlan {
    Chunks ch;
    int threads;           // threads per CTA
    int gauss_per_thread;  // gaussians each thread owns (1 or 2)
    int n_slab;            // CTAs along the pixel axis
    long long npairs;      // pixel pairs per batch element
    long long pairs_per_slab;
    int chunk_pairs;       // pixel pairs per shared-memory stage
    int stages;
    int planes;            // moment planes per (slab, batch): 6 per chunk + C
    int sep_ok;            // a separable instantiation exists for this shape
    int row_kernel;        // ... and it is the row-streaming one (8 / 16 channels, backward_row.cu)
    int rows, cols;        // image size
    int nrp, ncb;          // separable: row pairs (2 rows) and blocks (4 columns) per row pair
    int rp_per_slab;       // separable: row pairs per slab (same n_slab as the general kernel)
    size_t off_geo;
    size_t off_prec[MAX_CHUNKS];
    size_t off_axes;       // row-streaming kernel: y per row, [B][H]
    size_t off_part;       // [n_slab][B][planes][N]
    size_t off_tasks;      // ordered skipping path: [task_capacity] int4, then [B][ceil(N/32)] int4
    size_t off_slab_range; //   and [B][N] int (valid when task_capacity > 0)
    int task_capacity;     // B * ceil(N/32) * (most slabs either partition has); 0 without separable kernels
    size_t bytes;
};

int make_chunks(int C, Chunks* out);
int plan_forward(int B, int N, int H, int W, int C, int device, FwdPlan* p);
// fine_slabs: the partition used when the caller passes a spatial order (many short slabs, so
// that the few slabs each gaussian group reaches still fill the machine).  The workspace
// size covers both partitions.
// separable_grid: size the plain slab count for the separable kernel's occupancy (the kernel
// that will run) instead of the general kernel's.
int plan_backward(int B, int N, int H, int W, int C, int device, BwdPlan* p, bool fine_slabs = false,
                  bool separable_grid = false);

// Where the per-gaussian parameters live.  The default is the reference's separate
// contiguous tensors; the feature-level entry points point all of them into the rows of one
// [M, 6+C] tensor (the module's projection output) instead.  Strides are in floats.
struct ParamLayout {
    int pos_s, s0_s, s1_s, col_s;  // row strides of positions, shape0, shape1, colours
    int log_scale;                 // shape0 holds log-scales: scale = exp(v) + eps
    const float* pos_off;          // [M,2] added to the positions, or nullptr
    float* d_unused;               // backward: a column (row stride pos_s) to fill with zeros, or nullptr
};

// Extras of a forward that is the first half of a fused forward + loss + backward call.
struct FwdExtras {
    float* geo_out;       // the prologue also writes the backward's geometry records here, or nullptr
    int leave_partials;   // do not add the gaussian splits up: the caller reads [n_split][B][C+1][HW] itself
};

// What a backward may find already done by such a forward (see backward_impl).
struct BwdPrepared {
    unsigned char* status;  // the forward's status area: narrow count, axis flags
};

// Body of igs_forward_sr / igs_forward_cov (kind = ShapeKind).  use_plan, when given,
// replaces the plan the call would compute itself.
int forward_impl(int kind, const float* pos, const float* s0, const float* s1, const float* s2, const float* alpha,
                 const float* colors, const float* x, const int64_t* xs, const float* y, const int64_t* ys, int B, int N,
                 int H, int W, int C, float eps, int normalize, float* out, float* wsum, void* workspace,
                 size_t workspace_bytes, int device, void* stream, const FwdPlan* use_plan = nullptr,
                 const ParamLayout* layout = nullptr, const int* order = nullptr, int hints = 0,
                 const FwdExtras* extras = nullptr);

// occupancy (CTAs per SM) of the instantiation a plan selects; defined next to the kernels
int forward_ctas_per_sm(int ct, int device);
int backward_ctas_per_sm(int ct, int device);
int backward_sep_ctas_per_sm(int ct, int device);
int forward_px_per_thread(int ct);
int forward_threads(int ct);
int forward_chunk_g(int ct);
bool forward_has_separable(int ct);
int forward_sep_tile_h();
int forward_sep_tile_w();
int backward_threads(int ct);
int backward_gauss_per_thread(int ct);
int backward_chunk_pairs(int ct);

}  // namespace igs
