// Shared device helpers for the sm_100a splat kernels: packed-fp32 (f32x2) math,
// ex2, mbarrier + 1-D bulk (TMA) copies with bounded waits, record layouts.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/igs_b200.h"

namespace igs {

// ---------------------------------------------------------------------------
// Record layouts
// ---------------------------------------------------------------------------
// Geometry record, one per gaussian, 8 floats (32 B):
//   {px, py, A, B2, Cq, alpha, hx, hy}
// with the exponent coefficients pre-scaled so that the weight is
//   e = 2^(A*dx^2 + B2*dx*dy + Cq*dy^2),  A = k*c00, B2 = 2k*c01, Cq = k*c11,
//   k = -0.5*log2(e).
constexpr int GEO_FLOATS = 8;
constexpr float EXP2_SCALE = -0.72134752044448170368f;  // -0.5 * log2(e)

// Forward record, one per gaussian and channel chunk, padded to a multiple of 4 floats:
//   {px, py, A, B2,  Cq, al, al*c0, al*c1,  al*c2, ..., hx, hy}
// (hx, hy: half-widths of the box outside which the weight is exactly zero, see pack.cu).
// Each value is stored once and duplicated into an f32x2 operand in registers (a move on
// the otherwise idle ALU pipe): a record then costs 3 sixteen-byte broadcast reads at
// C = 3 instead of the 5 a pre-duplicated record needs, and the shared-memory return path
// (4 cycles per 16-byte warp read) stops co-limiting the kernel.
__host__ __device__ constexpr int fwd_rec_floats(int ct) { return (8 + ct + 3) / 4 * 4; }

// Exponents (log2 units) below -CULL_T are treated as "certainly flushed to zero":
// ex2.approx.ftz returns exactly 0 below -126; the margin absorbs fp32 rounding.
constexpr float CULL_T = 130.0f;

// Words of the workspace's 256-byte status area.
constexpr int STATUS_WORD = 0;       // kernels: a bounded wait gave up
constexpr int GRID_FLAG_WORD = 1;    // bit 0 = grid not separable, bit 1 = axes not monotone, bit 2 = upstream not finite,
                                     // bit 3 = the separability check ran (bit 0 is an answer, not a default)
constexpr int NARROW_COUNT_WORD = 2; // pack: gaussians whose reach is well inside the image
constexpr int EXEC_COUNT_WORD = 4;   // (64 bits) culling kernels: (gaussian, pixel) evaluations not skipped
constexpr int TASK_COUNT_WORD = 6;   // ordered backward: tasks on its list ...
constexpr int TASK_NEXT_WORD = 7;    // ... and the next one to hand out
constexpr int GRID_NOT_SEPARABLE = 1, GRID_NOT_MONOTONE = 2, GRID_CHECKED = 8;
// Skipping a term w * t because w is exactly zero is only lossless while t is finite
// (0 * NaN and 0 * inf are NaN).  Gaussians with a non-finite parameter get an infinite box
// (pack.cu); a non-finite upstream value (gout / weight sum) sets this bit, and the backward
// then runs its dense kernel, which propagates the NaN the way the reference does.
constexpr int UPSTREAM_NOT_FINITE = 4;
constexpr int NO_BACKWARD_SKIPPING = GRID_NOT_MONOTONE | UPSTREAM_NOT_FINITE;

// Backward pixel record, one per PAIR of consecutive pixels and channel chunk:
//   {x0,x1, y0,y1, gS0,gS1, gn0_0,gn0_1, ...}  padded to 4 floats
__host__ __device__ constexpr int bwd_rec_floats(int ct) { return (6 + 2 * ct + 3) / 4 * 4; }

// Backward block record (separable grids), one per 2-row x 4-column block of pixels:
//   {x0,x1,x2,x3, y0,y1,-,-} then, per pixel pair (row 0 cols 01, row 0 cols 23, row 1 cols
//   01, row 1 cols 23), {gS0,gS1, gn0_0,gn0_1, ...} padded to 4 floats
__host__ __device__ constexpr int bwd_sep_pair_floats(int ct) { return (2 + 2 * ct + 3) / 4 * 4; }
__host__ __device__ constexpr int bwd_sep_rec_floats(int ct) { return 8 + 4 * bwd_sep_pair_floats(ct); }

// Moment planes written by the backward kernel per (slab, gaussian):
//   M0, Mx, My, Mxx, Mxy, Myy, then one plane per channel of the chunk
constexpr int N_MOMENTS = 6;

// Channel-chunk sizes the kernels are instantiated for; any channel count is covered
// by a sequence of chunks (linearity of every sum in the colours).
__host__ __device__ inline int chunk_template(int c) {
    return c <= 1 ? 1 : c == 2 ? 2 : c == 3 ? 3 : c == 4 ? 4 : c <= 8 ? 8 : 16;
}

// ---------------------------------------------------------------------------
// Packed fp32 math (two lanes per 64-bit register pair; Blackwell-only PTX)
// ---------------------------------------------------------------------------
typedef unsigned long long f2;

__device__ __forceinline__ f2 pk(float lo, float hi) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk(f2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
    f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 sub2(f2 a, f2 b) {
    f2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float ex2f(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ f2 ex2_2(f2 q) {
    float a, b;
    upk(q, a, b);
    return pk(ex2f(a), ex2f(b));
}

// ---------------------------------------------------------------------------
// mbarrier + bulk copy (global -> shared, this CTA only), every wait bounded
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity; gives up after a fixed number of polls
// (each poll itself blocks for a hardware-defined time slice), returning false.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int it = 0; it < (1 << 20); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// bytes: multiple of 16; dst and src 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Status word written by kernels when a bounded wait gives up (0 = fine).
constexpr int STATUS_WAIT_TIMEOUT = 1;

// ---------------------------------------------------------------------------
// Host-side plumbing shared by the .cu files
// ---------------------------------------------------------------------------
void count_launch(int n = 1);
int sm_count(int device);

// Kernel ids for igs_profile_read (include/igs_b200.h lists them as IGS_KERNEL_*).
enum KernelId { K_PACK = 0, K_FORWARD, K_REDUCE, K_PIXEL_TERMS, K_BACKWARD, K_FINALIZE, K_COORD_GRAD, K_GRID_CHECK, K_COUNT };

// When profiling is enabled, brackets one launch with CUDA events on its own stream;
// otherwise does nothing.
struct KernelTimer {
    int id;
    int dev = -1;
    cudaStream_t stream;
    cudaEvent_t start = nullptr, stop = nullptr;
    KernelTimer(int id, cudaStream_t s);
    ~KernelTimer();
};

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
        if (ok && prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace igs
