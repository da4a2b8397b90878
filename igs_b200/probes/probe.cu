// Micro-benchmarks that give the roofline its denominators on the GPU at hand:
// the issue rate of the FP32 FMA pipe (scalar FFMA and packed f32x2 FMA) and of the
// MUFU ex2 unit, each from a kernel that does nothing else.  Bench tooling: built into
// its own small library (libigs_probes.so), not into the splat library.  Each entry point
// synchronises and writes a rate to a HOST double; return 0 = ok, -1 = bad argument,
// -4 = device cannot be selected, positive = cudaError_t.
#include "../csrc/common.cuh"

namespace igs {

constexpr int PROBE_THREADS = 256;
constexpr int PROBE_CHAINS = 8;
constexpr int PROBE_ITERS = 4096;

__global__ void __launch_bounds__(PROBE_THREADS) probe_ffma_kernel(float* sink, float m, float c) {
    float v[PROBE_CHAINS];
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = (float)(threadIdx.x + k);
#pragma unroll 16
    for (int it = 0; it < PROBE_ITERS; ++it) {
#pragma unroll
        for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = fmaf(v[k], m, c);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) s += v[k];
    if (sink && s == 123.456f) sink[0] = s;
}

__global__ void __launch_bounds__(PROBE_THREADS) probe_ffma2_kernel(float* sink, float m, float c) {
    f2 v[PROBE_CHAINS];
    const f2 mm = pk(m, m), cc = pk(c, c);
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = pk((float)(threadIdx.x + k), (float)k);
#pragma unroll 16
    for (int it = 0; it < PROBE_ITERS; ++it) {
#pragma unroll
        for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = fma2(v[k], mm, cc);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) {
        float lo, hi;
        upk(v[k], lo, hi);
        s += lo + hi;
    }
    if (sink && s == 123.456f) sink[0] = s;
}

// f32x2 FMAs whose three operands are three different register pairs (a*b + v with a, b, v
// distinct per chain), as in the splat kernels' accumulations; probe_ffma2_kernel multiplies
// by and adds the same two values in every instruction, which the operand reuse cache serves.
__global__ void __launch_bounds__(PROBE_THREADS) probe_ffma2_3op_kernel(float* sink, float m, float c) {
    f2 v[PROBE_CHAINS], a[PROBE_CHAINS], b[PROBE_CHAINS];
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) {
        v[k] = pk((float)(threadIdx.x + k), (float)k);
        a[k] = pk(m + k * 1e-6f, m - k * 1e-6f);
        b[k] = pk(c + k * 1e-6f, c - k * 1e-6f);
    }
#pragma unroll 8
    for (int it = 0; it < PROBE_ITERS; ++it) {
#pragma unroll
        for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = fma2(a[k], b[k], v[k]);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) {
        float lo, hi;
        upk(v[k], lo, hi);
        s += lo + hi;
    }
    if (sink && s == 123.456f) sink[0] = s;
}

__global__ void __launch_bounds__(PROBE_THREADS) probe_ex2_kernel(float* sink, float c) {
    float v[PROBE_CHAINS];
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = -(float)(threadIdx.x + k) * 1e-3f;
#pragma unroll 16
    for (int it = 0; it < PROBE_ITERS; ++it) {
#pragma unroll
        for (int k = 0; k < PROBE_CHAINS; ++k) v[k] = ex2f(v[k]) - c;
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < PROBE_CHAINS; ++k) s += v[k];
    if (sink && s == 123.456f) sink[0] = s;
}

// The kernels' own instruction mix with every dependency removed: NF independent f32x2
// FMAs and two ex2 (each followed by the FADD that keeps its chain bounded) per
// iteration, NF = 11 for the forward mix and 22 for the backward mix.  What this
// reaches is the ceiling of the FMA pipe for that mix on this GPU: MUFU instructions
// are not free for the FMA pipe's issue port.
template <int NF>
__global__ void __launch_bounds__(PROBE_THREADS) probe_mix_kernel(float* sink, float m, float c) {
    f2 v[NF];
    float e0 = -1e-3f * threadIdx.x, e1 = -2e-3f * threadIdx.x;
    const f2 mm = pk(m, m), cc = pk(c, c);
#pragma unroll
    for (int k = 0; k < NF; ++k) v[k] = pk((float)(threadIdx.x + k), (float)k);
#pragma unroll 4
    for (int it = 0; it < PROBE_ITERS / 2; ++it) {
#pragma unroll
        for (int k = 0; k < NF; ++k) v[k] = fma2(v[k], mm, cc);
        e0 = ex2f(e0) - 1.5f;
        e1 = ex2f(e1) - 1.5f;
    }
    float s = e0 + e1;
#pragma unroll
    for (int k = 0; k < NF; ++k) {
        float lo, hi;
        upk(v[k], lo, hi);
        s += lo + hi;
    }
    if (sink && s == 123.456f) sink[0] = s;
}

// Runs `launch` a few times and returns the best per-launch time in seconds (<0 on error).
template <typename F>
static double best_time(F launch, cudaError_t* err) {
    cudaEvent_t e0, e1;
    *err = cudaEventCreate(&e0);
    if (*err != cudaSuccess) return -1.0;
    *err = cudaEventCreate(&e1);
    if (*err != cudaSuccess) {
        cudaEventDestroy(e0);
        return -1.0;
    }
    double best = 1e30;
    for (int rep = 0; rep < 6; ++rep) {
        cudaEventRecord(e0, 0);
        launch();
        cudaEventRecord(e1, 0);
        *err = cudaEventSynchronize(e1);
        if (*err != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep >= 2 && ms * 1e-3 < best) best = ms * 1e-3;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (*err == cudaSuccess) *err = cudaGetLastError();
    return best;
}

static int probe_sm_count(int device) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 148;
    }
    return n;
}

}  // namespace igs

using namespace igs;

extern "C" {

int igs_probe_fp32_rate(int device, int packed, double* lane_instr_per_s) {
    if (!lane_instr_per_s) return IGS_ERR_ARG;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    const int blocks = probe_sm_count(device) * 16;
    cudaError_t err;
    const double t = best_time(
        [&] {
            if (packed == 2)
                probe_ffma2_3op_kernel<<<blocks, PROBE_THREADS>>>(nullptr, 0.999f, 0.001f);
            else if (packed)
                probe_ffma2_kernel<<<blocks, PROBE_THREADS>>>(nullptr, 0.999f, 0.001f);
            else
                probe_ffma_kernel<<<blocks, PROBE_THREADS>>>(nullptr, 0.999f, 0.001f);
        },
        &err);
    if (err != cudaSuccess) return (int)err;
    const double lanes = (double)blocks * PROBE_THREADS * PROBE_CHAINS * (double)PROBE_ITERS * (packed ? 2.0 : 1.0);
    *lane_instr_per_s = lanes / t;
    return IGS_OK;
}

int igs_probe_mix_rate(int device, int backward_mix, double* lane_instr_per_s) {
    if (!lane_instr_per_s) return IGS_ERR_ARG;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    // 96 KB of (unused) dynamic shared memory per CTA holds residency at 2 CTAs of 256
    // threads per SM: the splat kernels' own 16 warps per SM
    const int blocks = probe_sm_count(device) * 8;
    cudaError_t err = backward_mix ? cudaFuncSetAttribute(probe_mix_kernel<22>,
                                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)
                                   : cudaFuncSetAttribute(probe_mix_kernel<11>,
                                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (err != cudaSuccess) return (int)err;
    const double t = best_time(
        [&] {
            if (backward_mix)
                probe_mix_kernel<22><<<blocks, PROBE_THREADS, 96 * 1024>>>(nullptr, 0.999f, 0.001f);
            else
                probe_mix_kernel<11><<<blocks, PROBE_THREADS, 96 * 1024>>>(nullptr, 0.999f, 0.001f);
        },
        &err);
    if (err != cudaSuccess) return (int)err;
    // FMA-pipe lane-instructions: two per f32x2 FMA plus the two scalar FADDs
    const double per_iter = (backward_mix ? 44.0 : 22.0) + 2.0;
    *lane_instr_per_s = (double)blocks * PROBE_THREADS * (PROBE_ITERS / 2) * per_iter / t;
    return IGS_OK;
}

int igs_probe_ex2_rate(int device, double* results_per_s) {
    if (!results_per_s) return IGS_ERR_ARG;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    const int blocks = probe_sm_count(device) * 16;
    cudaError_t err;
    const double t = best_time(
        [&] {
            probe_ex2_kernel<<<blocks, PROBE_THREADS>>>(nullptr, 0.5f);
        },
        &err);
    if (err != cudaSuccess) return (int)err;
    // each iteration also issues one FADD per chain; the MUFU unit (16/clk/SM) is the slower pipe
    *results_per_s = (double)blocks * PROBE_THREADS * PROBE_CHAINS * (double)PROBE_ITERS / t;
    return IGS_OK;
}

}  // extern "C"
