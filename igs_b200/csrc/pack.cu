// Per-gaussian prologue kernel: one thread per gaussian turns the caller's raw
// parameters into the geometry record (backward) and the duplicated forward
// records (one array per channel chunk).
#include "pack.cuh"

namespace igs {

__global__ void __launch_bounds__(256) pack_kernel(PackArgs a) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.M) return;
    const float px = a.pos[2 * i], py = a.pos[2 * i + 1];
    float c00, c01, c11;
    if (a.kind == SHAPE_SCALE_ROT) {
        const CovInv ci = cov_inv_from_scale_rot(a.shape0[2 * i], a.shape0[2 * i + 1], a.shape1[i], a.eps);
        c00 = ci.c00;
        c01 = ci.c01;
        c11 = ci.c11;
    } else {
        c00 = a.shape0[i];
        c01 = a.shape1[i];
        c11 = a.shape2[i];
    }
    const float A = EXP2_SCALE * c00, B2 = 2.0f * EXP2_SCALE * c01, Cq = EXP2_SCALE * c11;
    const float al = a.alpha[i];
    if (a.geo) {
        float4* g = reinterpret_cast<float4*>(a.geo + i * GEO_FLOATS);
        g[0] = make_float4(px, py, A, B2);
        g[1] = make_float4(Cq, al, 0.f, 0.f);
    }
    for (int k = 0; k < a.ch.n; ++k) {
        float* rec = a.frec[k];
        if (!rec) continue;
        const int ct = a.ch.ct[k], cr = a.ch.cr[k], c0 = a.ch.c0[k];
        const int rs = fwd_rec_floats(ct);
        // colours pre-multiplied by alpha: numerator += e * (alpha * colour)
        float* r = rec + i * rs;
        r[0] = px; r[1] = py; r[2] = A; r[3] = B2; r[4] = Cq; r[5] = al;
        for (int c = 0; c < rs - 6; ++c) r[6 + c] = (c < cr) ? al * a.colors[i * a.C + c0 + c] : 0.f;
    }
}

cudaError_t launch_pack(const PackArgs& a, cudaStream_t s) {
    if (a.M <= 0) return cudaSuccess;
    const int threads = 256;
    const long long blocks = (a.M + threads - 1) / threads;
    {
        KernelTimer timer(K_PACK, s);
        pack_kernel<<<(unsigned)blocks, threads, 0, s>>>(a);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace igs
