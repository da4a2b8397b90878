// igs_forward_sr_static: the forward from scales and rotations for hosts that cannot
// hand the library a workspace because they have no way to allocate device memory.
//
// Who that is.  igs_forward_sr wants a scratch buffer from its caller (the packed
// gaussian records and, when the gaussians are split across CTAs, the partial sums).
// Under PyTorch that is one torch.empty.  A host that is not PyTorch may own nothing
// but the input and output buffers it was given: a plug-in running inside someone
// else's renderer or inference server, where every device allocation belongs to the
// embedding application and its budget was fixed at start-up; or a latency-critical
// loop that must not touch the driver's allocator (cudaMalloc and cudaFree serialise
// against the whole device) once it is running.  For those callers the scratch lives
// in a fixed array inside this library's device image.
//
// What it costs.  Every GPU that loads libigs_b200.so keeps IGS_STATIC_SCRATCH_BYTES of
// device memory for the array until the process exits, whether or not this entry point
// is ever called.  Shapes whose scratch does not fit are refused with IGS_ERR_LIMIT.
//
// Sharing.  There is one array per device and every call uses it from offset zero.  It
// keeps whatever the previous call left; each call rewrites the records it reads and
// clears its status word first, so stale contents are never consumed.  Two calls whose
// kernels overlap on the same GPU (different streams, or different host threads on
// different streams) would write the same bytes at the same time: the caller must
// order them on one stream.
//
// Address.  The array's name is a host-side handle, not a device address; every call
// looks the device address up with cudaGetSymbolAddress while its device is current (a
// cheap host-side lookup once the library's device code is loaded, and it stays right if
// the application tears the device's context down and brings it up again).  The very
// first lookup on a device may load the device code: make the first call during start-up,
// before any stream capture is begun on that device.
//
// Status.  A kernel that gives up on a bounded wait sets the first word of the array, which
// the caller cannot reach through a workspace pointer: igs_read_status_static reads it.
#include "pack.cuh"
#include "plan.cuh"

namespace igs {

static __device__ __align__(256) unsigned char g_static_scratch[IGS_STATIC_SCRATCH_BYTES];

// Device address of the array on the current device.
static int static_scratch_address(void** out) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!p) return IGS_ERR_DEVICE;
    *out = p;
    return IGS_OK;
}

static int check_device_index(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return IGS_ERR_DEVICE;
    }
    return IGS_OK;
}

}  // namespace igs

using namespace igs;

extern "C" int igs_forward_sr_static(const float* positions, const float* scales, const float* rotations,
                                     const float* alphas, const float* colors, const float* x,
                                     const int64_t* x_strides, const float* y, const int64_t* y_strides, int B, int N,
                                     int H, int W, int C, float eps, int normalize, float* out, float* wsum, int device,
                                     void* stream) {
    if (B < 0 || N < 0 || H < 0 || W < 0 || C < 1) return IGS_ERR_ARG;
    int rc = check_device_index(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;

    FwdPlan p;
    rc = plan_forward(B, N, H, W, C, device, &p);
    if (rc) return rc;
    if (p.bytes > IGS_STATIC_SCRATCH_BYTES) {
        // fall back to a single gaussian split: no partial sums, only the records
        p.n_split = 1;
        long long per = ((long long)N + p.chunk_g - 1) / p.chunk_g * p.chunk_g;
        p.per_split = (int)(per > 0 ? per : p.chunk_g);
        p.bytes = p.off_partial;  // records end where the (now unused) partial sums began
    }
    if (p.bytes > IGS_STATIC_SCRATCH_BYTES) return IGS_ERR_LIMIT;

    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc) return rc;
    return forward_impl(SHAPE_SCALE_ROT, positions, scales, rotations, nullptr, alphas, colors, x, x_strides, y,
                        y_strides, B, N, H, W, C, eps, normalize, out, wsum, scratch, IGS_STATIC_SCRATCH_BYTES, device,
                        stream, &p);
}

extern "C" int igs_read_status_static(int device, void* stream, int* host_status) {
    if (!host_status) return IGS_ERR_ARG;
    int rc = check_device_index(device);
    if (rc) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return IGS_ERR_DEVICE;
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc) return rc;
    return igs_read_status(scratch, device, stream, host_status);
}
