// A whole-layer entry point that never allocates.
//
// Some hosts of this library are not allowed to call cudaMalloc at all: an inference
// server that hands every byte of device memory to its own arena at start-up, a plug-in
// running inside another framework's caching allocator, or a latency-critical loop where
// an allocation (which may synchronise the whole device) is forbidden.  For them the
// packed im2row matrix -- the one piece of scratch memory a layer needs between its two
// kernels -- lives in the fixed array below instead of a cudaMalloc'd workspace.
//
// Cost: a GPU keeps TNNS_NOALLOC_SCRATCH_BYTES of device memory reserved from the moment the
// part of the library that holds the array is loaded on it until the process exits.  With CUDA's
// default lazy module loading that moment is the FIRST call of the entry point on the device (the
// address look-up below loads the module); with CUDA_MODULE_LOADING=EAGER it is the creation of
// the CUDA context.  Either way a host that hands all device memory to its own arena must make
// one call -- an empty batch (N = 0) is enough -- BEFORE the arena takes the memory; afterwards
// the array could no longer be placed and the call reports TNNS_ERR_NOMEM.
#include <mutex>

#include "internal.h"

// The scratch itself.  Device code could name it directly; host code must not use the
// symbol as a pointer (on the host it is only a handle) and asks the runtime for the
// device address instead, once per device, in setup_device() below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[TNNS_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;

struct DeviceState {
    bool ready;
    void* scratch;      // device address of g_noalloc_scratch on this device
    int sm_count;
    size_t smem_optin;
};

std::mutex g_mutex;
DeviceState g_state[kMaxDevices];

// Once per device, with that device current: resolve the device address of the scratch
// array and read the two device attributes the launch heuristics use.  None of these
// calls allocates device memory.
int setup_device(int device, DeviceState** out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& st = g_state[device];
    if (!st.ready) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e == cudaErrorMemoryAllocation) {
            // loading the array's module needs TNNS_NOALLOC_SCRATCH_BYTES of free device memory
            cudaGetLastError();
            return tnns_fail(TNNS_ERR_NOMEM,
                             "device %d has no room left for the %zu-byte scratch array: make the first call (an empty batch is "
                             "enough) before other allocators take the device's memory, or set CUDA_MODULE_LOADING=EAGER",
                             device, (size_t)TNNS_NOALLOC_SCRATCH_BYTES);
        }
        if (e != cudaSuccess || !ptr)
            return tnns_fail(TNNS_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", device, cudaGetErrorString(e));
        int sms = 0, smem = 0, major = 0;
        TNNS_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10) return tnns_fail(TNNS_ERR_UNSUPPORTED, "device %d is not sm_100: this library contains sm_100a code only", device);
        TNNS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        TNNS_CUDA_TRY(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        st.scratch = ptr;
        st.sm_count = sms;
        st.smem_optin = (size_t)smem;
        st.ready = true;
    }
    *out = &st;
    return TNNS_OK;
}

}  // namespace

extern "C" size_t tnns_cuda_noalloc_scratch_bytes(void) { return TNNS_NOALLOC_SCRATCH_BYTES; }

extern "C" int tnns_cuda_conv_noalloc(int type, const int64_t* d_packed_weights, const float* d_x, const float* d_thr, float* d_y,
                                      const tnns_shape_t* s, float alpha, int layout, void* stream) {
    if (!d_packed_weights || !d_x || !d_thr || !d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (type < TNN || type > BNN) return tnns_fail(TNNS_ERR_INVALID, "unknown network type %d", type);
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    if (reinterpret_cast<uintptr_t>(d_packed_weights) & 15) return tnns_fail(TNNS_ERR_INVALID, "packed weights must be 16-byte aligned");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (g.KN <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive kernel count");
    const size_t need = tnns_packed_bytes(type, s);
    if (need > TNNS_NOALLOC_SCRATCH_BYTES)
        return tnns_fail(TNNS_ERR_UNSUPPORTED,
                         "packed im2row matrix needs %zu bytes but the built-in scratch holds %zu: split the batch into smaller "
                         "calls or use tnns_cuda_conv_ws with your own workspace",
                         need, (size_t)TNNS_NOALLOC_SCRATCH_BYTES);
    int device = 0;
    TNNS_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return tnns_fail(TNNS_ERR_UNSUPPORTED, "device index %d beyond %d", device, kMaxDevices);
    // before the empty-batch return: a start-up call with N = 0 is how a host resolves (and thereby
    // reserves) the scratch array on this device while memory is still free
    DeviceState* st = nullptr;
    if ((rc = setup_device(device, &st))) return rc;
    if (g.N == 0) return TNNS_OK;

    // The launchers only read these three fields of a context; nothing here owns memory.
    tnns_cuda_ctx view = {};
    view.device = device;
    view.sm_count = st->sm_count;
    view.smem_optin = st->smem_optin;

    const bool act_ternary = (type == TNN || type == TBN);
    // The pack kernel writes every word of every row (padding pixels, channel tails and the
    // pad-to-four words included), so whatever an earlier call left in the scratch is
    // overwritten before the GEMM reads it: nothing has to be cleared.
    rc = tnns_launch_pack(&view, act_ternary, d_x, d_thr, st->scratch, g, layout, TNNS_PACK_AUTO, (cudaStream_t)stream);
    if (rc) return rc;
    const long long M = (long long)g.N * g.OH * g.OW;
    return tnns_launch_gemm_popc(&view, type, st->scratch, d_packed_weights, d_y, M, g.KN, g.Kp, g.OH * g.OW, g.C * g.KH * g.KW, alpha,
                                 layout, true, (cudaStream_t)stream);
}
