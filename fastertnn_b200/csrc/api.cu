// Device-resident C ABI: contexts, weights, error reporting, layer entry points.
#include <algorithm>
#include <vector>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "internal.h"
#include "prelu_thresholds.cuh"

// ---------------------------------------------------------------------------------------
// thread-local error state
// ---------------------------------------------------------------------------------------
static thread_local int tl_status = TNNS_OK;
static thread_local char tl_detail[512] = "";
static thread_local unsigned long long tl_launches = 0;

int tnns_fail(int status, const char* fmt, ...) {
    tl_status = status;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_detail, sizeof(tl_detail), fmt, ap);
    va_end(ap);
    return status;
}
void tnns_count_launch(void) { tl_launches++; }
void tnns_add_launches(unsigned long long n) { tl_launches += n; }

extern "C" {

int tnns_cuda_last_error(void) { return tl_status; }
const char* tnns_cuda_error_detail(void) { return tl_detail; }
unsigned long long tnns_cuda_launch_count(void) { return tl_launches; }

const char* tnns_cuda_strerror(int status) {
    switch (status) {
        case TNNS_OK: return "success";
        case TNNS_ERR_INVALID: return "invalid argument";
        case TNNS_ERR_CUDA: return "CUDA runtime error";
        case TNNS_ERR_NOMEM: return "out of memory";
        case TNNS_ERR_UNSUPPORTED: return "shape not supported by the requested algorithm";
        case TNNS_ERR_DEVICE_WAIT: return "bounded on-device wait expired";
        default: return "unknown status";
    }
}

int tnns_out_dim(int in, int pad, int k, int stride) { return (in + 2 * pad - k) / stride + 1; }
int tnns_k_words(int C, int KH, int KW) { return KH * KW * ((C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS); }
int tnns_k_padded(int C, int KH, int KW) { return 4 * ((tnns_k_words(C, KH, KW) + 3) / 4); }

}  // extern "C"

int tnns_make_geom(const tnns_shape_t* s, TnnsGeom* g) {
    if (!s) return tnns_fail(TNNS_ERR_INVALID, "shape is NULL");
    if (s->N < 0 || s->C <= 0 || s->H <= 0 || s->W <= 0 || s->KN < 0 || s->KH <= 0 || s->KW <= 0 || s->PH < 0 || s->PW < 0 ||
        s->SH <= 0 || s->SW <= 0)
        return tnns_fail(TNNS_ERR_INVALID, "non-positive dimension in shape (N=%d C=%d H=%d W=%d KN=%d KH=%d KW=%d P=%d,%d S=%d,%d)",
                         s->N, s->C, s->H, s->W, s->KN, s->KH, s->KW, s->PH, s->PW, s->SH, s->SW);
    if (s->H + 2 * s->PH < s->KH || s->W + 2 * s->PW < s->KW)
        return tnns_fail(TNNS_ERR_INVALID, "kernel %dx%d larger than padded image %dx%d", s->KH, s->KW, s->H + 2 * s->PH,
                         s->W + 2 * s->PW);
    g->N = s->N; g->C = s->C; g->H = s->H; g->W = s->W;
    g->KN = s->KN; g->KH = s->KH; g->KW = s->KW;
    g->PH = s->PH; g->PW = s->PW; g->SH = s->SH; g->SW = s->SW;
    g->OH = tnns_out_dim(s->H, s->PH, s->KH, s->SH);
    g->OW = tnns_out_dim(s->W, s->PW, s->KW, s->SW);
    g->Cp = (s->C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS;
    g->Kw = s->KH * s->KW * g->Cp;
    g->Kp = 4 * ((g->Kw + 3) / 4);
    return TNNS_OK;
}

static inline bool type_act_ternary(int type) { return type == TNN || type == TBN; }
static inline bool type_wgt_ternary(int type) { return type == TNN || type == BTN; }

// Every entry point that launches work opens with this: a context belongs to one device, but the
// calling thread's current device is whatever its last CUDA call left it (a thread that holds two
// contexts is on the second one's device after creating it).  Makes the context's device current,
// and refuses weights that live on another device.
static int enter(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w = nullptr) {
    int cur = -1;
    TNNS_CUDA_TRY(cudaGetDevice(&cur));
    if (cur != ctx->device) TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    if (w && w->device != ctx->device)
        return tnns_fail(TNNS_ERR_INVALID, "weights live on device %d, context on %d", w->device, ctx->device);
    return TNNS_OK;
}
#define TNNS_ENTER(...)                   \
    do {                                  \
        int rc__ = enter(__VA_ARGS__);    \
        if (rc__) return rc__;            \
    } while (0)

extern "C" {

size_t tnns_packed_bytes(int type, const tnns_shape_t* s) {
    TnnsGeom g;
    if (tnns_make_geom(s, &g) != TNNS_OK) return 0;
    return (size_t)g.N * g.OH * g.OW * g.Kp * 8 * (type_act_ternary(type) ? 2 : 1);
}

int tnns_cuda_create(int device, tnns_cuda_ctx** out) {
    if (!out) return tnns_fail(TNNS_ERR_INVALID, "ctx out-pointer is NULL");
    *out = nullptr;
    int count = 0;
    TNNS_CUDA_TRY(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return tnns_fail(TNNS_ERR_INVALID, "device %d out of range (have %d)", device, count);
    TNNS_CUDA_TRY(cudaSetDevice(device));
    tnns_cuda_ctx* ctx = new (std::nothrow) tnns_cuda_ctx();
    if (!ctx) return tnns_fail(TNNS_ERR_NOMEM, "host allocation of context failed");
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess && prop.major != 10) {
        delete ctx;
        return tnns_fail(TNNS_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library contains sm_100a code only", device,
                         prop.major, prop.minor);
    }
    if (e == cudaSuccess) e = cudaMalloc(&ctx->d_status, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMallocHost(&ctx->h_status, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->s_copy_in, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->s_compute, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->s_copy_out, cudaStreamNonBlocking);
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
        e = cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_done[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        tnns_cuda_destroy(ctx);
        return tnns_fail(TNNS_ERR_CUDA, "context set-up failed: %s", cudaGetErrorString(e));
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    *out = ctx;
    return TNNS_OK;
}

void tnns_cuda_destroy(tnns_cuda_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    for (int i = 0; i < 2; i++) {
        if (ctx->stage_in[i]) cudaFree(ctx->stage_in[i]);
        if (ctx->stage_out[i]) cudaFree(ctx->stage_out[i]);
        if (ctx->stage_pack[i]) cudaFree(ctx->stage_pack[i]);
        if (ctx->ev_in[i]) cudaEventDestroy(ctx->ev_in[i]);
        if (ctx->ev_done[i]) cudaEventDestroy(ctx->ev_done[i]);
        if (ctx->ev_out[i]) cudaEventDestroy(ctx->ev_out[i]);
    }
    if (ctx->stage_thr) cudaFree(ctx->stage_thr);
    if (ctx->fused_sync) cudaFree(ctx->fused_sync);
    if (ctx->s_copy_in) cudaStreamDestroy(ctx->s_copy_in);
    if (ctx->s_compute) cudaStreamDestroy(ctx->s_compute);
    if (ctx->s_copy_out) cudaStreamDestroy(ctx->s_copy_out);
    delete ctx;
}

int tnns_cuda_sync(tnns_cuda_ctx* ctx) {
    if (!ctx) return tnns_fail(TNNS_ERR_INVALID, "ctx is NULL");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    TNNS_CUDA_TRY(cudaDeviceSynchronize());
    TNNS_CUDA_TRY(cudaMemcpy(ctx->h_status, ctx->d_status, sizeof(unsigned int), cudaMemcpyDeviceToHost));
    if (*ctx->h_status != 0) {
        const unsigned int code = *ctx->h_status;
        cudaMemset(ctx->d_status, 0, sizeof(unsigned int));
        // a launch that gave up may have left before its words were consistent: start from zeros again
        if (ctx->fused_sync) cudaMemset(ctx->fused_sync, 0, ctx->fused_sync_words * sizeof(unsigned int));
        return tnns_fail(TNNS_ERR_DEVICE_WAIT, "device status word = 0x%x (a bounded wait gave up)", code);
    }
    return TNNS_OK;
}

// Failure-detection self-test: launches a kernel whose only mbarrier wait can never be satisfied.
// The bounded wait gives up after about a second, the kernel returns normally, and the next
// tnns_cuda_sync reports TNNS_ERR_DEVICE_WAIT; the context stays usable.
int tnns_cuda_selftest_wait_expiry(tnns_cuda_ctx* ctx) {
    if (!ctx) return tnns_fail(TNNS_ERR_INVALID, "ctx is NULL");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    return tnns_launch_wait_selftest(ctx, 0);
}

// The constants of the threshold form of "PReLU, then the next layer's quantiser" (prelu_thresholds.cuh),
// computed by the same code the kernels run.
int tnns_prelu_thresholds(float t, float alpha, float bias, int ternary, float* n1, float* t2) {
    if (!n1 || !t2) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (!(alpha > 0.f && alpha <= 1.f)) return tnns_fail(TNNS_ERR_INVALID, "the threshold form needs 0 < alpha <= 1 (got %g)", (double)alpha);
    const tnns_thr::Pair r = tnns_thr::make(t + 0.0f, alpha, bias, ternary != 0);
    *n1 = r.n1;
    *t2 = r.t2;
    return TNNS_OK;
}

// --- plain memory helpers so C callers need no CUDA headers -------------------------------
int tnns_cuda_malloc(tnns_cuda_ctx* ctx, size_t bytes, void** out) {
    if (!ctx || !out) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    *out = nullptr;
    TNNS_CUDA_TRY(cudaMalloc(out, bytes ? bytes : 16));
    return TNNS_OK;
}
int tnns_cuda_mem_info(tnns_cuda_ctx* ctx, size_t* free_bytes, size_t* total_bytes) {
    if (!ctx || !free_bytes || !total_bytes) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    TNNS_CUDA_TRY(cudaMemGetInfo(free_bytes, total_bytes));
    return TNNS_OK;
}
int tnns_cuda_malloc_host(tnns_cuda_ctx* ctx, size_t bytes, void** out) {
    if (!ctx || !out) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    *out = nullptr;
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    TNNS_CUDA_TRY(cudaHostAlloc(out, std::max<size_t>(bytes, 16), cudaHostAllocPortable | cudaHostAllocMapped));
    return TNNS_OK;
}

void tnns_cuda_free_host(tnns_cuda_ctx* ctx, void* p) {
    (void)ctx;
    if (p) cudaFreeHost(p);
}

void tnns_cuda_free(tnns_cuda_ctx* ctx, void* p) {
    if (!ctx || !p) return;
    cudaSetDevice(ctx->device);
    cudaFree(p);
}
int tnns_cuda_memcpy_h2d(tnns_cuda_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    TNNS_CUDA_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    return TNNS_OK;
}
int tnns_cuda_memcpy_d2h(tnns_cuda_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    TNNS_CUDA_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return TNNS_OK;
}

// --- weights ---------------------------------------------------------------------------------
static int upload_weights_impl(tnns_cuda_ctx* ctx, int type, const int64_t* packed_host, int KN, int C, int KH, int KW,
                               int K_words, int K_unpack, tnns_cuda_weights** out) {
    if (!ctx || !packed_host || !out) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    *out = nullptr;
    if (type < TNN || type > BNN) return tnns_fail(TNNS_ERR_INVALID, "unknown network type %d", type);
    if (KN <= 0 || K_words <= 0 || K_unpack < 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive weight dimension");
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    tnns_cuda_weights* w = new (std::nothrow) tnns_cuda_weights();
    if (!w) return tnns_fail(TNNS_ERR_NOMEM, "host allocation failed");
    memset(w, 0, sizeof(*w));
    w->type = type; w->KN = KN; w->C = C; w->KH = KH; w->KW = KW; w->device = ctx->device;
    w->Cp = C > 0 ? (C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS : 0;
    w->Kw = K_words;
    w->Kp = 4 * ((K_words + 3) / 4);
    w->K_unpack = K_unpack;
    w->packed_bytes = (size_t)KN * w->Kp * 8 * (type_wgt_ternary(type) ? 2 : 1);
    cudaError_t e = cudaMalloc(&w->d_packed, w->packed_bytes);
    // cudaMemcpyDefault: the packed rows may live on the host or (packed by tnns_cuda_pack_weights) on a device
    if (e == cudaSuccess) e = cudaMemcpy(w->d_packed, packed_host, w->packed_bytes, cudaMemcpyDefault);
    if (e != cudaSuccess) {
        tnns_cuda_free_weights(ctx, w);
        return tnns_fail(e == cudaErrorMemoryAllocation ? TNNS_ERR_NOMEM : TNNS_ERR_CUDA, "weight upload failed: %s",
                         cudaGetErrorString(e));
    }
    int rc = tnns_build_i8_weights(ctx, w);
    if (rc != TNNS_OK) {
        tnns_cuda_free_weights(ctx, w);
        return rc;
    }
    if (C > 0 && tnns_dense_eligible(type, C, KH, KW)) {
        // few input channels: also keep the kernel as a 1x1 layer over only the real positions of a window.  The
        // repacked rows are in the reference's packed format, so the same upload builds that layer's operand images.
        const int Kd = tnns_dense_channels(C, KH, KW), Kw_d = Kd / TNNS_WORD_BITS, Kp_d = 4 * ((Kw_d + 3) / 4);
        uint64_t* d_tmp = nullptr;
        e = cudaMalloc(&d_tmp, (size_t)KN * Kp_d * 8 * (type_wgt_ternary(type) ? 2 : 1));
        if (e == cudaSuccess) {
            rc = tnns_launch_repack_weights_dense(ctx, w, d_tmp, Kp_d);
            if (rc == TNNS_OK && (e = cudaDeviceSynchronize()) == cudaSuccess)
                rc = upload_weights_impl(ctx, type, reinterpret_cast<const int64_t*>(d_tmp), KN, Kd, 1, 1, Kw_d, K_unpack, &w->dense);
            cudaFree(d_tmp);
        }
        if (e != cudaSuccess || rc != TNNS_OK) {
            tnns_cuda_free_weights(ctx, w);
            return rc != TNNS_OK ? rc : tnns_fail(e == cudaErrorMemoryAllocation ? TNNS_ERR_NOMEM : TNNS_ERR_CUDA, "dense weight form failed: %s", cudaGetErrorString(e));
        }
    }
    *out = w;
    return TNNS_OK;
}

int tnns_cuda_upload_weights(tnns_cuda_ctx* ctx, int type, const int64_t* packed_host, int KN, int C, int KH, int KW,
                             tnns_cuda_weights** out) {
    if (C <= 0 || KH <= 0 || KW <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive weight dimension");
    return upload_weights_impl(ctx, type, packed_host, KN, C, KH, KW, tnns_k_words(C, KH, KW), C * KH * KW, out);
}

int tnns_cuda_upload_weights_packed(tnns_cuda_ctx* ctx, int type, const int64_t* packed_host, int KN, int K_words,
                                    int K_unpack, tnns_cuda_weights** out) {
    return upload_weights_impl(ctx, type, packed_host, KN, 0, 0, 0, K_words, K_unpack, out);
}

void tnns_cuda_free_weights(tnns_cuda_ctx* ctx, tnns_cuda_weights* w) {
    if (!w) return;
    if (ctx) cudaSetDevice(ctx->device);
    if (w->d_packed) cudaFree(w->d_packed);
    if (w->d_i8) cudaFree(w->d_i8);
    if (w->d_f4) cudaFree(w->d_f4);
    if (w->d_jtab) cudaFree(w->d_jtab);
    if (w->dense) tnns_cuda_free_weights(nullptr, w->dense);
    delete w;
}

int tnns_cuda_pack_weights(tnns_cuda_ctx* ctx, int ternary, const float* d_w, const float* d_thr, int64_t* d_packed, int KN, int C,
                           int KH, int KW, void* stream) {
    if (!ctx || !d_w || !d_thr || !d_packed) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (KN <= 0 || C <= 0 || KH <= 0 || KW <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive weight dimension");
    TNNS_ENTER(ctx);
    return tnns_launch_pack_weights(ctx, ternary != 0, d_w, d_thr, d_packed, KN, C, KH, KW, (cudaStream_t)stream);
}

// --- kernels -----------------------------------------------------------------------------------
int tnns_cuda_pack(tnns_cuda_ctx* ctx, int ternary, const float* d_x, const float* d_thr, int64_t* d_packed,
                   const tnns_shape_t* s, int layout, int algo, void* stream) {
    if (!ctx || !d_x || !d_thr || !d_packed) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (reinterpret_cast<uintptr_t>(d_packed) & 15) return tnns_fail(TNNS_ERR_INVALID, "packed buffer must be 16-byte aligned");
    if (algo < TNNS_PACK_AUTO || algo > TNNS_PACK_STAGED) return tnns_fail(TNNS_ERR_INVALID, "unknown pack algorithm %d", algo);
    TNNS_ENTER(ctx);
    return tnns_launch_pack(ctx, ternary != 0, d_x, d_thr, d_packed, g, layout, algo, (cudaStream_t)stream);
}

int tnns_cuda_gemm(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const int64_t* d_a, float* d_y, int N, int OH, int OW,
                   float alpha, int layout, int algo, void* stream) {
    if (!ctx || !w || !d_a || !d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (N < 0 || OH <= 0 || OW <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive output dimension");
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    TNNS_ENTER(ctx, w);
    if (reinterpret_cast<uintptr_t>(d_a) & 15) return tnns_fail(TNNS_ERR_INVALID, "packed operand must be 16-byte aligned");
    const long long M = (long long)N * OH * OW;
    const int K_unpack = w->K_unpack;
    switch (algo) {
        case TNNS_GEMM_POPC_SIMPLE:
            return tnns_launch_gemm_popc(ctx, w->type, d_a, w->d_packed, d_y, M, w->KN, w->Kp, OH * OW, K_unpack, alpha, layout,
                                         false, (cudaStream_t)stream);
        case TNNS_GEMM_POPC_TILED:
            return tnns_launch_gemm_popc(ctx, w->type, d_a, w->d_packed, d_y, M, w->KN, w->Kp, OH * OW, K_unpack, alpha, layout,
                                         true, (cudaStream_t)stream);
        case TNNS_GEMM_AUTO:
            // Measured on B200 (large layer, us per launch): 4-bit tensor path 90, int8 tensor path
            // 126, integer pipe 2140; the order is the same on every layer shape of the benchmark
            // set down to batch-1 56x56x256 (15 / 18 / 44).  The integer-pipe kernel remains for
            // rows too long for the tensor paths' exact range.
            if (w->d_f4 && w->Kp < 65536)
                return tnns_launch_gemm_tc(ctx, w, d_a, d_y, M, OH * OW, alpha, layout, true, (cudaStream_t)stream);
            return tnns_launch_gemm_popc(ctx, w->type, d_a, w->d_packed, d_y, M, w->KN, w->Kp, OH * OW, K_unpack, alpha, layout,
                                         true, (cudaStream_t)stream);
        case TNNS_GEMM_I8_TC:
            return tnns_launch_gemm_tc(ctx, w, d_a, d_y, M, OH * OW, alpha, layout, false, (cudaStream_t)stream);
        case TNNS_GEMM_F4_TC:
            return tnns_launch_gemm_tc(ctx, w, d_a, d_y, M, OH * OW, alpha, layout, true, (cudaStream_t)stream);
        default:
            return tnns_fail(TNNS_ERR_INVALID, "unknown GEMM algorithm %d", algo);
    }
}

// --- quantise only, and the GEMM that gathers its own im2row rows -----------------------------------
int tnns_cuda_quantise(tnns_cuda_ctx* ctx, int ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                       int W, int layout, void* stream) {
    if (!ctx || !d_x || !d_thr || !d_image) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (N < 0 || C <= 0 || H <= 0 || W <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive dimension");
    if (reinterpret_cast<uintptr_t>(d_image) & 31) return tnns_fail(TNNS_ERR_INVALID, "image must be 32-byte aligned");
    TNNS_ENTER(ctx);
    return tnns_launch_quantise(ctx, ternary != 0, d_x, d_thr, d_image, N, C, H, W, layout, (cudaStream_t)stream);
}

int tnns_cuda_gemm_implicit(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const tnns_shape_t* s,
                            float alpha, int layout, void* stream) {
    if (!ctx || !w || !d_image || !d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    if (reinterpret_cast<uintptr_t>(d_image) & 31) return tnns_fail(TNNS_ERR_INVALID, "image must be 32-byte aligned");
    if (!w->d_f4 || !w->d_jtab || w->Kp >= 65536) return tnns_fail(TNNS_ERR_UNSUPPORTED, "implicit im2row needs the 4-bit tensor-core GEMM");
    TNNS_ENTER(ctx, w);
    return tnns_launch_gemm_tc(ctx, w, d_image, d_y, (long long)g.N * g.OH * g.OW, g.OH * g.OW, alpha, layout, true, (cudaStream_t)stream,
                               nullptr, nullptr, 1, &g);
}

// --- the same with the copy engine gathering 4-bit tiles -------------------------------------------
size_t tnns_e2m1_image_bytes(int N, int C, int H, int W) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0) return 0;
    return (size_t)N * H * W * ((C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS) * 32;
}

int tnns_cuda_im2col_supported(const tnns_cuda_weights* w, const tnns_shape_t* s) {
    TnnsGeom g;
    if (!w || tnns_make_geom(s, &g)) return 0;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW) return 0;
    return tnns_im2col_supported(w, g) ? 1 : 0;
}

int tnns_cuda_quantise_e2m1(tnns_cuda_ctx* ctx, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H, int W,
                            int layout, void* stream) {
    if (!ctx || !d_x || !d_thr || !d_image) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (N < 0 || C <= 0 || H <= 0 || W <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive dimension");
    if (reinterpret_cast<uintptr_t>(d_image) & 31) return tnns_fail(TNNS_ERR_INVALID, "image must be 32-byte aligned");
    TNNS_ENTER(ctx);
    return tnns_launch_quantise(ctx, true, d_x, d_thr, d_image, N, C, H, W, layout, (cudaStream_t)stream, TNNS_IMG_E2M1);
}

int tnns_cuda_gemm_im2col(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const tnns_shape_t* s,
                          float alpha, int layout, int pairs, void* stream) {
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    if (!ctx || !w || !d_image || !d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    TNNS_ENTER(ctx, w);
    if (reinterpret_cast<uintptr_t>(d_image) & 31) return tnns_fail(TNNS_ERR_INVALID, "image must be 32-byte aligned");
    return tnns_launch_gemm_im2col(ctx, w, d_image, d_y, g, alpha, layout, (cudaStream_t)stream, pairs);
}

// --- bordered 4-bit images and the slab-fed GEMM (stride-1 layers) ----------------------------------
size_t tnns_e2m1_bordered_image_bytes(int N, int C, int H, int W, int PH, int PW) { return tnns_bordered_image_bytes(N, C, H, W, PH, PW); }

static inline size_t slab_image_bytes(int N, int C, int H, int W, int PH, int PW) {
    return (tnns_bordered_image_bytes(N, C, H, W, PH, PW) + 127) & ~(size_t)127;
}
size_t tnns_slab_workspace_bytes(int N, int C, int H, int W, int PH, int PW) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || PH < 0 || PW < 0) return 0;
    return slab_image_bytes(N, C, H, W, PH, PW) + tnns_fused_sync_bytes(N);
}

// the stand-alone quantise kernel that writes the bordered image takes either layout
// (a 1x1 image is the same memory in both layouts and is read as pixel-major: fully connected layers)
static int quantise_layout(int layout, int H, int W) { return (H == 1 && W == 1) ? TNNS_NHWC : layout; }
static bool bordered_quantise_ok(const float* d_x, int N, int C, int H, int W, int layout) {
    if (quantise_layout(layout, H, W) == TNNS_NHWC) return tnns_quantise_tma_nhwc_supported(d_x, N, C, H, W);
    return tnns_quantise_tma_supported(d_x, H, W, layout);
}

int tnns_cuda_quantise_e2m1_bordered(tnns_cuda_ctx* ctx, int ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                                     int W, int PH, int PW, int layout, void* stream) {
    if (!ctx || !d_x || !d_thr || !d_image) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || PH < 0 || PW < 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive dimension");
    if (reinterpret_cast<uintptr_t>(d_image) & 127) return tnns_fail(TNNS_ERR_INVALID, "bordered image must be 128-byte aligned");
    if (!bordered_quantise_ok(d_x, N, C, H, W, layout))
        return tnns_fail(TNNS_ERR_UNSUPPORTED,
                         "the bordered image is written from a 16-byte aligned base: NCHW with H*W a multiple of four (at least 32), or NHWC "
                         "with C a multiple of four and at least 128 pixels in all");
    TNNS_ENTER(ctx);
    return tnns_launch_quantise_tma(ctx, ternary != 0, d_x, d_thr, d_image, N, C, H, W, (cudaStream_t)stream, TNNS_IMG_E2M1, PH, PW,
                                    quantise_layout(layout, H, W));
}

static int slab_geom(const tnns_cuda_weights* w, const tnns_shape_t* s, TnnsGeom* g) {
    int rc = tnns_make_geom(s, g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    return TNNS_OK;
}

int tnns_cuda_slab_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s) {
    TnnsGeom g;
    if (!ctx || !w || !s || tnns_make_geom(s, &g)) return 0;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW) return 0;
    return tnns_slab_supported(ctx, w, g, false) ? 1 : 0;
}

// Where the library itself prefers the slab-fed route (tnns_cuda_conv with TNNS_GEMM_AUTO, ConvStack).
// Measured on B200, quantise + GEMM in us, slab-fed / im2col-fed (or, binary activations, gathering warps):
//   256 x 64x56x56 -> 64      GEMM alone 55 / 93          256 x 128x28x28 -> 128   55 / 58
//   1 x 256x56x56 -> 256 BTN  13.1 / 14.0                 64 x 512x32x32 -> 512 BTN  95 / 102
//   64 x 512x32x32 -> 512     95 / 79 (one launch)        256 x 256x14x14 -> 256   37 / 35
// The slab removes the per-tap copy requests, which is what bounds 32- and 64-byte pixels, and it is the only
// copy-engine form of binary activations; on 128-byte pixels the tensor pipe bounds both forms and the padded
// lattice's extra rows (13 % at 32x32, 31 % at 14x14) decide for the im2col form.
int tnns_cuda_slab_preferred(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s) {
    TnnsGeom g;
    if (!ctx || !w || !s || tnns_make_geom(s, &g)) return 0;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW) return 0;
    if (!tnns_slab_supported(ctx, w, g, false)) return 0;
    const double useful = (double)g.OH * g.OW / ((double)(g.H + 2 * g.PH) * (g.W + 2 * g.PW));
    if (useful < 0.75) return 0;
    return (!type_act_ternary(w->type) || g.Cp <= 2) ? 1 : 0;
}

// next_format of the public slab entry points -> (format, binary) of the launcher
static int slab_next(int next_format, int* fmt, int* binary) {
    switch (next_format) {
        case 0: *fmt = 0; *binary = 1; return TNNS_OK;
        case 1: *fmt = 1; *binary = 0; return TNNS_OK;
        case 2: *fmt = 2; *binary = 0; return TNNS_OK;
        case 3: *fmt = 3; *binary = 0; return TNNS_OK;
        case 5: *fmt = 3; *binary = 1; return TNNS_OK;
        default: return tnns_fail(TNNS_ERR_INVALID, "output format must be 0, 1, 2, 3 or 5");
    }
}

int tnns_cuda_gemm_slab(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const tnns_shape_t* s, float alpha,
                        int layout, int pairs, void* stream) {
    if (!ctx || !w || !d_image || !d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    TnnsGeom g;
    int rc = slab_geom(w, s, &g);
    if (rc) return rc;
    TNNS_ENTER(ctx, w);
    return tnns_launch_gemm_slab(ctx, w, d_image, d_y, g, alpha, layout, (cudaStream_t)stream, pairs);
}

int tnns_cuda_gemm_slab_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, void* d_image_out, const float* d_thr_next,
                                   int next_format, int next_PH, int next_PW, const tnns_shape_t* s, float alpha, int pairs, void* stream) {
    if (!ctx || !w || !d_image || !d_image_out || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    if (reinterpret_cast<uintptr_t>(d_image_out) & 15) return tnns_fail(TNNS_ERR_INVALID, "output image must be 16-byte aligned");
    int fmt, bin;
    int rc = slab_next(next_format, &fmt, &bin);
    if (rc) return rc;
    TnnsGeom g;
    if ((rc = slab_geom(w, s, &g))) return rc;
    TNNS_ENTER(ctx, w);
    return tnns_launch_gemm_slab(ctx, w, d_image, nullptr, g, alpha, TNNS_NCHW, (cudaStream_t)stream, pairs, d_image_out, d_thr_next, fmt, bin,
                                 next_PH, next_PW);
}

static int conv_slab_impl(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y, void* d_image_out,
                          const float* d_thr_next, int fmt, int bin, int next_PH, int next_PW, void* d_workspace, size_t workspace_bytes,
                          const tnns_shape_t* s, float alpha, int pairs, void* stream) {
    if (!ctx || !w || !d_x || !d_thr || !d_workspace) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    TnnsGeom g;
    int rc = slab_geom(w, s, &g);
    if (rc) return rc;
    if (g.N == 0) return TNNS_OK;
    if (reinterpret_cast<uintptr_t>(d_workspace) & 127) return tnns_fail(TNNS_ERR_INVALID, "workspace must be 128-byte aligned");
    const size_t need = tnns_slab_workspace_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW);
    if (workspace_bytes < need) return tnns_fail(TNNS_ERR_INVALID, "workspace of %zu bytes, need %zu", workspace_bytes, need);
    TNNS_ENTER(ctx, w);
    TnnsFusedInput f;
    f.d_x = d_x;
    f.d_thr = d_thr;
    f.d_sync = reinterpret_cast<unsigned int*>(static_cast<char*>(d_workspace) + slab_image_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW));
    return tnns_launch_gemm_slab(ctx, w, d_workspace, d_y, g, alpha, TNNS_NCHW, (cudaStream_t)stream, pairs, d_image_out, d_thr_next, fmt, bin, next_PH,
                                 next_PW, &f);
}

int tnns_cuda_conv_slab(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y, void* d_workspace,
                        size_t workspace_bytes, const tnns_shape_t* s, float alpha, int pairs, void* stream) {
    if (!d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    return conv_slab_impl(ctx, w, d_x, d_thr, d_y, nullptr, nullptr, 2, 0, 0, 0, d_workspace, workspace_bytes, s, alpha, pairs, stream);
}

int tnns_cuda_conv_slab_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, void* d_image_out,
                                   const float* d_thr_next, int next_format, int next_PH, int next_PW, void* d_workspace, size_t workspace_bytes,
                                   const tnns_shape_t* s, float alpha, int pairs, void* stream) {
    if (!d_image_out || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (reinterpret_cast<uintptr_t>(d_image_out) & 15) return tnns_fail(TNNS_ERR_INVALID, "output image must be 16-byte aligned");
    int fmt, bin;
    int rc = slab_next(next_format, &fmt, &bin);
    if (rc) return rc;
    return conv_slab_impl(ctx, w, d_x, d_thr, nullptr, d_image_out, d_thr_next, fmt, bin, next_PH, next_PW, d_workspace, workspace_bytes, s, alpha, pairs,
                          stream);
}

int tnns_cuda_conv_slab_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout) {
    TnnsGeom g;
    if (!ctx || !w || !s || tnns_make_geom(s, &g)) return 0;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW) return 0;
    return (tnns_slab_supported(ctx, w, g, true) && tnns_quantise_tma_supported(d_x, g.H, g.W, layout)) ? 1 : 0;
}

// The one-launch slab form (quantiser warps inside the GEMM kernel) measured slower than its two launches on
// every shape tried (64 x 512x32x32 -> 512: 98 against 95 us; 256 x 128x28x28 -> 128: 86 against 55), so the
// library never picks it by itself; it stays available on request (TNNS_GEMM_F4_SLAB_FUSED, tnns_cuda_conv_slab).
int tnns_cuda_conv_slab_one_launch_preferred(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout) {
    (void)ctx; (void)w; (void)s; (void)d_x; (void)layout;
    return 0;
}

// --- layers with few input channels as a dense 1x1 layer (dense.cu) -------------------------------
// geometry of the virtual layer: N x OH x OW pixels of Kd channels, 1x1 filter, stride 1, no padding
static bool dense_geom(const tnns_cuda_weights* w, const TnnsGeom& g, TnnsGeom* gv) {
    if (!w->dense || g.C != w->C || g.KH != w->KH || g.KW != w->KW || g.KN != w->KN) return false;
    const int Kd = w->dense->C;
    *gv = g;
    gv->C = Kd; gv->H = g.OH; gv->W = g.OW; gv->KH = gv->KW = 1; gv->PH = gv->PW = 0; gv->SH = gv->SW = 1;
    gv->Cp = Kd / TNNS_WORD_BITS; gv->Kw = gv->Cp; gv->Kp = 4 * ((gv->Cp + 3) / 4);
    return tnns_im2col_supported(w->dense, *gv);
}

size_t tnns_dense_workspace_bytes(const tnns_shape_t* s) {
    TnnsGeom g;
    if (!s || tnns_make_geom(s, &g)) return 0;
    return (((size_t)g.N * g.OH * g.OW * (size_t)(tnns_dense_channels(g.C, g.KH, g.KW) / 2)) + 127) & ~(size_t)127;
}

int tnns_cuda_dense_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s) {
    TnnsGeom g, gv;
    if (!ctx || !w || !s || tnns_make_geom(s, &g)) return 0;
    return dense_geom(w, g, &gv) ? 1 : 0;
}

static int conv_dense_impl(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y, void* d_image_out,
                           const float* d_thr_next, int next_format, void* d_workspace, size_t workspace_bytes, const tnns_shape_t* s,
                           float alpha, int layout, void* stream, int next_PH = 0, int next_PW = 0) {
    if (!ctx || !w || !d_x || !d_thr || !d_workspace) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    TnnsGeom g, gv;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    if (!dense_geom(w, g, &gv)) return tnns_fail(TNNS_ERR_UNSUPPORTED, "layer outside the dense few-channel route (ternary activations, at most 16 channels)");
    if (reinterpret_cast<uintptr_t>(d_workspace) & 127) return tnns_fail(TNNS_ERR_INVALID, "workspace must be 128-byte aligned");
    const size_t need = tnns_dense_workspace_bytes(s);
    if (workspace_bytes < need) return tnns_fail(TNNS_ERR_INVALID, "workspace of %zu bytes, need %zu", workspace_bytes, need);
    TNNS_ENTER(ctx, w);
    if (g.N == 0) return TNNS_OK;
    rc = tnns_launch_dense_quantise(ctx, d_x, d_thr, d_workspace, g, gv.C, layout, (cudaStream_t)stream);
    if (rc) return rc;
    return tnns_launch_gemm_im2col(ctx, w->dense, d_workspace, d_y, gv, alpha, layout, (cudaStream_t)stream, 0, d_image_out, d_thr_next, next_format,
                                   nullptr, next_PH, next_PW);
}

int tnns_cuda_conv_dense(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y, void* d_workspace,
                         size_t workspace_bytes, const tnns_shape_t* s, float alpha, int layout, void* stream) {
    if (!d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    return conv_dense_impl(ctx, w, d_x, d_thr, d_y, nullptr, nullptr, 1, d_workspace, workspace_bytes, s, alpha, layout, stream);
}

int tnns_cuda_conv_dense_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, void* d_image_out,
                                    const float* d_thr_next, int next_format, int next_PH, int next_PW, void* d_workspace, size_t workspace_bytes,
                                    const tnns_shape_t* s, float alpha, int layout, void* stream) {
    if (!d_image_out || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (reinterpret_cast<uintptr_t>(d_image_out) & (next_format == 3 ? 127 : 15)) return tnns_fail(TNNS_ERR_INVALID, "output image must be 16-byte (bordered: 128-byte) aligned");
    if (next_format < 0 || next_format > 3) return tnns_fail(TNNS_ERR_INVALID, "output format must be 0, 1, 2 or 3");
    return conv_dense_impl(ctx, w, d_x, d_thr, nullptr, d_image_out, d_thr_next, next_format, d_workspace, workspace_bytes, s, alpha, layout, stream,
                           next_PH, next_PW);
}

// The algorithm tnns_cuda_conv / _conv_ws resolve TNNS_GEMM_AUTO (with TNNS_PACK_AUTO) to, workspace permitting.
int tnns_cuda_conv_auto_algo(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout) {
    if (!ctx || !w || !s) return TNNS_GEMM_AUTO;
    if (tnns_cuda_dense_supported(ctx, w, s)) return TNNS_GEMM_F4_DENSE;
    if (layout == TNNS_NCHW && tnns_cuda_slab_preferred(ctx, w, s) && tnns_cuda_conv_slab_supported(ctx, w, s, d_x, layout))
        return tnns_cuda_conv_slab_one_launch_preferred(ctx, w, s, d_x, layout) ? TNNS_GEMM_F4_SLAB_FUSED : TNNS_GEMM_F4_SLAB;
    if (layout == TNNS_NHWC && tnns_cuda_slab_preferred(ctx, w, s) && tnns_quantise_tma_nhwc_supported(d_x, s->N, s->C, s->H, s->W))
        return TNNS_GEMM_F4_SLAB;  // two launches: the quantiser inside the GEMM kernel reads NCHW only
    if (tnns_cuda_conv_fused_preferred(const_cast<tnns_cuda_ctx*>(ctx), w, s, d_x, layout)) return TNNS_GEMM_F4_FUSED;
    return TNNS_GEMM_F4_TC;
}

// --- chained layers without the fp32 round trip ------------------------------------------------
static inline size_t fused_image_bytes(int N, int C, int H, int W) { return (tnns_e2m1_image_bytes(N, C, H, W) + 127) & ~(size_t)127; }

size_t tnns_fused_workspace_bytes(int N, int C, int H, int W) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0) return 0;
    return fused_image_bytes(N, C, H, W) + tnns_fused_sync_bytes(N);
}

int tnns_cuda_conv_fused_supported(const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout) {
    TnnsGeom g;
    if (!w || !s || tnns_make_geom(s, &g)) return 0;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW) return 0;
    return tnns_fused_supported(w, g, d_x, layout) ? 1 : 0;
}

static int conv_fused_impl(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y,
                           void* d_image_out, const float* d_thr_next, int next_format, void* d_workspace, size_t workspace_bytes,
                           const tnns_shape_t* s, float alpha, int pairs, void* stream, int layout = TNNS_NCHW) {
    if (!ctx || !w || !d_x || !d_thr || !d_workspace) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    if (g.N == 0) return TNNS_OK;
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    if (reinterpret_cast<uintptr_t>(d_workspace) & 127) return tnns_fail(TNNS_ERR_INVALID, "workspace must be 128-byte aligned");
    const size_t need = tnns_fused_workspace_bytes(g.N, g.C, g.H, g.W);
    if (workspace_bytes < need) return tnns_fail(TNNS_ERR_INVALID, "workspace of %zu bytes, need %zu", workspace_bytes, need);
    TNNS_ENTER(ctx, w);
    TnnsFusedInput f;
    f.d_x = d_x;
    f.d_thr = d_thr;
    f.d_sync = reinterpret_cast<unsigned int*>(static_cast<char*>(d_workspace) + fused_image_bytes(g.N, g.C, g.H, g.W));
    return tnns_launch_gemm_im2col(ctx, w, d_workspace, d_y, g, alpha, layout, (cudaStream_t)stream, pairs, d_image_out, d_thr_next,
                                   next_format, &f);
}

int tnns_cuda_conv_fused(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y,
                         void* d_workspace, size_t workspace_bytes, const tnns_shape_t* s, float alpha, int pairs, void* stream) {
    if (!d_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    return conv_fused_impl(ctx, w, d_x, d_thr, d_y, nullptr, nullptr, 1, d_workspace, workspace_bytes, s, alpha, pairs, stream);
}

int tnns_cuda_conv_fused_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr,
                                    void* d_image_out, const float* d_thr_next, int next_format, void* d_workspace,
                                    size_t workspace_bytes, const tnns_shape_t* s, float alpha, int pairs, void* stream) {
    if (!d_image_out || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (reinterpret_cast<uintptr_t>(d_image_out) & 15) return tnns_fail(TNNS_ERR_INVALID, "output image must be 16-byte aligned");
    if (next_format < 0 || next_format > 2) return tnns_fail(TNNS_ERR_INVALID, "output format must be 0, 1 or 2");
    return conv_fused_impl(ctx, w, d_x, d_thr, nullptr, d_image_out, d_thr_next, next_format, d_workspace, workspace_bytes, s, alpha, pairs,
                           stream);
}

// The rule tnns_cuda_conv applies with TNNS_GEMM_AUTO: the one-launch route where the layer qualifies
// and every SM has at least three 128-row tiles (measured, one launch / two launches in us: 32 images of
// 512x32x32 -> 512, 3.5 tiles per SM: 49 / 54; 256 x 256x14x14 -> 256, 2.6: 43 / 40; 16 images, 1.7: 33 / 31.5).
int tnns_cuda_conv_fused_preferred(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout) {
    if (!ctx || !tnns_cuda_conv_fused_supported(w, s, d_x, layout)) return 0;
    const long long tiles = (((long long)s->N * tnns_out_dim(s->H, s->PH, s->KH, s->SH) * tnns_out_dim(s->W, s->PW, s->KW, s->SW) + 127) / 128) *
                            ((s->KN + 255) / 256);
    return tiles >= 3LL * ctx->sm_count ? 1 : 0;
}

size_t tnns_packed_image_bytes(int ternary, int N, int C, int H, int W) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0) return 0;
    return (size_t)N * (ternary ? 2 : 1) * H * W * ((C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS) * 8;
}

int tnns_cuda_gemm_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const int64_t* d_a, void* d_image,
                              const float* d_thr_next, int next_ternary, int N, int OH, int OW, float alpha, void* stream) {
    if (!ctx || !w || !d_a || !d_image || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (N < 0 || OH <= 0 || OW <= 0) return tnns_fail(TNNS_ERR_INVALID, "non-positive output dimension");
    TNNS_ENTER(ctx, w);
    if ((reinterpret_cast<uintptr_t>(d_a) & 15) || (reinterpret_cast<uintptr_t>(d_image) & 15))
        return tnns_fail(TNNS_ERR_INVALID, "packed operand and image must be 16-byte aligned");
    if (!w->d_f4 || w->Kp >= 65536) return tnns_fail(TNNS_ERR_UNSUPPORTED, "packed output needs the tensor-core GEMM");
    if (next_ternary < 0 || next_ternary > 2) return tnns_fail(TNNS_ERR_INVALID, "output format must be 0, 1 or 2");
    return tnns_launch_gemm_tc(ctx, w, d_a, nullptr, (long long)N * OH * OW, OH * OW, alpha, TNNS_NCHW, true, (cudaStream_t)stream,
                               d_image, d_thr_next, next_ternary);
}

int tnns_cuda_gemm_im2col_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, void* d_image_out,
                                     const float* d_thr_next, int next_format, const tnns_shape_t* s, float alpha, int pairs,
                                     void* stream) {
    if (!ctx || !w || !d_image || !d_image_out || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    TNNS_ENTER(ctx, w);
    if ((reinterpret_cast<uintptr_t>(d_image) & 31) || (reinterpret_cast<uintptr_t>(d_image_out) & 15))
        return tnns_fail(TNNS_ERR_INVALID, "input image must be 32-byte, output image 16-byte aligned");
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    if (next_format < 0 || next_format > 2) return tnns_fail(TNNS_ERR_INVALID, "output format must be 0, 1 or 2");
    return tnns_launch_gemm_im2col(ctx, w, d_image, nullptr, g, alpha, TNNS_NCHW, (cudaStream_t)stream, pairs, d_image_out, d_thr_next,
                                   next_format);
}

int tnns_cuda_gemm_im2col_bordered_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, void* d_image_out,
                                       const float* d_thr_next, int next_PH, int next_PW, const tnns_shape_t* s, float alpha, int pairs,
                                       void* stream) {
    if (!ctx || !w || !d_image || !d_image_out || !d_thr_next) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    TNNS_ENTER(ctx, w);
    if ((reinterpret_cast<uintptr_t>(d_image) & 31) || (reinterpret_cast<uintptr_t>(d_image_out) & 127))
        return tnns_fail(TNNS_ERR_INVALID, "input image must be 32-byte, bordered output image 128-byte aligned");
    if (pairs < 0 || pairs > 2) return tnns_fail(TNNS_ERR_INVALID, "pairs must be 0, 1 or 2");
    return tnns_launch_gemm_im2col(ctx, w, d_image, nullptr, g, alpha, TNNS_NCHW, (cudaStream_t)stream, pairs, d_image_out, d_thr_next, 3, nullptr,
                                   next_PH, next_PW);
}

int tnns_cuda_im2row_packed(tnns_cuda_ctx* ctx, int ternary, const void* d_image, int64_t* d_packed, const tnns_shape_t* s,
                            void* stream) {
    if (!ctx || !d_image || !d_packed) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if ((reinterpret_cast<uintptr_t>(d_packed) & 15) || (reinterpret_cast<uintptr_t>(d_image) & 15))
        return tnns_fail(TNNS_ERR_INVALID, "image and packed buffer must be 16-byte aligned");
    TNNS_ENTER(ctx);
    return tnns_launch_pack(ctx, ternary != 0, reinterpret_cast<const float*>(d_image), reinterpret_cast<const float*>(d_image), d_packed, g,
                            TNNS_SRC_PACKED_IMAGE, TNNS_PACK_AUTO, (cudaStream_t)stream);
}

int tnns_cuda_conv_ws(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y,
                      void* d_workspace, size_t workspace_bytes, const tnns_shape_t* s, float alpha, int layout, int pack_algo,
                      int gemm_algo, void* stream) {
    if (!ctx || !w || !d_x || !d_thr || !d_y || !d_workspace) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape (KN=%d C=%d %dx%d) does not match the uploaded weights (KN=%d C=%d %dx%d)", s->KN,
                         s->C, s->KH, s->KW, w->KN, w->C, w->KH, w->KW);
    TNNS_ENTER(ctx, w);
    if (g.N == 0) return TNNS_OK;
    const bool auto_both = pack_algo == TNNS_PACK_AUTO && gemm_algo == TNNS_GEMM_AUTO;
    if (auto_both) {
        // the library's own choice; a slab-fed form is taken only when the caller's workspace holds its bordered image
        const int pick = tnns_cuda_conv_auto_algo(ctx, w, s, d_x, layout);
        if (pick == TNNS_GEMM_F4_DENSE && (reinterpret_cast<uintptr_t>(d_workspace) & 127) == 0 && tnns_dense_workspace_bytes(s) <= workspace_bytes)
            gemm_algo = pick;
        if (pick == TNNS_GEMM_F4_SLAB || pick == TNNS_GEMM_F4_SLAB_FUSED) {
            const size_t ws_need = pick == TNNS_GEMM_F4_SLAB_FUSED ? tnns_slab_workspace_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW)
                                                                   : tnns_bordered_image_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW);
            if ((reinterpret_cast<uintptr_t>(d_workspace) & 127) == 0 && ws_need <= workspace_bytes) gemm_algo = pick;
        }
    }
    if (gemm_algo == TNNS_GEMM_F4_DENSE) {
        // few input channels: only the real positions of every window, as a 1x1 layer
        if (pack_algo != TNNS_PACK_AUTO) return tnns_fail(TNNS_ERR_UNSUPPORTED, "the dense few-channel route has its own quantise step");
        return conv_dense_impl(ctx, w, d_x, d_thr, d_y, nullptr, nullptr, 1, d_workspace, workspace_bytes, s, alpha, layout, stream);
    }
    if (gemm_algo == TNNS_GEMM_F4_SLAB || gemm_algo == TNNS_GEMM_F4_SLAB_FUSED) {
        // stride-1 layers from a bordered 4-bit image: one slab of pixels per tile serves every filter tap
        const bool one_launch = gemm_algo == TNNS_GEMM_F4_SLAB_FUSED;
        const size_t ws_need = one_launch ? tnns_slab_workspace_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW)
                                          : tnns_bordered_image_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW);
        if (pack_algo != TNNS_PACK_AUTO || (layout != TNNS_NCHW && (one_launch || layout != TNNS_NHWC)) || !tnns_slab_supported(ctx, w, g, one_launch) ||
            !bordered_quantise_ok(d_x, g.N, g.C, g.H, g.W, layout) || (reinterpret_cast<uintptr_t>(d_workspace) & 127) || ws_need > workspace_bytes)
            return tnns_fail(TNNS_ERR_UNSUPPORTED, "layer, layout, workspace size or alignment outside the slab-fed route");
        if (one_launch) return tnns_cuda_conv_slab(ctx, w, d_x, d_thr, d_y, d_workspace, workspace_bytes, s, alpha, 0, stream);
        rc = tnns_launch_quantise_tma(ctx, type_act_ternary(w->type), d_x, d_thr, d_workspace, g.N, g.C, g.H, g.W, (cudaStream_t)stream, TNNS_IMG_E2M1,
                                      g.PH, g.PW, quantise_layout(layout, g.H, g.W));
        if (rc) return rc;
        return tnns_launch_gemm_slab(ctx, w, d_workspace, d_y, g, alpha, layout, (cudaStream_t)stream);
    }
    // Default route: quantise the input once into a packed image (1/16 of the fp32 bytes) and let
    // the 4-bit tensor-core GEMM gather its im2row rows from it, so the KH*KW-times larger im2row
    // matrix is never written.  Forcing a pack or GEMM algorithm selects the explicit two-kernel
    // route (pack to the im2row matrix, then GEMM).
    // Where the layer qualifies (ternary activations, C a multiple of 256) the image is written as
    // 4-bit operands and the copy engine delivers the GEMM's activation tiles (im2col tensor copies).
    if (gemm_algo == TNNS_GEMM_F4_FUSED || auto_both) {
        // one launch: the quantise step runs inside the GEMM kernel.  Taken on request, and by
        // default where every SM has several tiles, so that the quantisation of later images hides
        // under the MMAs of earlier ones (with one or two tiles per SM the two steps mostly run one
        // after the other anyway, and the stand-alone quantise kernel is the faster of the two).
        // Measured on B200, fused / two launches in us: 64 x 512x32x32 -> 512 (6.9 tiles per SM)
        // 81 / 95, 256 x 128x28x28 -> 128 (10.6) 58 / 66, 256 x 64x56x56 -> 64 (42) 130 / 142;
        // 256 x 256x14x14 -> 256 (2.6) 43 / 40, 16 x 512x32x32 -> 512 (1.7) 37 / 37.
        const bool can = pack_algo == TNNS_PACK_AUTO && tnns_fused_supported(w, g, d_x, layout) &&
                         (reinterpret_cast<uintptr_t>(d_workspace) & 127) == 0 &&
                         tnns_fused_workspace_bytes(g.N, g.C, g.H, g.W) <= workspace_bytes;
        if (gemm_algo == TNNS_GEMM_F4_FUSED && !can)
            return tnns_fail(TNNS_ERR_UNSUPPORTED, "layer, layout, workspace size or alignment outside the fused quantise + GEMM route");
        if (can && (gemm_algo == TNNS_GEMM_F4_FUSED || tnns_cuda_conv_fused_preferred(ctx, w, s, d_x, layout)))
            return conv_fused_impl(ctx, w, d_x, d_thr, d_y, nullptr, nullptr, 1, d_workspace, workspace_bytes, s, alpha, 0, stream, layout);
    }
    const bool auto_route = pack_algo == TNNS_PACK_AUTO && (gemm_algo == TNNS_GEMM_AUTO || gemm_algo == TNNS_GEMM_F4_TC);
    if (auto_route && tnns_im2col_supported(w, g) && tnns_e2m1_image_bytes(g.N, g.C, g.H, g.W) <= workspace_bytes) {
        if (reinterpret_cast<uintptr_t>(d_workspace) & 31) return tnns_fail(TNNS_ERR_INVALID, "workspace must be 32-byte aligned");
        rc = tnns_launch_quantise(ctx, true, d_x, d_thr, d_workspace, g.N, g.C, g.H, g.W, layout, (cudaStream_t)stream, TNNS_IMG_E2M1);
        if (rc) return rc;
        return tnns_launch_gemm_im2col(ctx, w, d_workspace, d_y, g, alpha, layout, (cudaStream_t)stream);
    }
    const size_t image_bytes = tnns_packed_image_bytes(type_act_ternary(w->type), g.N, g.C, g.H, g.W);
    if (pack_algo == TNNS_PACK_AUTO && (gemm_algo == TNNS_GEMM_AUTO || gemm_algo == TNNS_GEMM_F4_TC) && w->d_f4 && w->d_jtab &&
        w->Kp < 65536 && image_bytes <= workspace_bytes) {
        if (reinterpret_cast<uintptr_t>(d_workspace) & 31) return tnns_fail(TNNS_ERR_INVALID, "workspace must be 32-byte aligned");
        rc = tnns_launch_quantise(ctx, type_act_ternary(w->type), d_x, d_thr, d_workspace, g.N, g.C, g.H, g.W, layout, (cudaStream_t)stream);
        if (rc) return rc;
        return tnns_launch_gemm_tc(ctx, w, d_workspace, d_y, (long long)g.N * g.OH * g.OW, g.OH * g.OW, alpha, layout, true,
                                   (cudaStream_t)stream, nullptr, nullptr, 1, &g);
    }
    // the explicit route materialises the im2row matrix
    const size_t need = tnns_packed_bytes(w->type, s);
    if (workspace_bytes < need)
        return tnns_fail(TNNS_ERR_INVALID, "workspace of %zu bytes; the packed im2row matrix this route writes needs %zu", workspace_bytes, need);
    rc = tnns_cuda_pack(ctx, type_act_ternary(w->type), d_x, d_thr, (int64_t*)d_workspace, s, layout, pack_algo, stream);
    if (rc) return rc;
    return tnns_cuda_gemm(ctx, w, (const int64_t*)d_workspace, d_y, g.N, g.OH, g.OW, alpha, layout, gemm_algo, stream);
}

int tnns_cuda_conv(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y,
                   const tnns_shape_t* s, float alpha, int layout, int pack_algo, int gemm_algo, void* stream) {
    if (!ctx || !w) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    TNNS_ENTER(ctx, w);
    // room for the im2row matrix (explicit route) and, where the layer qualifies, for the 4-bit
    // image of the copy-engine route, which is larger than the matrix for 1x1 kernels
    size_t need = std::max<size_t>(tnns_packed_bytes(w->type, s), 16);
    if (tnns_im2col_supported(w, g)) need = std::max(need, tnns_fused_workspace_bytes(g.N, g.C, g.H, g.W));
    if (tnns_slab_supported(ctx, w, g, false)) need = std::max(need, tnns_slab_workspace_bytes(g.N, g.C, g.H, g.W, g.PH, g.PW));
    if (tnns_cuda_dense_supported(ctx, w, s)) need = std::max(need, tnns_dense_workspace_bytes(s));
    if (ctx->workspace_bytes < need) {
        // earlier launches may still read the old workspace
        TNNS_CUDA_TRY(cudaDeviceSynchronize());
        if (ctx->workspace) cudaFree(ctx->workspace);
        ctx->workspace = nullptr;
        ctx->workspace_bytes = 0;
        TNNS_CUDA_TRY(cudaMalloc(&ctx->workspace, need));
        ctx->workspace_bytes = need;
    }
    return tnns_cuda_conv_ws(ctx, w, d_x, d_thr, d_y, ctx->workspace, ctx->workspace_bytes, s, alpha, layout, pack_algo, gemm_algo,
                             stream);
}

// --- host-buffer layer: sliced, copy/compute overlapped -------------------------------------------
// Grows a pair of equally sized device buffers; on failure both are released and the
// recorded size drops to zero, so a later call starts from a clean state.
static int grow_pair(void* p[2], size_t* have, size_t need) {
    if (*have >= need && p[0] && p[1]) return TNNS_OK;
    for (int i = 0; i < 2; i++) {
        if (p[i]) cudaFree(p[i]);
        p[i] = nullptr;
    }
    *have = 0;
    for (int i = 0; i < 2; i++) {
        cudaError_t e = cudaMalloc(&p[i], need);
        if (e != cudaSuccess) {
            if (p[0]) cudaFree(p[0]);
            p[0] = p[1] = nullptr;
            return tnns_fail(e == cudaErrorMemoryAllocation ? TNNS_ERR_NOMEM : TNNS_ERR_CUDA, "staging allocation of %zu bytes failed: %s",
                             need, cudaGetErrorString(e));
        }
    }
    *have = need;
    return TNNS_OK;
}

int tnns_cuda_conv_host(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* h_x, const float* h_thr, float* h_y,
                        const tnns_shape_t* s, float alpha, int layout) {
    if (!ctx || !w || !h_x || !h_thr || !h_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    TnnsGeom g;
    int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    if (s->KN != w->KN || s->C != w->C || s->KH != w->KH || s->KW != w->KW)
        return tnns_fail(TNNS_ERR_INVALID, "shape does not match the uploaded weights");
    TNNS_ENTER(ctx, w);
    if (g.N == 0) return TNNS_OK;

    // (Letting the one-launch kernel work on page-locked host buffers directly -- tensor copies and
    // epilogue stores over PCIe, no staging -- measured slower than the copy engines: 4.2 ms against
    // 3.2 ms on the large layer; the SMs' reads of host memory reach about 32 GB/s.)
    // slice the batch so that copies and kernels overlap; nb = images of a full slice
    const int nb = std::max(1, (g.N + 7) / 8);
    const size_t in_img = (size_t)g.C * g.H * g.W * sizeof(float);
    const size_t out_img = (size_t)g.KN * g.OH * g.OW * sizeof(float);
    tnns_shape_t ss = *s;
    ss.N = nb;
    size_t pack_slice = std::max<size_t>(tnns_packed_bytes(w->type, &ss), 16);
    if (tnns_im2col_supported(w, g)) pack_slice = std::max(pack_slice, tnns_fused_workspace_bytes(nb, g.C, g.H, g.W));

    // staging buffers are shared by both slots' sizes; growing needs the device idle
    bool must_grow = ctx->stage_in_bytes < in_img * nb || ctx->stage_out_bytes < out_img * nb ||
                     ctx->stage_pack_bytes < pack_slice || ctx->stage_thr_count < (size_t)g.N;
    if (must_grow) {
        TNNS_CUDA_TRY(cudaDeviceSynchronize());
        if ((rc = grow_pair(ctx->stage_in, &ctx->stage_in_bytes, in_img * nb))) return rc;
        if ((rc = grow_pair(ctx->stage_out, &ctx->stage_out_bytes, out_img * nb))) return rc;
        if ((rc = grow_pair(ctx->stage_pack, &ctx->stage_pack_bytes, pack_slice))) return rc;
        if (ctx->stage_thr_count < (size_t)g.N) {
            if (ctx->stage_thr) cudaFree(ctx->stage_thr);
            ctx->stage_thr = nullptr;
            ctx->stage_thr_count = 0;
            TNNS_CUDA_TRY(cudaMalloc(&ctx->stage_thr, (size_t)g.N * sizeof(float)));
            ctx->stage_thr_count = (size_t)g.N;
        }
    }

    // Slice plan: about eight slices of nb images, the first and the last of them cut in two (a
    // quarter, then the rest): the download stream trails the upload stream by one slice, so small
    // slices at both ends shorten what the slicing adds to the transfer time.  Slices larger than
    // nb in the middle measured slower (the download stream then idles while a large slice
    // uploads: 3.35 ms against 3.19 ms on the large layer), and so did sixteen equal slices (every
    // slice costs event waits on three streams).
    std::vector<int> plan;
    {
        const int quarter = std::max(1, nb / 4);
        int left = g.N;
        const bool taper = nb >= 2 && g.N >= 3 * nb;
        if (taper) { plan.push_back(quarter); plan.push_back(nb - quarter); left -= 2 * nb; }
        while (left > 0) { plan.push_back(std::min(nb, left)); left -= plan.back(); }
        if (taper) { plan.push_back(nb - quarter); plan.push_back(quarter); }
    }

    // Every failure inside the loop leaves through one exit that drains the three streams first:
    // copies and kernels of earlier slices are still queued, and the caller may free h_x / h_y (the
    // drop-in tnns_conv frees its output buffer) as soon as this function returns.
    cudaError_t e = cudaMemcpyAsync(ctx->stage_thr, h_thr, (size_t)g.N * sizeof(float), cudaMemcpyHostToDevice, ctx->s_copy_in);
    rc = TNNS_OK;
    int n0 = 0;
    for (int k = 0; k < (int)plan.size() && e == cudaSuccess && rc == TNNS_OK; n0 += plan[k], k++) {
        const int slot = k & 1;
        const int cnt = plan[k];
        ss.N = cnt;
        if (k >= 2) e = cudaStreamWaitEvent(ctx->s_copy_in, ctx->ev_done[slot], 0);  // kernels of slice k-2 done with stage_in
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(ctx->stage_in[slot], (const char*)h_x + (size_t)n0 * in_img, in_img * cnt, cudaMemcpyHostToDevice, ctx->s_copy_in);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->ev_in[slot], ctx->s_copy_in);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->s_compute, ctx->ev_in[slot], 0);
        if (e == cudaSuccess && k >= 2) e = cudaStreamWaitEvent(ctx->s_compute, ctx->ev_out[slot], 0);  // download of slice k-2 done with stage_out
        if (e != cudaSuccess) break;
        rc = tnns_cuda_conv_ws(ctx, w, (const float*)ctx->stage_in[slot], ctx->stage_thr + n0, (float*)ctx->stage_out[slot],
                               ctx->stage_pack[slot], ctx->stage_pack_bytes, &ss, alpha, layout, TNNS_PACK_AUTO, TNNS_GEMM_AUTO,
                               ctx->s_compute);
        if (rc) break;
        e = cudaEventRecord(ctx->ev_done[slot], ctx->s_compute);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->s_copy_out, ctx->ev_done[slot], 0);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync((char*)h_y + (size_t)n0 * out_img, ctx->stage_out[slot], out_img * cnt, cudaMemcpyDeviceToHost, ctx->s_copy_out);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->ev_out[slot], ctx->s_copy_out);
    }
    const cudaError_t s0 = cudaStreamSynchronize(ctx->s_copy_out), s1 = cudaStreamSynchronize(ctx->s_compute),
                      s2 = cudaStreamSynchronize(ctx->s_copy_in);
    if (rc) return rc;  // tnns_cuda_conv_ws recorded its own error
    if (e == cudaSuccess) e = s0 != cudaSuccess ? s0 : (s1 != cudaSuccess ? s1 : s2);
    if (e != cudaSuccess)
        return tnns_fail(e == cudaErrorMemoryAllocation ? TNNS_ERR_NOMEM : TNNS_ERR_CUDA, "host-buffer layer failed: %s", cudaGetErrorString(e));
    return TNNS_OK;
}

}  // extern "C"
