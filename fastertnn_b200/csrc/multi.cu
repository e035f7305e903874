// One host batch over several GPUs behind one call.
//
// Rows of the im2row matrix are independent (the reference's GEMM walks them one by one with no
// state between rows, include/tnns/mm.h:22-31) and an image's rows depend on that image alone, so a
// layer is partitioned by image index: shard g of G owns a contiguous range of images, which is a
// contiguous slice of the NCHW / NHWC input and of the output.  The packed weights are uploaded to
// every device once; the data path needs no exchange between devices.
//
// tnns_shard_run is the host-side engine: one host thread per shard, all released together by a
// start barrier, every shard's status collected.  A shard that fails (or returns early) does not
// stop the others: the call completes them and reports which shards are missing.
// tnns_cuda_multi_* puts contexts, weights and the host-buffer layer on top of it.
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include "internal.h"

void tnns_add_launches(unsigned long long n);  // api.cu: credits kernels launched by worker threads to the caller

namespace {

struct StartBarrier {
    std::mutex m;
    std::condition_variable cv;
    int waiting = 0, total = 0;
    void arrive_and_wait() {
        std::unique_lock<std::mutex> lock(m);
        if (++waiting == total) cv.notify_all();
        else cv.wait(lock, [&] { return waiting == total; });
    }
};

struct ShardResult {
    int status = TNNS_OK;
    unsigned long long launches = 0;
    char detail[256] = "";
};

}  // namespace

struct tnns_cuda_multi {
    std::vector<int> devices;
    std::vector<tnns_cuda_ctx*> ctx;
};

struct tnns_cuda_multi_weights {
    std::vector<tnns_cuda_weights*> w;
    int type, KN, C, KH, KW;
};

extern "C" {

void tnns_shard_range(int N, int shard, int shards, int* n0, int* n1) {
    int a = 0, b = 0;
    if (N > 0 && shards > 0 && shard >= 0 && shard < shards) {
        const int base = N / shards, extra = N % shards;  // the first N % shards shards own one image more
        a = shard * base + (shard < extra ? shard : extra);
        b = a + base + (shard < extra ? 1 : 0);
    }
    if (n0) *n0 = a;
    if (n1) *n1 = b;
}

int tnns_shard_run(int shards, int N, tnns_shard_fn fn, void* arg, int* shard_status) {
    if (shards <= 0 || N < 0 || !fn) return tnns_fail(TNNS_ERR_INVALID, "shard run: %d shards, %d images, callback %s", shards, N, fn ? "set" : "NULL");
    std::vector<ShardResult> res(shards);
    StartBarrier start;
    start.total = shards;
    auto body = [&](int g) {
        int n0, n1;
        tnns_shard_range(N, g, shards, &n0, &n1);
        const unsigned long long before = tnns_cuda_launch_count();
        start.arrive_and_wait();  // no shard begins before every host thread is up
        const int rc = fn(g, shards, n0, n1, arg);
        res[g].status = rc;
        res[g].launches = tnns_cuda_launch_count() - before;
        if (rc != TNNS_OK) {
            // the error text lives in this thread's storage and dies with the thread
            const char* d = tnns_cuda_last_error() == rc ? tnns_cuda_error_detail() : "";
            snprintf(res[g].detail, sizeof(res[g].detail), "%s", d);
        }
    };
    std::vector<std::thread> threads;
    threads.reserve(shards);
    int spawned = 0;
    try {
        for (int g = 1; g < shards; g++, spawned++) threads.emplace_back(body, g);
    } catch (...) {
        // a host thread could not be started: the barrier must still open for those that run
        std::lock_guard<std::mutex> lock(start.m);
        start.total = spawned + 1;
        for (int g = spawned + 1; g < shards; g++) res[g].status = TNNS_ERR_NOMEM;
        start.cv.notify_all();
    }
    body(0);  // the calling thread is shard 0
    for (auto& t : threads) t.join();
    int first = -1, failed = 0;
    for (int g = 0; g < shards; g++) {
        if (shard_status) shard_status[g] = res[g].status;
        if (g > 0) tnns_add_launches(res[g].launches);
        if (res[g].status != TNNS_OK) {
            failed++;
            if (first < 0) first = g;
        }
    }
    if (first < 0) return TNNS_OK;
    char list[160] = "";
    size_t used = 0;
    for (int g = 0; g < shards && used + 8 < sizeof(list); g++)
        if (res[g].status != TNNS_OK) used += snprintf(list + used, sizeof(list) - used, "%s%d", used ? "," : "", g);
    return tnns_fail(res[first].status, "%d of %d shards failed (shards %s; the others completed); shard %d: %s", failed, shards, list, first,
                     res[first].detail[0] ? res[first].detail : tnns_cuda_strerror(res[first].status));
}

int tnns_cuda_multi_create(const int* devices, int count, tnns_cuda_multi** out) {
    if (!out) return tnns_fail(TNNS_ERR_INVALID, "out-pointer is NULL");
    *out = nullptr;
    if (!devices || count <= 0 || count > 64) return tnns_fail(TNNS_ERR_INVALID, "device list of %d entries", count);
    for (int i = 0; i < count; i++)
        for (int j = 0; j < i; j++)
            if (devices[i] == devices[j]) return tnns_fail(TNNS_ERR_INVALID, "device %d listed twice", devices[i]);
    tnns_cuda_multi* m = new (std::nothrow) tnns_cuda_multi();
    if (!m) return tnns_fail(TNNS_ERR_NOMEM, "host allocation failed");
    for (int i = 0; i < count; i++) {
        tnns_cuda_ctx* c = nullptr;
        const int rc = tnns_cuda_create(devices[i], &c);
        if (rc != TNNS_OK) {
            tnns_cuda_multi_destroy(m);
            return rc;
        }
        m->devices.push_back(devices[i]);
        m->ctx.push_back(c);
    }
    *out = m;
    return TNNS_OK;
}

void tnns_cuda_multi_destroy(tnns_cuda_multi* m) {
    if (!m) return;
    for (tnns_cuda_ctx* c : m->ctx) tnns_cuda_destroy(c);
    delete m;
}

int tnns_cuda_multi_device_count(const tnns_cuda_multi* m) { return m ? (int)m->ctx.size() : 0; }

tnns_cuda_ctx* tnns_cuda_multi_context(const tnns_cuda_multi* m, int index) {
    return (m && index >= 0 && index < (int)m->ctx.size()) ? m->ctx[index] : nullptr;
}

int tnns_cuda_multi_upload_weights(tnns_cuda_multi* m, int type, const int64_t* packed_host, int KN, int C, int KH, int KW,
                                   tnns_cuda_multi_weights** out) {
    if (!m || !packed_host || !out) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    *out = nullptr;
    tnns_cuda_multi_weights* mw = new (std::nothrow) tnns_cuda_multi_weights();
    if (!mw) return tnns_fail(TNNS_ERR_NOMEM, "host allocation failed");
    mw->type = type; mw->KN = KN; mw->C = C; mw->KH = KH; mw->KW = KW;
    for (tnns_cuda_ctx* c : m->ctx) {
        tnns_cuda_weights* w = nullptr;
        const int rc = tnns_cuda_upload_weights(c, type, packed_host, KN, C, KH, KW, &w);
        if (rc != TNNS_OK) {
            tnns_cuda_multi_free_weights(m, mw);
            return rc;
        }
        mw->w.push_back(w);
    }
    *out = mw;
    return TNNS_OK;
}

void tnns_cuda_multi_free_weights(tnns_cuda_multi* m, tnns_cuda_multi_weights* mw) {
    if (!mw) return;
    for (size_t i = 0; i < mw->w.size(); i++) tnns_cuda_free_weights(m && i < m->ctx.size() ? m->ctx[i] : nullptr, mw->w[i]);
    delete mw;
}

}  // extern "C"

namespace {
struct ConvHostJob {
    const tnns_cuda_multi* m;
    const tnns_cuda_multi_weights* w;
    const float* h_x;
    const float* h_thr;
    float* h_y;
    tnns_shape_t s;
    size_t in_img, out_img;  // floats per image
    float alpha;
    int layout;
};

int conv_host_shard(int shard, int, int n0, int n1, void* arg) {
    const ConvHostJob* j = static_cast<const ConvHostJob*>(arg);
    if (n1 <= n0) return TNNS_OK;
    tnns_shape_t s = j->s;
    s.N = n1 - n0;
    return tnns_cuda_conv_host(j->m->ctx[shard], j->w->w[shard], j->h_x + (size_t)n0 * j->in_img, j->h_thr + n0, j->h_y + (size_t)n0 * j->out_img,
                               &s, j->alpha, j->layout);
}
}  // namespace

extern "C" int tnns_cuda_multi_conv_host(tnns_cuda_multi* m, const tnns_cuda_multi_weights* w, const float* h_x, const float* h_thr, float* h_y,
                                         const tnns_shape_t* s, float alpha, int layout, int* shard_status) {
    if (!m || !w || !h_x || !h_thr || !h_y) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (w->w.size() != m->ctx.size()) return tnns_fail(TNNS_ERR_INVALID, "weights were uploaded to %zu devices, the group has %zu", w->w.size(), m->ctx.size());
    TnnsGeom g;
    const int rc = tnns_make_geom(s, &g);
    if (rc) return rc;
    ConvHostJob job;
    job.m = m; job.w = w; job.h_x = h_x; job.h_thr = h_thr; job.h_y = h_y; job.s = *s;
    job.in_img = (size_t)g.C * g.H * g.W;
    job.out_img = (size_t)g.KN * g.OH * g.OW;
    job.alpha = alpha;
    job.layout = layout;
    return tnns_shard_run((int)m->ctx.size(), g.N, conv_host_shard, &job, shard_status);
}
