// ggml backend plugin for NVIDIA B200 (sm_100a).
//
// Implements the five interface tables of ggml/src/ggml-backend-impl.h (reg :191-201, device :137-179,
// buffer type :17-29, buffer :41-58, backend :87-117) and exports ggml_backend_init/ggml_backend_score
// (:215-218), so that an unmodified whisper.cpp picks it up through ggml_backend_load() and runs
// whisper_encode / whisper_decode / whisper_full on it.  Every node of the whisper graphs is executed
// by a kernel of libb200_kernels.so (include/b200_whisper.h); supports_op is exactly the set of nodes
// graph_compute can run, there is no host fallback inside this file.
#include "ggml.h"
#include "ggml-backend.h"
#include "ggml-backend-impl.h"
#include "b200_whisper.h"

#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>
#include <string>
#include <unordered_map>
#include <vector>

#define B200_MAX_DEVICES 16

static bool cuda_ok(cudaError_t e, const char * what) {
    if (e == cudaSuccess) return true;
    fprintf(stderr, "ggml-b200: %s failed: %s\n", what, cudaGetErrorString(e));
    return false;
}

static bool is_quant(enum ggml_type t) { return t == GGML_TYPE_Q5_0 || t == GGML_TYPE_Q8_0; }

// The buffer interface has no way to report a failed copy (set_tensor / get_tensor return void).  A failure is logged,
// remembered, and the next graph_compute on that device returns GGML_STATUS_FAILED instead of computing on bad data;
// the process is never aborted for it.
static std::atomic<int> g_sticky_error[16];
static void note_buffer_error(int device, const char * what) {
    fprintf(stderr, "ggml-b200: %s failed on device %d; the next graph_compute on it reports GGML_STATUS_FAILED\n", what, device);
    if (device >= 0 && device < 16) g_sticky_error[device] = 1;
}
extern "C" int b200_stat_sticky_error(int device) { return device >= 0 && device < 16 ? g_sticky_error[device].load() : 0; }

// ---------------------------------------------------------------------------------------------
// statistics (exposed through get_proc_address for tests and the benchmark)
// ---------------------------------------------------------------------------------------------
static std::atomic<int64_t> g_nodes_computed{0};    // non-view nodes executed by this backend
static std::atomic<int64_t> g_graphs_computed{0};
static std::atomic<int64_t> g_h2d_bytes{0};
static std::atomic<int64_t> g_d2h_bytes{0};
static std::atomic<int64_t> g_host_ns_compute{0};   // host time inside graph_compute (launching)
static std::atomic<int64_t> g_host_ns_sync{0};      // host time waiting in synchronize
static inline int64_t now_ns() { return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

// Optional per-operator timing (off by default): CUDA events recorded on the backend's own stream
// around every launch group, summed per class after the graph finishes.  Used by the benchmark for
// its roofline line; the extra event records and the sync make it unsuitable for throughput runs.
enum b200_timing_class { TC_MMQ_VEC = 0, TC_MMQ_GEMM, TC_MM_F16, TC_FATTN, TC_FATTN_DEC, TC_NORM, TC_BINARY, TC_SCALE, TC_GELU, TC_CPY,
                         TC_GET_ROWS, TC_IM2COL, TC_SOFT_MAX, TC_CONCAT, TC_COUNT };
static const char * const g_tc_names[TC_COUNT] = { "mul_mat_vec_q", "mul_mat_q", "mul_mat_f16", "flash_attn_ext", "flash_attn_decode", "norm", "binary",
                                                   "scale", "gelu", "cpy", "get_rows", "im2col", "soft_max", "concat" };
static std::atomic<int> g_timing_on{0};
static std::mutex       g_timing_mu;
static double  g_tc_ms[TC_COUNT];
static double  g_tc_work[TC_COUNT];     // algorithmic bytes (memory-bound classes) or FLOPs (mul_mat_q, mul_mat_f16, flash_attn_ext)
static int64_t g_tc_count[TC_COUNT];

extern "C" {
void b200_timing_enable(int on) { g_timing_on = on; }
void b200_timing_reset(void) {
    std::lock_guard<std::mutex> lk(g_timing_mu);
    for (int i = 0; i < TC_COUNT; ++i) { g_tc_ms[i] = 0; g_tc_work[i] = 0; g_tc_count[i] = 0; }
}
int b200_timing_classes(void) { return TC_COUNT; }
const char * b200_timing_name(int c) { return c >= 0 && c < TC_COUNT ? g_tc_names[c] : ""; }
void b200_timing_get(int c, int64_t * count, double * ms, double * work) {
    std::lock_guard<std::mutex> lk(g_timing_mu);
    *count = g_tc_count[c]; *ms = g_tc_ms[c]; *work = g_tc_work[c];
}
int64_t b200_stat_nodes(void)   { return g_nodes_computed.load(); }
int64_t b200_stat_graphs(void)  { return g_graphs_computed.load(); }
int64_t b200_stat_h2d(void)     { return g_h2d_bytes.load(); }
int64_t b200_stat_d2h(void)     { return g_d2h_bytes.load(); }
int64_t b200_stat_host_ns_compute(void) { return g_host_ns_compute.load(); }
int64_t b200_stat_host_ns_sync(void)    { return g_host_ns_sync.load(); }
}

// Logits side output (off by default; switched through get_proc_address, see b200_whisper.h)
static std::atomic<int> g_topk_k{0};
static std::atomic<int> g_skip_logits_readback{0};
static std::mutex g_logits_mu;
static std::unordered_map<const void *, int> g_logits_ptrs;     // device addresses of logits tensors seen by graph_compute

// ---------------------------------------------------------------------------------------------
// buffer
// ---------------------------------------------------------------------------------------------
struct b200_buffer_ctx {
    int    device;
    void * base;
};

// Tensor-pipe operands of quantised weight tensors (b200_mma_pack_weights), made on first use by a many-column
// product and kept until the weight's buffer is written again or freed.  Key: device address of the tensor data.
struct mma_weights { void * h; float * d; };
static std::mutex g_mma_mu;
static std::unordered_map<const void *, mma_weights> g_mma_cache;

static void mma_cache_drop_range(const void * base, size_t size) {
    std::lock_guard<std::mutex> lk(g_mma_mu);
    for (auto it = g_mma_cache.begin(); it != g_mma_cache.end();) {
        const char * p = (const char *) it->first;
        if (p >= (const char *) base && p < (const char *) base + size) {
            cudaFree(it->second.h);
            it = g_mma_cache.erase(it);
        } else {
            ++it;
        }
    }
}

static void b200_buffer_free(ggml_backend_buffer_t buffer) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    mma_cache_drop_range(ctx->base, buffer->size);
    cudaFree(ctx->base);
    delete ctx;
}

static void * b200_buffer_get_base(ggml_backend_buffer_t buffer) {
    return ((b200_buffer_ctx *) buffer->context)->base;
}

static void b200_buffer_memset_tensor(ggml_backend_buffer_t buffer, struct ggml_tensor * tensor, uint8_t value, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    if (is_quant(tensor->type)) mma_cache_drop_range(tensor->data, 1);
    cuda_ok(cudaMemsetAsync((char *) tensor->data + offset, value, size, cudaStreamPerThread), "memset_tensor");
    cuda_ok(cudaStreamSynchronize(cudaStreamPerThread), "memset_tensor sync");
}

// Block-quantised tensors live in device memory as planes (see b200_whisper.h); set/get translate on the device: the raw
// block bytes cross the bus once, in one copy, into a staging buffer, and one launch scatters them into the planes
// (get_tensor: the reverse).  The staging buffer is per device, grows on demand and is shared under a lock - weights are
// written once, at model load, by one thread at a time.
struct staging_buf { std::mutex mu; void * p = nullptr; size_t size = 0; };
static staging_buf g_staging[B200_MAX_DEVICES];

static void * staging_reserve(staging_buf & sb, size_t size) {
    if (sb.size >= size) return sb.p;
    if (sb.p) { cudaFree(sb.p); sb.p = nullptr; sb.size = 0; }
    const size_t want = (size + ((size_t) 1 << 22) - 1) & ~(((size_t) 1 << 22) - 1);
    if (cudaMalloc(&sb.p, want) != cudaSuccess) { cudaGetLastError(); sb.p = nullptr; return nullptr; }
    sb.size = want;
    return sb.p;
}

// Waits for a stream.  With one host thread per whisper_state there can be more threads than cores, and a thread that
// spins in cudaStreamSynchronize then takes its core away from the threads that are launching work: in that case the
// wait sleeps on a blocking-sync event (one per host thread and device, never destroyed).  With few states the spinning
// wait is kept: waking a sleeping thread costs tens of microseconds, several times per decoder step.
static int live_backends(int device);
static cudaError_t stream_wait_blocking(cudaStream_t st) {
    static const int force = getenv("GGML_B200_SPIN_SYNC") ? atoi(getenv("GGML_B200_SPIN_SYNC")) : -1;      // 1 spin, 0 sleep
    // cores this process can count on: the host's, shared with the other ranks of a one-process-per-GPU launch
    static const int cores = [] {
        int c = (int) std::thread::hardware_concurrency();
        const char * lws = getenv("LOCAL_WORLD_SIZE");
        const int ranks = lws ? atoi(lws) : 1;
        return ranks > 1 ? c / ranks : c;
    }();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= B200_MAX_DEVICES) return cudaStreamSynchronize(st);
    const bool spin = force >= 0 ? force != 0 : 2 * live_backends(dev) <= (cores > 0 ? cores : 8);
    if (spin) return cudaStreamSynchronize(st);
    thread_local cudaEvent_t ev[B200_MAX_DEVICES] = {};
    if (!ev[dev] && cudaEventCreateWithFlags(&ev[dev], cudaEventBlockingSync | cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        ev[dev] = nullptr;
        return cudaStreamSynchronize(st);
    }
    cudaError_t e = cudaEventRecord(ev[dev], st);
    if (e != cudaSuccess) return e;
    return cudaEventSynchronize(ev[dev]);
}

static void b200_buffer_set_tensor(ggml_backend_buffer_t buffer, struct ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    g_h2d_bytes += (int64_t) size;
    cudaStream_t st = cudaStreamPerThread;
    if (is_quant(tensor->type)) {
        mma_cache_drop_range(tensor->data, 1);
        const size_t  bs = ggml_type_size(tensor->type);
        const int64_t nb_total = (int64_t) (ggml_nbytes(tensor) / bs);
        if (tensor->view_src != nullptr || offset % bs != 0 || size % bs != 0) {
            note_buffer_error(ctx->device, "set_tensor on a view or a partial block of a block-quantised tensor");
            return;
        }
        const int64_t first = (int64_t) (offset / bs), count = (int64_t) (size / bs);
        staging_buf & sb = g_staging[ctx->device];
        std::lock_guard<std::mutex> lk(sb.mu);
        void * stage = staging_reserve(sb, size);
        bool ok = stage != nullptr;
        ok = ok && cuda_ok(cudaMemcpyAsync(stage, data, size, cudaMemcpyHostToDevice, st), "set_tensor upload");
        ok = ok && b200_blocks_to_planes_device((int) tensor->type, stage, tensor->data, nb_total, first, count, (void *) st) == 0;
        ok = cuda_ok(stream_wait_blocking(st), "set_tensor sync") && ok;
        if (!ok) note_buffer_error(ctx->device, "set_tensor");
        return;
    }
    bool ok = cuda_ok(cudaMemcpyAsync((char *) tensor->data + offset, data, size, cudaMemcpyHostToDevice, st), "set_tensor");
    ok = ok && cuda_ok(stream_wait_blocking(st), "set_tensor sync");
    if (!ok) note_buffer_error(ctx->device, "set_tensor");
}

static void b200_buffer_get_tensor(ggml_backend_buffer_t buffer, const struct ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    if (g_skip_logits_readback.load(std::memory_order_relaxed)) {      // the caller samples from the side output only
        std::lock_guard<std::mutex> lk(g_logits_mu);
        if (g_logits_ptrs.count(tensor->data)) return;
    }
    cudaSetDevice(ctx->device);
    g_d2h_bytes += (int64_t) size;
    cudaStream_t st = cudaStreamPerThread;
    if (is_quant(tensor->type)) {
        const size_t  bs = ggml_type_size(tensor->type);
        const int64_t nb_total = (int64_t) (ggml_nbytes(tensor) / bs);
        if (tensor->view_src != nullptr || offset % bs != 0 || size % bs != 0) {
            note_buffer_error(ctx->device, "get_tensor on a view or a partial block of a block-quantised tensor");
            memset(data, 0, size);
            return;
        }
        const int64_t first = (int64_t) (offset / bs), count = (int64_t) (size / bs);
        staging_buf & sb = g_staging[ctx->device];
        std::lock_guard<std::mutex> lk(sb.mu);
        void * stage = staging_reserve(sb, size);
        bool ok = stage != nullptr;
        ok = ok && b200_planes_to_blocks_device((int) tensor->type, tensor->data, stage, nb_total, first, count, (void *) st) == 0;
        ok = ok && cuda_ok(cudaMemcpyAsync(data, stage, size, cudaMemcpyDeviceToHost, st), "get_tensor download");
        ok = cuda_ok(stream_wait_blocking(st), "get_tensor sync") && ok;
        if (!ok) { note_buffer_error(ctx->device, "get_tensor"); memset(data, 0, size); }
        return;
    }
    bool ok = cuda_ok(cudaMemcpyAsync(data, (const char *) tensor->data + offset, size, cudaMemcpyDeviceToHost, st), "get_tensor");
    ok = ok && cuda_ok(stream_wait_blocking(st), "get_tensor sync");
    if (!ok) { note_buffer_error(ctx->device, "get_tensor"); memset(data, 0, size); }
}

static void b200_buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    mma_cache_drop_range(ctx->base, buffer->size);
    cuda_ok(cudaMemsetAsync(ctx->base, value, buffer->size, cudaStreamPerThread), "clear");
    cuda_ok(cudaStreamSynchronize(cudaStreamPerThread), "clear sync");
}

static const struct ggml_backend_buffer_i b200_buffer_iface = {
    /* .free_buffer   = */ b200_buffer_free,
    /* .get_base      = */ b200_buffer_get_base,
    /* .init_tensor   = */ nullptr,
    /* .memset_tensor = */ b200_buffer_memset_tensor,
    /* .set_tensor    = */ b200_buffer_set_tensor,
    /* .get_tensor    = */ b200_buffer_get_tensor,
    /* .cpy_tensor    = */ nullptr,
    /* .clear         = */ b200_buffer_clear,
    /* .reset         = */ nullptr,
};

// ---------------------------------------------------------------------------------------------
// buffer type (one per device)
// ---------------------------------------------------------------------------------------------
struct b200_device_ctx {
    int         device;
    std::string name;
    std::string description;
    struct ggml_backend_buffer_type buft;
    std::string buft_name;
};

static const char * b200_buft_get_name(ggml_backend_buffer_type_t buft) {
    return ((b200_device_ctx *) buft->context)->buft_name.c_str();
}

static ggml_backend_buffer_t b200_buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    b200_device_ctx * dctx = (b200_device_ctx *) buft->context;
    if (cudaSetDevice(dctx->device) != cudaSuccess) return nullptr;
    void * base = nullptr;
    const size_t alloc = size > 0 ? size : 1;
    cudaError_t e = cudaMalloc(&base, alloc);
    if (e != cudaSuccess) {
        cudaGetLastError();
        fprintf(stderr, "ggml-b200: allocating %.2f MiB on device %d failed: %s\n", alloc / 1024.0 / 1024.0, dctx->device, cudaGetErrorString(e));
        return nullptr;
    }
    b200_buffer_ctx * ctx = new b200_buffer_ctx{dctx->device, base};
    return ggml_backend_buffer_init(buft, b200_buffer_iface, ctx, size);
}

static size_t b200_buft_get_alignment(ggml_backend_buffer_type_t) { return 256; }

static bool b200_buft_is_host(ggml_backend_buffer_type_t) { return false; }

// ---------------------------------------------------------------------------------------------
// backend (stream)
// ---------------------------------------------------------------------------------------------
struct b200_backend_ctx {
    int          device;
    cudaStream_t stream;
    void *       scratch      = nullptr;   // Q8_0-quantised activations of the current GEMM
    size_t       scratch_size = 0;
    std::string  name;
    std::vector<cudaEvent_t> events;       // timing mode only
    std::atomic<int64_t> last_decode_ns{0};   // when this instance last submitted a decode-step graph
    // quantised activation columns of the decode path (up to COLQ_MAX_COLS columns of up to COLQ_MAX_K values)
    void *       colq = nullptr;
    std::vector<const float *> colq_ptrs;    // columns currently held in colq ...
    int64_t      colq_K = 0;
    int64_t      colq_seq = -2;              // ... written (or reused) by the item with this sequence number
    std::atomic<int64_t> served_ns{0};       // when a leader last enqueued a step for this instance (0: not in a batch)
    cudaEvent_t  sync_event = nullptr;       // blocking-sync event: waiting threads sleep instead of spinning on a core
    int64_t      item_seq = 0;
    // side output of the last decoder graph: top-k / max / log-sum-exp of up to 8 logits rows (b200_topk_rows)
    b200_topk_result * topk = nullptr;       // 8 entries, as the kernels address them
    b200_topk_result * topk_host = nullptr;  // the same entries as the host reads them, when they live in mapped pinned host memory:
                                             // the kernel stores its few words per row straight into host memory and b200_last_topk
                                             // needs no copy and no wait of its own after the step has been synchronised
    int          topk_rows = 0;              // rows valid after the last decoder graph of this instance
    // what the scratch holds: the quantised form `qx_mode` of the activations at qx_data (N rows of K values, row stride
    // in bytes).  Products that follow each other on the same activations (Q, K and V of a layer; the 64 cross-attention
    // K/V products on the encoder output) quantise them once.  Cleared at the start of every graph and by every node
    // whose output overlaps the range.
    const void * qx_data = nullptr;
    int64_t      qx_N = 0, qx_K = 0, qx_stride = 0;
    int          qx_mode = 0;
};
static inline void qx_forget(b200_backend_ctx * ctx) { ctx->qx_data = nullptr; }
static inline void qx_note_write(b200_backend_ctx * ctx, const struct ggml_tensor * t) {
    if (!ctx->qx_data || !t || !t->data) return;
    const char * a0 = (const char *) ctx->qx_data, * a1 = a0 + ctx->qx_N * ctx->qx_stride;
    const char * b0 = (const char *) t->data,      * b1 = b0 + ggml_nbytes(t);
    if (b0 < a1 && a0 < b1) ctx->qx_data = nullptr;
}
#define COLQ_MAX_K 8192
#define COLQ_MAX_COLS 64
static inline int8_t * colq_q(b200_backend_ctx * ctx) { return (int8_t *) ctx->colq; }
static inline float *  colq_d(b200_backend_ctx * ctx) { return (float *) ((char *) ctx->colq + (size_t) COLQ_MAX_COLS * COLQ_MAX_K); }

static thread_local b200_backend_ctx * tl_last_decode_ctx = nullptr;

static void batcher_join(b200_backend_ctx * ctx);
static void batcher_leave(b200_backend_ctx * ctx);

static const char * b200_backend_get_name(ggml_backend_t backend) {
    return ((b200_backend_ctx *) backend->context)->name.c_str();
}

static void b200_backend_free(ggml_backend_t backend) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    batcher_leave(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->colq) cudaFree(ctx->colq);
    if (ctx->topk_host) cudaFreeHost(ctx->topk_host);
    else if (ctx->topk) cudaFree(ctx->topk);
    if (tl_last_decode_ctx == ctx) tl_last_decode_ctx = nullptr;
    if (ctx->sync_event) cudaEventDestroy(ctx->sync_event);
    for (cudaEvent_t e : ctx->events) cudaEventDestroy(e);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    delete backend;
}

static void b200_backend_synchronize(ggml_backend_t backend) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    cudaSetDevice(ctx->device);
    const int64_t t0 = now_ns();
    // With many whisper_states per GPU there are more host threads than cores; a spinning wait would take the cores
    // away from the threads that are launching work.
    if (ctx->sync_event && cudaEventRecord(ctx->sync_event, ctx->stream) == cudaSuccess) cuda_ok(cudaEventSynchronize(ctx->sync_event), "synchronize");
    else cuda_ok(cudaStreamSynchronize(ctx->stream), "synchronize");
    g_host_ns_sync += now_ns() - t0;
}

static bool ensure_scratch(b200_backend_ctx * ctx, size_t size) {
    if (ctx->scratch_size >= size) return true;
    qx_forget(ctx);
    if (ctx->scratch) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->scratch);
        ctx->scratch = nullptr;
        ctx->scratch_size = 0;
    }
    size = (size + (1u << 20) - 1) & ~((size_t) (1u << 20) - 1);
    if (cudaMalloc(&ctx->scratch, size) != cudaSuccess) { cudaGetLastError(); return false; }
    ctx->scratch_size = size;
    return true;
}

// Packed tensor-pipe copy of a quantised weight tensor; made once (pack kernel on this backend's stream, then a
// stream synchronise under the lock, so that every other stream may use it afterwards).  Null when device memory
// is short: the caller then keeps to the dp4a product.
static bool mma_weights_of(b200_backend_ctx * ctx, const struct ggml_tensor * w, int64_t nb_total, mma_weights * out) {
    std::lock_guard<std::mutex> lk(g_mma_mu);
    auto it = g_mma_cache.find(w->data);
    if (it != g_mma_cache.end()) { *out = it->second; return true; }
    const size_t h_bytes = (size_t) nb_total * 64, d_bytes = (size_t) nb_total * 4;
    void * p = nullptr;
    if (cudaMalloc(&p, h_bytes + d_bytes) != cudaSuccess) { cudaGetLastError(); return false; }
    mma_weights mw = { p, (float *) ((char *) p + h_bytes) };
    if (b200_mma_pack_weights((int) w->type, w->data, nb_total, mw.h, mw.d, (void *) ctx->stream) != 0 ||
        cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return false;
    }
    g_mma_cache[w->data] = mw;
    *out = mw;
    return true;
}

static inline bool qx_holds(const b200_backend_ctx * ctx, const void * x, int64_t N, int64_t K, int64_t stride, int mode) {
    static const bool reuse = getenv("GGML_B200_NO_QX_REUSE") == nullptr;
    return reuse && ctx->qx_data == x && ctx->qx_N == N && ctx->qx_K == K && ctx->qx_stride == stride && ctx->qx_mode == mode;
}
static inline void qx_set(b200_backend_ctx * ctx, const void * x, int64_t N, int64_t K, int64_t stride, int mode) {
    ctx->qx_data = x; ctx->qx_N = N; ctx->qx_K = K; ctx->qx_stride = stride; ctx->qx_mode = mode;
}

// Quantised weights x f32 activations for more than 8 columns: activations are quantised into this backend's
// scratch, then the tensor-pipe product (K a multiple of 128, 32 columns or more) or the dp4a product runs.
static int gemm_quant(b200_backend_ctx * ctx, const struct ggml_tensor * w, const float * x, int64_t x_stride_bytes, int64_t N,
                      void * dst, int64_t ldd, const b200_epilogue * ep) {
    static const bool use_mma = getenv("GGML_B200_NO_MMA") == nullptr;
    // the tcgen05 / tensor-memory product gives the same bits but measures slower than the mma.sync form (every
    // 32-block needs its own accumulator hand-off through tensor memory): opt-in
    static const bool use_tc  = getenv("GGML_B200_TC") != nullptr && atoi(getenv("GGML_B200_TC")) != 0;
    void * st = (void *) ctx->stream;
    const int64_t K = w->ne[0], M = w->ne[1];
    const int64_t nb_total = (int64_t) (ggml_nbytes(w) / ggml_type_size(w->type));
    if (use_tc) {
        // tcgen05 product: reads the weight planes as they are (no repacked copy), activations as int8 + scales
        const size_t q_bytes = (size_t) N * K, d_bytes = (size_t) N * (K / 32) * 4;
        const size_t q_pad = (q_bytes + 255) & ~(size_t) 255;
        if (!ensure_scratch(ctx, q_pad + d_bytes)) return (int) cudaErrorMemoryAllocation;
        int8_t * xq = (int8_t *) ctx->scratch;
        float *  xd = (float *) ((char *) ctx->scratch + q_pad);
        if (!qx_holds(ctx, x, N, K, x_stride_bytes, 1)) {
            int e = b200_quantize_q8_0(x, N, K, x_stride_bytes, xq, xd, st);
            if (e) return e;
            qx_set(ctx, x, N, K, x_stride_bytes, 1);
        }
        return b200_mul_mat_tc_ep((int) w->type, w->data, nb_total, M, K, xq, xd, N, dst, ldd, ep, st);
    }
    mma_weights mw;
    if (use_mma && N >= 32 && K % 128 == 0 && mma_weights_of(ctx, w, nb_total, &mw)) {
        const size_t h_bytes = (size_t) N * (K / 32) * 64, d_bytes = (size_t) N * (K / 32) * 4;
        if (!ensure_scratch(ctx, h_bytes + d_bytes)) return (int) cudaErrorMemoryAllocation;
        float * xd = (float *) ((char *) ctx->scratch + h_bytes);
        if (!qx_holds(ctx, x, N, K, x_stride_bytes, 2)) {
            int e = b200_mma_quantize(x, N, K, x_stride_bytes, ctx->scratch, xd, st);
            if (e) return e;
            qx_set(ctx, x, N, K, x_stride_bytes, 2);
        }
        return b200_mul_mat_mma_ep(mw.h, mw.d, M, K, ctx->scratch, xd, N, dst, ldd, ep, st);
    }
    const size_t q_bytes = (size_t) N * K, d_bytes = (size_t) N * (K / 32) * 4;
    const size_t q_pad = (q_bytes + 255) & ~(size_t) 255;
    if (!ensure_scratch(ctx, q_pad + d_bytes)) return (int) cudaErrorMemoryAllocation;
    int8_t * xq = (int8_t *) ctx->scratch;
    float *  xd = (float *) ((char *) ctx->scratch + q_pad);
    if (!qx_holds(ctx, x, N, K, x_stride_bytes, 1)) {
        int e = b200_quantize_q8_0(x, N, K, x_stride_bytes, xq, xd, st);
        if (e) return e;
        qx_set(ctx, x, N, K, x_stride_bytes, 1);
    }
    return b200_mul_mat_q_ep((int) w->type, w->data, nb_total, M, K, xq, xd, N, dst, ldd, ep, st);
}

static bool is_view_op(enum ggml_op op) {
    return op == GGML_OP_NONE || op == GGML_OP_RESHAPE || op == GGML_OP_VIEW || op == GGML_OP_PERMUTE || op == GGML_OP_TRANSPOSE;
}

static bool b200_op_supported(const struct ggml_tensor * op);

// returns 0 on success, else an error code of the kernel library
static int compute_node(b200_backend_ctx * ctx, struct ggml_tensor * node) {
    void * st = (void *) ctx->stream;
    const struct ggml_tensor * s0 = node->src[0];
    const struct ggml_tensor * s1 = node->src[1];
    int64_t ne0[4], nb0[4], ne1[4], nb1[4], ned[4], nbd[4];
    for (int i = 0; i < 4; ++i) {
        ned[i] = node->ne[i]; nbd[i] = (int64_t) node->nb[i];
        if (s0) { ne0[i] = s0->ne[i]; nb0[i] = (int64_t) s0->nb[i]; }
        if (s1) { ne1[i] = s1->ne[i]; nb1[i] = (int64_t) s1->nb[i]; }
    }
    switch (node->op) {
        case GGML_OP_MUL_MAT: {
            if (is_quant(s0->type)) {
                const int64_t K = s0->ne[0], M = s0->ne[1], N = s1->ne[1];
                const int64_t nb_total = (int64_t) (ggml_nbytes(s0) / ggml_type_size(s0->type));
                if (N <= 8) {
                    return b200_mul_mat_vec_q((int) s0->type, s0->data, nb_total, M, K, (const float *) s1->data, nb1[1], N,
                                              (float *) node->data, nbd[1] / 4, st);
                }
                return gemm_quant(ctx, s0, (const float *) s1->data, nb1[1], N, node->data, nbd[1] / 4, nullptr);
            }
            return b200_mul_mat_f16(s0->data, ne0, nb0, s1->data, (int) s1->type, ne1, nb1, (float *) node->data, nbd, st);
        }
        case GGML_OP_FLASH_ATTN_EXT: {
            const struct ggml_tensor * k = node->src[1], * v = node->src[2], * mask = node->src[3];
            float scale;
            memcpy(&scale, (const float *) node->op_params + 0, sizeof(float));
            return b200_flash_attn_ext((const float *) s0->data, nb0[1], nb0[2], k->data, (int64_t) k->nb[1], (int64_t) k->nb[2],
                                       v->data, (int64_t) v->nb[1], (int64_t) v->nb[2],
                                       mask ? mask->data : nullptr, mask ? (int64_t) mask->nb[1] : 0,
                                       (float *) node->data, s0->ne[1], k->ne[1], s0->ne[2], scale, st);
        }
        case GGML_OP_NORM: {
            float eps;
            memcpy(&eps, node->op_params, sizeof(float));
            return b200_norm((const float *) s0->data, (float *) node->data, ne0[0], ne0[1], ne0[2], ne0[3], nb0, nbd, eps, st);
        }
        case GGML_OP_ADD:
            return b200_binary(0, (const float *) s0->data, ne0, nb0, (const float *) s1->data, ne1, nb1, (float *) node->data, nbd, st);
        case GGML_OP_MUL:
            return b200_binary(1, (const float *) s0->data, ne0, nb0, (const float *) s1->data, ne1, nb1, (float *) node->data, nbd, st);
        case GGML_OP_SCALE: {
            float s;
            memcpy(&s, node->op_params, sizeof(float));
            return b200_scale((const float *) s0->data, (float *) node->data, ggml_nelements(node), s, st);
        }
        case GGML_OP_UNARY:
            return b200_gelu((const float *) s0->data, (float *) node->data, ggml_nelements(node), st);
        case GGML_OP_CPY:
        case GGML_OP_DUP:
        case GGML_OP_CONT:
            return b200_cpy(s0->data, (int) s0->type, ne0, nb0, node->data, (int) node->type, ned, nbd, st);
        case GGML_OP_GET_ROWS: {
            const int64_t arg = is_quant(s0->type) ? (int64_t) (ggml_nbytes(s0) / ggml_type_size(s0->type)) : nb0[1];
            return b200_get_rows((int) s0->type, s0->data, arg, s0->ne[0], (const int32_t *) s1->data, s1->ne[0], (float *) node->data, st);
        }
        case GGML_OP_IM2COL: {
            const int32_t * p = (const int32_t *) node->op_params;
            return b200_im2col_1d_f16((const float *) s1->data, nb1[1], s1->ne[0], s1->ne[1], s0->ne[0], node->ne[1], p[0], p[2], p[4], node->data, st);
        }
        case GGML_OP_SOFT_MAX: {
            float scale;
            memcpy(&scale, (const float *) node->op_params + 0, sizeof(float));
            return b200_soft_max((const float *) s0->data, s1 ? s1->data : nullptr, s1 ? (int) s1->type : 0, s1 ? nb1[1] : 0, s1 ? ne1[1] : 0,
                                 (float *) node->data, ne0[0], ggml_nrows(s0), ne0[1], scale, st);
        }
        case GGML_OP_CONCAT: {
            const int dim = ((const int32_t *) node->op_params)[0];
            return b200_concat((const float *) s0->data, ne0, nb0, (const float *) s1->data, ne1, nb1, (float *) node->data, ned, nbd, dim, st);
        }
        default:
            return B200_ERR_ARG;
    }
}

// ---------------------------------------------------------------------------------------------
// Execution plan.  A graph is turned into a list of launch items; an item is either one node or a fused
// node sequence (NORM->MUL->ADD, MUL_MAT(<= 8 columns)->ADD/SCALE/GELU/CPY).  A fused launch evaluates the
// same single-precision operations in the same order as the nodes it replaces, so the bits that reach
// memory do not change; what goes away is the round trip of the intermediates through HBM and the launches.
//
// Items refer to nodes by position, so one plan serves every graph with the same structure: the decode
// graphs of several whisper_states differ only in addresses and in the number of cached keys.  That is what
// the batcher below uses to run their steps together - one pass over the weights for up to 8 states per
// launch, one launch of the attention / LayerNorm kernels for all of them.
// ---------------------------------------------------------------------------------------------
struct graph_info {
    std::unordered_map<const struct ggml_tensor *, int> index;   // node -> position
    std::vector<int> uses;                                        // consumers inside the graph
};

static void analyse_graph(struct ggml_cgraph * g, graph_info & gi) {
    const int n = ggml_graph_n_nodes(g);
    gi.uses.assign(n, 0);
    gi.index.reserve(n * 2);
    for (int i = 0; i < n; ++i) gi.index[ggml_graph_node(g, i)] = i;
    for (int i = 0; i < n; ++i) {
        const struct ggml_tensor * t = ggml_graph_node(g, i);
        for (int k = 0; k < GGML_MAX_SRC; ++k) {
            if (!t->src[k]) continue;
            auto it = gi.index.find(t->src[k]);
            if (it != gi.index.end()) gi.uses[it->second]++;
        }
        if (t->view_src) {
            auto it = gi.index.find(t->view_src);
            if (it != gi.index.end()) gi.uses[it->second]++;
        }
    }
}

// operand is available before position i (a leaf, or a node computed earlier)
static bool ready_before(const graph_info & gi, const struct ggml_tensor * t, int i) {
    const struct ggml_tensor * base = t;
    while (base->view_src) base = base->view_src;
    auto it = gi.index.find(t);
    if (it != gi.index.end() && it->second >= i) return false;
    it = gi.index.find(base);
    if (it != gi.index.end() && it->second >= i) return false;
    return true;
}

static bool overlaps(const struct ggml_tensor * a, const struct ggml_tensor * b) {
    const char * a0 = (const char *) a->data, * b0 = (const char *) b->data;
    return a0 < b0 + ggml_nbytes(b) && b0 < a0 + ggml_nbytes(a);
}

static bool only_feeds(const graph_info & gi, const struct ggml_tensor * t, int pos) {
    return gi.uses[pos] == 1 && !(t->flags & GGML_TENSOR_FLAG_OUTPUT);
}

enum plan_kind { PK_NODE = 0, PK_LAYER_NORM, PK_GEMV, PK_FA_DECODE, PK_GEMM };

struct plan_item {
    int kind;
    int node;           // NORM / MUL_MAT / FLASH_ATTN_EXT / generic node
    int last;           // node whose memory receives the result (== node when nothing is fused)
    // PK_GEMV epilogue
    int n_steps;
    int step_kind[4];
    int step_node[4];   // the ADD / SCALE / UNARY node of the step
    int step_src[4];    // ADD: which src of that node is the added operand
    int store_f16;
};

struct exec_plan {
    std::vector<plan_item> items;
    int n_nodes = 0;
};

static bool is_decode_attention(const struct ggml_tensor * node) {
    return node->op == GGML_OP_FLASH_ATTN_EXT && node->src[0]->ne[1] <= 8;
}

static void build_plan(struct ggml_cgraph * g, exec_plan & plan, bool fuse) {
    const int n = ggml_graph_n_nodes(g);
    plan.items.clear();
    plan.n_nodes = n;
    graph_info gi;
    if (fuse) analyse_graph(g, gi);
    std::vector<char> fused(n, 0);
    for (int i = 0; i < n; ++i) {
        struct ggml_tensor * node = ggml_graph_node(g, i);
        if (is_view_op(node->op) || ggml_is_empty(node) || fused[i]) continue;
        plan_item it;
        memset(&it, 0, sizeof(it));
        it.kind = PK_NODE; it.node = i; it.last = i;
        if (fuse && node->op == GGML_OP_NORM && i + 2 < n && only_feeds(gi, node, i)) {
            struct ggml_tensor * mul = ggml_graph_node(g, i + 1);
            struct ggml_tensor * add = ggml_graph_node(g, i + 2);
            const struct ggml_tensor * x = node->src[0];
            auto vec_ok = [&](const struct ggml_tensor * v) {
                return v->type == GGML_TYPE_F32 && v->ne[0] == x->ne[0] && v->ne[1] == 1 && v->ne[2] == 1 && v->ne[3] == 1 && v->nb[0] == 4;
            };
            if (mul->op == GGML_OP_MUL && add->op == GGML_OP_ADD && mul->src[0] == node && add->src[0] == mul && only_feeds(gi, mul, i + 1) &&
                vec_ok(mul->src[1]) && vec_ok(add->src[1]) && ready_before(gi, mul->src[1], i) && ready_before(gi, add->src[1], i) &&
                x->type == GGML_TYPE_F32 && x->ne[2] == 1 && x->ne[3] == 1 && x->nb[0] == 4 && add->nb[0] == 4 && ggml_are_same_shape(x, add)) {
                it.kind = PK_LAYER_NORM; it.last = i + 2;
                fused[i + 1] = 1; fused[i + 2] = 1;
            }
        } else if (node->op == GGML_OP_MUL_MAT && is_quant(node->src[0]->type)) {
            it.kind = node->src[1]->ne[1] <= 8 ? PK_GEMV : PK_GEMM;
            if (fuse) {
                struct ggml_tensor * cur = node;
                const int64_t M = node->ne[0], N = node->ne[1];
                int cur_pos = i;
                for (int j = i + 1; j < n && it.n_steps < 4; ++j) {
                    struct ggml_tensor * t = ggml_graph_node(g, j);
                    if (is_view_op(t->op)) {
                        if (t->src[0] == cur || t->view_src == cur) break;      // someone looks at cur itself
                        continue;
                    }
                    if (!only_feeds(gi, cur, cur_pos)) break;
                    int kind = 0, src = 0;
                    if (t->op == GGML_OP_ADD && (t->src[0] == cur || t->src[1] == cur) && t->type == GGML_TYPE_F32) {
                        src = t->src[0] == cur ? 1 : 0;
                        const struct ggml_tensor * o = t->src[src];
                        if (o == cur || o->type != GGML_TYPE_F32 || o->nb[0] != 4 || o->ne[0] != M || o->ne[2] != 1 || o->ne[3] != 1) break;
                        if (o->ne[1] != 1 && o->ne[1] != N) break;
                        if (!ggml_are_same_shape(t, cur) || !ready_before(gi, o, i)) break;
                        kind = B200_EP_ADD;
                    } else if (t->op == GGML_OP_SCALE && t->src[0] == cur) {
                        kind = B200_EP_SCALE;
                    } else if (t->op == GGML_OP_UNARY && t->src[0] == cur && ggml_get_unary_op(t) == GGML_UNARY_OP_GELU) {
                        kind = B200_EP_GELU;
                    } else if (t->op == GGML_OP_CPY && t->src[0] == cur && t->type == GGML_TYPE_F16 && ggml_is_contiguous(t) &&
                               ggml_nelements(t) == M * N && ggml_is_contiguous(cur)) {
                        it.store_f16 = 1;
                        fused[j] = 1;
                        it.last = j;
                        break;
                    } else {
                        break;
                    }
                    if (t->nb[0] != 4) break;
                    it.step_kind[it.n_steps] = kind; it.step_node[it.n_steps] = j; it.step_src[it.n_steps] = src;
                    it.n_steps++;
                    fused[j] = 1;
                    cur = t; cur_pos = j;
                    it.last = j;
                }
            }
        } else if (is_decode_attention(node)) {
            it.kind = PK_FA_DECODE;
        }
        plan.items.push_back(it);
    }
}

// Structure signature of a graph: operator, type and shape of every computing node, except the extents that only
// depend on how many keys are cached (attention inputs, the mask copy).  Equal signature = same plan applies.
static uint64_t graph_signature(struct ggml_cgraph * g) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { h ^= v; h *= 1099511628211ull; };
    const int n = ggml_graph_n_nodes(g);
    mix((uint64_t) n);
    for (int i = 0; i < n; ++i) {
        const struct ggml_tensor * t = ggml_graph_node(g, i);
        mix((uint64_t) t->op * 131 + (uint64_t) t->type);
        if (is_view_op(t->op)) continue;
        if (t->op == GGML_OP_CPY) { mix((uint64_t) t->src[0]->type); continue; }
        mix((uint64_t) t->ne[0]); mix((uint64_t) t->ne[1]); mix((uint64_t) t->ne[2]);
        if (t->src[0]) { mix((uint64_t) t->src[0]->type); mix((uint64_t) t->src[0]->ne[0]); }
        if (t->src[1] && t->op != GGML_OP_FLASH_ATTN_EXT) { mix((uint64_t) t->src[1]->type); mix((uint64_t) t->src[1]->ne[0]); mix((uint64_t) t->src[1]->ne[1]); }
    }
    return h;
}

// Does graph g satisfy what the plan assumes (operators in place, supported, no aliasing hazard for fused items)?
// A plan is found by a signature of operators, types and shapes only, so everything fusion relied on when the plan
// was built is checked again on the candidate graph: the intermediates of a fused item have exactly one consumer and
// are not graph outputs, shapes and strides of the operands are what the fused kernels take.
static bool graph_fits_plan(const exec_plan & plan, struct ggml_cgraph * g) {
    const int n_nodes = ggml_graph_n_nodes(g);
    if (n_nodes != plan.n_nodes) return false;
    {   // intermediates that a fused launch never writes to memory
        std::vector<const struct ggml_tensor *> inter;
        for (const plan_item & it : plan.items) {
            if (it.last == it.node) continue;
            if (it.kind == PK_LAYER_NORM) {
                inter.push_back(ggml_graph_node(g, it.node));
                inter.push_back(ggml_graph_node(g, it.node + 1));
            } else if (it.kind == PK_GEMV || it.kind == PK_GEMM) {
                inter.push_back(ggml_graph_node(g, it.node));
                for (int s = 0; s < it.n_steps; ++s) if (it.step_node[s] != it.last) inter.push_back(ggml_graph_node(g, it.step_node[s]));
            }
        }
        if (!inter.empty()) {
            std::unordered_map<const struct ggml_tensor *, int> uses;
            uses.reserve(inter.size() * 2);
            for (const struct ggml_tensor * t : inter) {
                if (t->flags & GGML_TENSOR_FLAG_OUTPUT) return false;
                uses[t] = 0;
            }
            // operands a fused epilogue adds (and what they are views of) must exist before the product runs
            std::unordered_map<const struct ggml_tensor *, int> needed_before;
            for (const plan_item & it : plan.items) {
                if (it.kind != PK_GEMV && it.kind != PK_GEMM) continue;
                for (int s = 0; s < it.n_steps; ++s) {
                    if (it.step_kind[s] != B200_EP_ADD) continue;
                    const struct ggml_tensor * o = ggml_graph_node(g, it.step_node[s])->src[it.step_src[s]];
                    for (; o; o = o->view_src) {
                        auto f = needed_before.find(o);
                        if (f == needed_before.end() || f->second > it.node) needed_before[o] = it.node;
                    }
                }
            }
            for (int i = 0; i < n_nodes; ++i) {
                const struct ggml_tensor * t = ggml_graph_node(g, i);
                if (!needed_before.empty()) {
                    auto f = needed_before.find(t);
                    if (f != needed_before.end() && i >= f->second) return false;
                }
                for (int k = 0; k < GGML_MAX_SRC; ++k) {
                    if (!t->src[k]) continue;
                    auto u = uses.find(t->src[k]);
                    if (u != uses.end()) u->second++;
                }
                if (t->view_src) {
                    auto u = uses.find(t->view_src);
                    if (u != uses.end()) u->second++;
                }
            }
            for (const auto & u : uses) if (u.second != 1) return false;
        }
    }
    for (const plan_item & it : plan.items) {
        struct ggml_tensor * node = ggml_graph_node(g, it.node);
        if (!b200_op_supported(node)) return false;
        if (it.kind == PK_LAYER_NORM) {
            if (node->op != GGML_OP_NORM) return false;
            struct ggml_tensor * mul = ggml_graph_node(g, it.node + 1), * out = ggml_graph_node(g, it.last);
            if (mul->op != GGML_OP_MUL || out->op != GGML_OP_ADD || mul->src[0] != node || out->src[0] != mul) return false;
            const struct ggml_tensor * x = node->src[0];
            auto vec_ok = [&](const struct ggml_tensor * v) {
                return v->type == GGML_TYPE_F32 && v->ne[0] == x->ne[0] && v->ne[1] == 1 && v->ne[2] == 1 && v->ne[3] == 1 && v->nb[0] == 4;
            };
            if (!vec_ok(mul->src[1]) || !vec_ok(out->src[1]) || x->type != GGML_TYPE_F32 || x->ne[2] != 1 || x->ne[3] != 1 || x->nb[0] != 4 ||
                out->nb[0] != 4 || !ggml_are_same_shape(x, out)) return false;
            // rows are read and written by the same threads, so exact in-place is fine; a shifted overlap is not
            if (overlaps(out, x) && !(out->data == x->data && out->nb[1] == x->nb[1])) return false;
            if (!b200_op_supported(mul) || !b200_op_supported(out)) return false;
        } else if (it.kind == PK_GEMV || it.kind == PK_GEMM) {
            if (node->op != GGML_OP_MUL_MAT || !is_quant(node->src[0]->type) || (node->src[1]->ne[1] > 8) != (it.kind == PK_GEMM)) return false;
            struct ggml_tensor * out = ggml_graph_node(g, it.last);
            const struct ggml_tensor * cur = node;
            for (int s = 0; s < it.n_steps; ++s) {
                struct ggml_tensor * t = ggml_graph_node(g, it.step_node[s]);
                if (t->nb[0] != 4 || t->type != GGML_TYPE_F32 || !ggml_are_same_shape(t, node)) return false;
                if (it.step_kind[s] == B200_EP_ADD) {
                    if (t->op != GGML_OP_ADD || t->src[1 - it.step_src[s]] != cur) return false;
                    const struct ggml_tensor * o = t->src[it.step_src[s]];
                    if (o == cur || o->type != GGML_TYPE_F32 || o->nb[0] != 4 || o->ne[0] != node->ne[0] || o->ne[2] != 1 || o->ne[3] != 1 ||
                        (o->ne[1] != 1 && o->ne[1] != node->ne[1])) return false;
                    // an added tensor may share memory with the result only element for element
                    if (overlaps(out, o) && !(o->data == out->data && o->nb[1] == out->nb[1])) return false;
                } else if (it.step_kind[s] == B200_EP_SCALE) {
                    if (t->op != GGML_OP_SCALE || t->src[0] != cur) return false;
                } else {
                    if (t->op != GGML_OP_UNARY || t->src[0] != cur) return false;
                }
                cur = t;
            }
            if (it.store_f16 && (out->op != GGML_OP_CPY || out->src[0] != cur || out->type != GGML_TYPE_F16 || !ggml_is_contiguous(out) ||
                                 !ggml_is_contiguous(cur) || ggml_nelements(out) != node->ne[0] * node->ne[1])) return false;
            // GEMV: every CTA reads the activations for the whole kernel, the result must not land on them
            // (the GEMM path reads a quantised copy made before the product starts)
            if (it.kind == PK_GEMV && it.last != it.node && overlaps(out, node->src[1])) return false;
        } else if (it.kind == PK_FA_DECODE) {
            if (!is_decode_attention(node)) return false;
        }
    }
    return true;
}

// timing class of a node and its algorithmic work (bytes for memory-bound classes, FLOPs for contractions)
static int node_class(const struct ggml_tensor * node, double * work) {
    const struct ggml_tensor * s0 = node->src[0];
    const struct ggml_tensor * s1 = node->src[1];
    const double out_bytes = (double) ggml_nbytes(node);
    switch (node->op) {
        case GGML_OP_MUL_MAT:
            if (is_quant(s0->type)) {
                if (s1->ne[1] <= 8) { *work = (double) ggml_nbytes(s0) + (double) ggml_nbytes(s1) + out_bytes; return TC_MMQ_VEC; }
                *work = 2.0 * (double) s0->ne[0] * (double) s0->ne[1] * (double) s1->ne[1];
                return TC_MMQ_GEMM;
            }
            *work = 2.0 * (double) s0->ne[0] * (double) s0->ne[1] * (double) s1->ne[1] * (double) s1->ne[2] * (double) s1->ne[3];
            return TC_MM_F16;
        case GGML_OP_FLASH_ATTN_EXT:
            if (s0->ne[1] <= 8) {   // decode: bound by streaming K and V once per query row
                *work = 2.0 * 2.0 * 64.0 * (double) s0->ne[1] * (double) s0->ne[2] * (double) node->src[1]->ne[1];
                return TC_FATTN_DEC;
            }
            *work = 4.0 * 64.0 * (double) s0->ne[1] * (double) s0->ne[2] * (double) node->src[1]->ne[1];
            return TC_FATTN;
        case GGML_OP_NORM:     *work = 2.0 * out_bytes; return TC_NORM;
        case GGML_OP_ADD: case GGML_OP_MUL: *work = 2.0 * out_bytes + (double) ggml_nbytes(s1); return TC_BINARY;
        case GGML_OP_SCALE:    *work = 2.0 * out_bytes; return TC_SCALE;
        case GGML_OP_UNARY:    *work = 2.0 * out_bytes; return TC_GELU;
        case GGML_OP_CPY: case GGML_OP_DUP: case GGML_OP_CONT: *work = (double) ggml_nbytes(s0) + out_bytes; return TC_CPY;
        case GGML_OP_GET_ROWS: *work = 2.0 * out_bytes; return TC_GET_ROWS;
        case GGML_OP_IM2COL:   *work = (double) ggml_nbytes(s1) + out_bytes; return TC_IM2COL;
        case GGML_OP_SOFT_MAX: *work = 2.0 * out_bytes; return TC_SOFT_MAX;
        case GGML_OP_CONCAT:   *work = 2.0 * out_bytes; return TC_CONCAT;
        default: *work = 0; return TC_CONCAT;
    }
}

// Runs one plan item for all graphs in gs (same structure) on ctx's stream.  Returns 0 or an error code.
static int run_item(b200_backend_ctx * ctx, const plan_item & it, struct ggml_cgraph * const * gs, int n_g) {
    void * st = (void *) ctx->stream;
    if (it.kind == PK_NODE) {
        for (int g = 0; g < n_g; ++g) {
            const int e = compute_node(ctx, ggml_graph_node(gs[g], it.node));
            if (e) return e;
        }
        return 0;
    }
    if (it.kind == PK_LAYER_NORM) {
        b200_ln_row rows[64];
        int n_rows = 0;
        bool launched_rows = false;
        struct ggml_tensor * n0 = ggml_graph_node(gs[0], it.node);
        const float * gamma = (const float *) ggml_graph_node(gs[0], it.node + 1)->src[1]->data;
        const float * beta  = (const float *) ggml_graph_node(gs[0], it.last)->src[1]->data;
        float eps;
        memcpy(&eps, n0->op_params, sizeof(float));
        const int64_t ne00 = n0->src[0]->ne[0];
        for (int g = 0; g < n_g; ++g) {
            struct ggml_tensor * nrm = ggml_graph_node(gs[g], it.node), * out = ggml_graph_node(gs[g], it.last);
            const struct ggml_tensor * x = nrm->src[0];
            const float * ga = (const float *) ggml_graph_node(gs[g], it.node + 1)->src[1]->data;
            const float * be = (const float *) out->src[1]->data;
            if (ga != gamma || be != beta || x->ne[1] > 64 || ne00 > 2048) {     // other weights or a tall input: on its own
                const int e = b200_layer_norm((const float *) x->data, ga, be, (float *) out->data, x->ne[0], x->ne[1], (int64_t) x->nb[1], (int64_t) out->nb[1], eps, st);
                if (e) return e;
                continue;
            }
            for (int64_t r = 0; r < x->ne[1]; ++r) {
                if (n_rows == 64) {
                    const int e = b200_layer_norm_rows(rows, n_rows, gamma, beta, ne00, eps, st);
                    if (e) return e;
                    n_rows = 0;
                    launched_rows = true;
                }
                rows[n_rows].x = (const float *) ((const char *) x->data + r * x->nb[1]);
                rows[n_rows].y = (float *) ((char *) out->data + r * out->nb[1]);
                ++n_rows;
            }
        }
        if (!n_rows) return 0;
        // Rows of several states go to a product next (5..32 columns: the quantised-column path): the same kernel also
        // leaves them quantised in the column buffer, marked as written by this item so that the product reuses them.
        static const bool fuse_q = getenv("GGML_B200_NO_FUSION") == nullptr;
        if (fuse_q && !launched_rows && n_rows > 4 && n_rows <= COLQ_MAX_COLS && ne00 % 32 == 0 && ne00 <= COLQ_MAX_K) {
            const int e = b200_layer_norm_rows_q(rows, n_rows, gamma, beta, ne00, eps, colq_q(ctx), colq_d(ctx), st);
            ctx->colq_ptrs.resize(n_rows);
            for (int i = 0; i < n_rows; ++i) ctx->colq_ptrs[i] = rows[i].y;
            ctx->colq_K = ne00;
            ctx->colq_seq = ctx->item_seq;
            return e;
        }
        return b200_layer_norm_rows(rows, n_rows, gamma, beta, ne00, eps, st);
    }
    if (it.kind == PK_GEMV) {
        struct ggml_tensor * n0 = ggml_graph_node(gs[0], it.node);
        const struct ggml_tensor * w = n0->src[0];
        const int64_t K = w->ne[0], M = w->ne[1];
        const int64_t nb_total = (int64_t) (ggml_nbytes(w) / ggml_type_size(w->type));
        b200_gemv_ep ep;
        memset(&ep, 0, sizeof(ep));
        ep.n_steps = it.n_steps; ep.store_f16 = it.store_f16;
        for (int s = 0; s < it.n_steps; ++s) {
            ep.kind[s] = it.step_kind[s];
            if (it.step_kind[s] == B200_EP_SCALE) memcpy(&ep.scalar[s], ggml_graph_node(gs[0], it.step_node[s])->op_params, sizeof(float));
        }
        b200_gemv_col cols[COLQ_MAX_COLS];
        const float * xs[COLQ_MAX_COLS];
        int n_cols = 0;
        int8_t * xq = colq_q(ctx);
        float *  xd = colq_d(ctx);
        // products of this many columns or more go to the tcgen05 kernel (one launch for up to 64 columns, time nearly
        // independent of the column count); fewer columns stay with the FMA-pipe kernels that stream the weights once
        static const int tc_min_cols = getenv("GGML_B200_TC_MIN_COLS") ? atoi(getenv("GGML_B200_TC_MIN_COLS")) : 48;
        static const bool use_tc = getenv("GGML_B200_TC") != nullptr && atoi(getenv("GGML_B200_TC")) != 0;
        auto flush = [&]() -> int {
            if (!n_cols) return 0;
            int e = 0;
            if (n_cols <= 4) {
                e = b200_mul_mat_vec_q_cols((int) w->type, w->data, nb_total, M, K, cols, n_cols, &ep, st);
            } else if (K <= COLQ_MAX_K) {
                // the columns are quantised once and stay valid for the products that follow immediately on the same
                // activations (the K, V and Q projections of a layer)
                const bool reuse = ctx->colq_seq + 1 == ctx->item_seq && ctx->colq_K == K && (int) ctx->colq_ptrs.size() == n_cols &&
                                   memcmp(ctx->colq_ptrs.data(), xs, sizeof(xs[0]) * n_cols) == 0;
                if (!reuse) {
                    for (int c0 = 0; c0 < n_cols && !e; c0 += 32)
                        e = b200_quantize_cols(xs + c0, n_cols - c0 < 32 ? n_cols - c0 : 32, K, xq + (size_t) c0 * K, xd + (size_t) c0 * (K / 32), st);
                    if (e) return e;
                    ctx->colq_ptrs.assign(xs, xs + n_cols);
                    ctx->colq_K = K;
                }
                ctx->colq_seq = ctx->item_seq;
                if (use_tc && n_cols >= tc_min_cols) {
                    e = b200_mul_mat_tc_cols((int) w->type, w->data, nb_total, M, K, xq, xd, cols, n_cols, &ep, st);
                } else {
                    // shared memory holds the quantised columns next to the weight rows: fewer columns per launch for long rows
                    const int cap = K > 2560 ? 16 : 32;
                    for (int c0 = 0; c0 < n_cols && !e; c0 += cap)
                        e = b200_mul_mat_cols_q((int) w->type, w->data, nb_total, M, K, xq + (size_t) c0 * K, xd + (size_t) c0 * (K / 32), cols + c0,
                                                n_cols - c0 < cap ? n_cols - c0 : cap, &ep, st);
                }
            } else {
                for (int c0 = 0; c0 < n_cols && !e; c0 += 8)
                    e = b200_mul_mat_vec_q_cols((int) w->type, w->data, nb_total, M, K, cols + c0, n_cols - c0 < 8 ? n_cols - c0 : 8, &ep, st);
            }
            n_cols = 0;
            return e;
        };
        int n_flushes = 0;
        for (int g = 0; g < n_g; ++g) {
            struct ggml_tensor * mm = ggml_graph_node(gs[g], it.node), * out = ggml_graph_node(gs[g], it.last);
            if (mm->src[0]->data != w->data) {            // a state of another model on the same device: its own launch
                int e = flush();
                if (e) return e;
                struct ggml_cgraph * one[1] = { gs[g] };
                ctx->colq_seq = -2;
                e = run_item(ctx, it, one, 1);
                if (e) return e;
                ctx->colq_seq = -2;
                continue;
            }
            const struct ggml_tensor * x = mm->src[1];
            const int64_t out_stride = it.store_f16 ? mm->ne[0] * 2 : (int64_t) out->nb[1];
            for (int64_t c = 0; c < x->ne[1]; ++c) {
                if (n_cols == COLQ_MAX_COLS) { const int e = flush(); if (e) return e; ++n_flushes; ctx->colq_seq = -2; }
                b200_gemv_col & col = cols[n_cols];
                memset(&col, 0, sizeof(col));
                col.x = (const float *) ((const char *) x->data + c * x->nb[1]);
                xs[n_cols] = col.x;
                col.dst = (char *) out->data + c * out_stride;
                for (int s = 0; s < it.n_steps; ++s) {
                    if (it.step_kind[s] != B200_EP_ADD) continue;
                    const struct ggml_tensor * o = ggml_graph_node(gs[g], it.step_node[s])->src[it.step_src[s]];
                    col.add[s] = (const float *) ((const char *) o->data + (o->ne[1] == 1 ? 0 : c * o->nb[1]));
                }
                ++n_cols;
            }
        }
        const int e = flush();
        if (n_flushes) ctx->colq_seq = -2;      // more than one group went through the buffer: nothing to reuse
        return e;
    }
    if (it.kind == PK_GEMM) {
        for (int g = 0; g < n_g; ++g) {
            struct ggml_tensor * mm = ggml_graph_node(gs[g], it.node), * out = ggml_graph_node(gs[g], it.last);
            const struct ggml_tensor * w = mm->src[0], * x = mm->src[1];
            const int64_t K = w->ne[0], M = w->ne[1], N = x->ne[1];
            const int64_t nb_total = (int64_t) (ggml_nbytes(w) / ggml_type_size(w->type));
            b200_epilogue ep;
            memset(&ep, 0, sizeof(ep));
            ep.n_steps = it.n_steps; ep.store_f16 = it.store_f16;
            for (int s = 0; s < it.n_steps; ++s) {
                struct ggml_tensor * t = ggml_graph_node(gs[g], it.step_node[s]);
                ep.step[s].kind = it.step_kind[s];
                if (it.step_kind[s] == B200_EP_SCALE) memcpy(&ep.step[s].scalar, t->op_params, sizeof(float));
                if (it.step_kind[s] == B200_EP_ADD) {
                    const struct ggml_tensor * o = t->src[it.step_src[s]];
                    ep.step[s].ptr = (const float *) o->data;
                    ep.step[s].stride_n = o->ne[1] == 1 ? 0 : (int64_t) o->nb[1] / 4;
                }
            }
            const int64_t ldd = it.store_f16 ? M : (int64_t) out->nb[1] / 4;
            int e = gemm_quant(ctx, w, (const float *) x->data, (int64_t) x->nb[1], N, out->data, ldd, &ep);
            if (e) return e;
        }
        return 0;
    }
    // PK_FA_DECODE
    {
        struct ggml_tensor * n0 = ggml_graph_node(gs[0], it.node);
        const struct ggml_tensor * q0 = n0->src[0], * k0 = n0->src[1], * v0 = n0->src[2];
        float scale;
        memcpy(&scale, (const float *) n0->op_params + 0, sizeof(float));
        b200_fa_row rows[COLQ_MAX_COLS];
        int n_rows = 0;
        static const bool fuse_q = getenv("GGML_B200_NO_FUSION") == nullptr;
        int n_launches = 0;
        bool last = false;
        auto flush = [&]() -> int {
            if (!n_rows) return 0;
            int e = 0;
            // One flush that covers all rows, followed by the output projection (5..64 columns: the quantised-column path):
            // the kernel also leaves the rows quantised in the column buffer, marked as written by this item.
            const int64_t kk = q0->ne[2] * 64;
            const bool with_q = fuse_q && last && n_launches == 0 && n_rows > 4 && kk <= COLQ_MAX_K && q0->ne[0] == 64;
            for (int r0 = 0; r0 < n_rows && !e; r0 += 32) {
                const int n = n_rows - r0 < 32 ? n_rows - r0 : 32;
                if (with_q)
                    e = b200_flash_attn_decode_rows_q(rows + r0, n, q0->ne[2], (int64_t) q0->nb[2], (int64_t) k0->nb[1], (int64_t) k0->nb[2],
                                                      (int64_t) v0->nb[1], (int64_t) v0->nb[2], scale, colq_q(ctx) + (size_t) r0 * kk, colq_d(ctx) + (size_t) r0 * (kk / 32), st);
                else
                    e = b200_flash_attn_decode_rows(rows + r0, n, q0->ne[2], (int64_t) q0->nb[2], (int64_t) k0->nb[1], (int64_t) k0->nb[2],
                                                    (int64_t) v0->nb[1], (int64_t) v0->nb[2], scale, st);
            }
            if (with_q && !e) {
                ctx->colq_ptrs.resize(n_rows);
                for (int i = 0; i < n_rows; ++i) ctx->colq_ptrs[i] = rows[i].dst;
                ctx->colq_K = kk;
                ctx->colq_seq = ctx->item_seq;
            }
            ++n_launches;
            n_rows = 0;
            return e;
        };
        for (int g = 0; g < n_g; ++g) {
            struct ggml_tensor * fa = ggml_graph_node(gs[g], it.node);
            const struct ggml_tensor * q = fa->src[0], * k = fa->src[1], * v = fa->src[2], * mask = fa->src[3];
            float sc;
            memcpy(&sc, (const float *) fa->op_params + 0, sizeof(float));
            const bool same = q->nb[2] == q0->nb[2] && k->nb[1] == k0->nb[1] && k->nb[2] == k0->nb[2] && v->nb[1] == v0->nb[1] &&
                              v->nb[2] == v0->nb[2] && sc == scale && q->ne[2] == q0->ne[2];
            const bool fast = same && k->ne[1] <= 8192 && !((uintptr_t) k->data & 15) && !((uintptr_t) v->data & 15) && !(k->nb[1] & 15) &&
                              !(k->nb[2] & 15) && !(v->nb[1] & 15) && !(v->nb[2] & 15);
            if (!fast) {
                int e = flush();
                if (e) return e;
                e = compute_node(ctx, fa);
                if (e) return e;
                ++n_launches;
                continue;
            }
            for (int64_t r = 0; r < q->ne[1]; ++r) {
                if (n_rows == COLQ_MAX_COLS) { const int e = flush(); if (e) return e; }
                rows[n_rows].q    = (const float *) ((const char *) q->data + r * q->nb[1]);
                rows[n_rows].k    = k->data;
                rows[n_rows].v    = v->data;
                rows[n_rows].mask = mask ? (const char *) mask->data + r * mask->nb[1] : nullptr;
                rows[n_rows].dst  = (float *) ((char *) fa->data + r * fa->nb[2]);
                rows[n_rows].n_kv = k->ne[1];
                ++n_rows;
            }
        }
        last = true;
        return flush();
    }
}

// Consecutive products on the same activation columns (the Q, K and V projections of a decoder layer, for 5..32 columns
// of states that step together) as ONE launch.  Returns -1 when the items do not qualify; the caller then runs them one
// by one.  Columns, outputs and epilogue operands are gathered exactly as run_item does for a single product.
static int run_gemv_group(b200_backend_ctx * ctx, const plan_item * its, int n_items, struct ggml_cgraph * const * gs, int n_g) {
    if (n_items < 2 || n_items > 3) return -1;
    void * st = (void *) ctx->stream;
    const struct ggml_tensor * w0 = ggml_graph_node(gs[0], its[0].node)->src[0];
    const int64_t K = w0->ne[0];
    if (K > COLQ_MAX_K) return -1;
    b200_gemv_col cols[3][32];
    b200_gemv_ep  eps[3];
    const float * xs[32];
    const void *  wp[3];
    int64_t       nbt[3], Ms[3];
    int n_cols = 0;
    for (int i = 0; i < n_items; ++i) {
        const plan_item & it = its[i];
        struct ggml_tensor * n0 = ggml_graph_node(gs[0], it.node);
        const struct ggml_tensor * w = n0->src[0];
        if (it.kind != PK_GEMV || w->type != w0->type || w->ne[0] != K || w->ne[1] >= 16384) return -1;
        wp[i] = w->data; Ms[i] = w->ne[1];
        nbt[i] = (int64_t) (ggml_nbytes(w) / ggml_type_size(w->type));
        memset(&eps[i], 0, sizeof(eps[i]));
        eps[i].n_steps = it.n_steps; eps[i].store_f16 = it.store_f16;
        for (int s = 0; s < it.n_steps; ++s) {
            eps[i].kind[s] = it.step_kind[s];
            if (it.step_kind[s] == B200_EP_SCALE) memcpy(&eps[i].scalar[s], ggml_graph_node(gs[0], it.step_node[s])->op_params, sizeof(float));
        }
        int nc = 0;
        for (int g = 0; g < n_g; ++g) {
            struct ggml_tensor * mm = ggml_graph_node(gs[g], it.node), * out = ggml_graph_node(gs[g], it.last);
            if (mm->src[0]->data != w->data) return -1;                 // a state of another model: not here
            const struct ggml_tensor * x = mm->src[1];
            const int64_t out_stride = it.store_f16 ? mm->ne[0] * 2 : (int64_t) out->nb[1];
            for (int64_t c = 0; c < x->ne[1]; ++c) {
                if (nc == 32) return -1;
                b200_gemv_col & col = cols[i][nc];
                memset(&col, 0, sizeof(col));
                col.x = (const float *) ((const char *) x->data + c * x->nb[1]);
                if (i == 0) xs[nc] = col.x; else if (xs[nc] != col.x) return -1;      // all products read the same columns
                col.dst = (char *) out->data + c * out_stride;
                for (int s = 0; s < it.n_steps; ++s) {
                    if (it.step_kind[s] != B200_EP_ADD) continue;
                    const struct ggml_tensor * o = ggml_graph_node(gs[g], it.step_node[s])->src[it.step_src[s]];
                    col.add[s] = (const float *) ((const char *) o->data + (o->ne[1] == 1 ? 0 : c * o->nb[1]));
                }
                ++nc;
            }
        }
        if (i == 0) n_cols = nc; else if (nc != n_cols) return -1;
    }
    if (n_cols <= 4) return -1;
    {   // many columns: each product is one tcgen05 launch of its own (run_item)
        static const int tc_min_cols = getenv("GGML_B200_TC_MIN_COLS") ? atoi(getenv("GGML_B200_TC_MIN_COLS")) : 48;
        static const bool use_tc = getenv("GGML_B200_TC") != nullptr && atoi(getenv("GGML_B200_TC")) != 0;
        if (use_tc && n_cols >= tc_min_cols) return -1;
    }
    int8_t * xq = colq_q(ctx);
    float *  xd = colq_d(ctx);
    const bool reuse = ctx->colq_seq + 1 == ctx->item_seq && ctx->colq_K == K && (int) ctx->colq_ptrs.size() == n_cols &&
                       memcmp(ctx->colq_ptrs.data(), xs, sizeof(xs[0]) * n_cols) == 0;
    if (!reuse) {
        const int e = b200_quantize_cols(xs, n_cols, K, xq, xd, st);
        if (e) return e;
        ctx->colq_ptrs.assign(xs, xs + n_cols);
        ctx->colq_K = K;
    }
    const b200_gemv_col * colp[3] = { cols[0], cols[1], cols[2] };
    const b200_gemv_ep *  epp[3]  = { &eps[0], &eps[1], &eps[2] };
    return b200_mul_mat_cols_q_multi((int) w0->type, n_items, wp, nbt, Ms, K, xq, xd, colp, n_cols, epp, st);
}

static bool is_noop(enum ggml_op op) {
    return op == GGML_OP_NONE || op == GGML_OP_RESHAPE || op == GGML_OP_VIEW || op == GGML_OP_PERMUTE || op == GGML_OP_TRANSPOSE;
}

// The logits product is the last node of a decoder graph (src/whisper.cpp:2830, 2953).  With the side output switched
// on, every logits row of every graph of the group gets its top-k / max / log-sum-exp written into the device buffer of
// the backend instance the graph belongs to (owners[g]), by one launch on the stream that ran the plan.
static int logits_side_output(b200_backend_ctx * ctx, struct ggml_cgraph * const * gs, b200_backend_ctx * const * owners, int n_g) {
    const int k = g_topk_k.load(std::memory_order_relaxed);
    const float * rows[64];
    b200_topk_result * outs[64];
    int n_rows = 0;
    int64_t n_vocab = 0;
    for (int g = 0; g < n_g; ++g) {
        struct ggml_tensor * t = ggml_graph_node(gs[g], -1);
        owners[g]->topk_rows = 0;
        if (t->op != GGML_OP_MUL_MAT || t->type != GGML_TYPE_F32 || t->ne[0] < 1024 || t->ne[1] > 8 || t->ne[2] != 1 || t->ne[3] != 1 || t->nb[0] != 4) continue;
        {
            std::lock_guard<std::mutex> lk(g_logits_mu);
            if (g_logits_ptrs.size() > 4096) g_logits_ptrs.clear();
            g_logits_ptrs[t->data] = 1;
        }
        if (k <= 0 || !owners[g]->topk) continue;
        if (n_vocab == 0) n_vocab = t->ne[0];
        if (t->ne[0] != n_vocab) continue;
        for (int64_t c = 0; c < t->ne[1]; ++c) {
            if (n_rows == 64) {
                const int e = b200_topk_rows(rows, outs, n_rows, n_vocab, k, (void *) ctx->stream);
                if (e) return e;
                n_rows = 0;
            }
            rows[n_rows] = (const float *) ((const char *) t->data + c * t->nb[1]);
            outs[n_rows] = owners[g]->topk + c;
            ++n_rows;
        }
        owners[g]->topk_rows = (int) t->ne[1];
    }
    return n_rows ? b200_topk_rows(rows, outs, n_rows, n_vocab, k, (void *) ctx->stream) : 0;
}

static int run_plan(b200_backend_ctx * ctx, const exec_plan & plan, struct ggml_cgraph * const * gs, int n_g, bool timing,
                    std::vector<int> * t_class, std::vector<double> * t_work, size_t * n_ev) {
    auto next_event = [&]() -> cudaEvent_t {
        if (*n_ev == ctx->events.size()) { cudaEvent_t e; cudaEventCreate(&e); ctx->events.push_back(e); }
        return ctx->events[(*n_ev)++];
    };
    ctx->colq_seq = -2;                      // activations of an earlier graph never carry over
    qx_forget(ctx);
    static const bool group_gemv = getenv("GGML_B200_NO_FUSION") == nullptr && getenv("GGML_B200_NO_QKV_GROUP") == nullptr;
    for (size_t ii = 0; ii < plan.items.size(); ++ii) {
        const plan_item & it = plan.items[ii];
        // views do nothing and do not separate a producer of quantised columns from the product that reuses them
        if (!(it.kind == PK_NODE && is_noop(ggml_graph_node(gs[0], it.node)->op))) ctx->item_seq++;
        if (group_gemv && !timing && it.kind == PK_GEMV && ii + 1 < plan.items.size() && plan.items[ii + 1].kind == PK_GEMV) {
            // products that follow each other on the same activations (Q, K, V): one launch
            const void * x0 = ggml_graph_node(gs[0], it.node)->src[1]->data;
            int n_items = 1;
            while (n_items < 3 && ii + n_items < plan.items.size() && plan.items[ii + n_items].kind == PK_GEMV &&
                   ggml_graph_node(gs[0], plan.items[ii + n_items].node)->src[1]->data == x0) ++n_items;
            if (n_items >= 2) {
                const int e = run_gemv_group(ctx, &plan.items[ii], n_items, gs, n_g);
                qx_forget(ctx);
                if (e > 0) return e;
                if (e == 0) {
                    ctx->item_seq += n_items - 1;
                    ctx->colq_seq = ctx->item_seq;          // the columns stay valid for a product that follows immediately
                    ii += n_items - 1;
                    continue;
                }
            }
        }
        if (timing) {
            double work = 0;
            struct ggml_tensor * node = ggml_graph_node(gs[0], it.node);
            const int cls = it.kind == PK_LAYER_NORM ? (node_class(node, &work), TC_NORM) : node_class(node, &work);
            t_class->push_back(cls);
            if (cls == TC_MMQ_VEC) {      // the weights cross HBM once per launch group, activations and results once per state
                const double wbytes = (double) ggml_nbytes(node->src[0]);
                t_work->push_back(wbytes + (work - wbytes) * n_g);
            } else {
                t_work->push_back(work * n_g);
            }
            if (*n_ev == 0) cudaEventRecord(next_event(), ctx->stream);      // one event per item boundary: item k runs between events k and k+1
        }
        const int e = run_item(ctx, it, gs, n_g);
        if (n_g > 1) qx_forget(ctx);
        else for (int nd = it.node; nd <= it.last; ++nd) qx_note_write(ctx, ggml_graph_node(gs[0], nd));      // an overwritten source is quantised again
        if (timing) cudaEventRecord(next_event(), ctx->stream);
        if (e != 0) {
            struct ggml_tensor * node = ggml_graph_node(gs[0], it.node);
            fprintf(stderr, "ggml-b200: node %d %s (%s) failed with code %d (%s)\n", it.node, node->name, ggml_op_name(node->op), e,
                    e < 10000 ? cudaGetErrorString((cudaError_t) e) : "argument error");
            return e;
        }
    }
    return 0;
}

// Test hook (no device work): builds the fused plan of `plan_graph` and says whether `candidate`, a graph with the same
// signature, may run on it.  Returns -1 when the signatures differ, else bit 0 = fits, bit 1 = the plan fuses something.
extern "C" int b200_plan_probe(struct ggml_cgraph * plan_graph, struct ggml_cgraph * candidate) {
    if (!plan_graph || !candidate) return -2;
    if (graph_signature(plan_graph) != graph_signature(candidate)) return -1;
    exec_plan plan;
    build_plan(plan_graph, plan, true);
    int fused = 0;
    for (const plan_item & it : plan.items) if (it.last != it.node) fused = 2;
    return (graph_fits_plan(plan, candidate) ? 1 : 0) | fused;
}

// ---------------------------------------------------------------------------------------------
// Cross-state batching of decode steps.  Every whisper_state owns a backend instance and a host thread; their
// single-token decode graphs arrive here independently.  Threads that arrive within a short window hand their
// graph to one of them (the leader), which launches every item once for the whole group on its own stream and
// then lets the others' streams wait on an event.  Columns stay independent, so each state gets exactly the
// bits it would get alone.  The wait is bounded (no thread ever waits on the GPU here, only on a host condition
// variable with a timeout).
// ---------------------------------------------------------------------------------------------
// An event a leader records after a merged step; it goes back to the free list only when every follower that was served
// by that step has made its own stream wait on it, so a follower that is descheduled for a long time can never find the
// event re-recorded by a later batch.
struct batch_event {
    cudaEvent_t      ev = nullptr;
    std::atomic<int> refs{0};
};

struct batch_req {
    b200_backend_ctx *   ctx;
    struct ggml_cgraph * g;
    uint64_t             sig;
    int                  state;     // 0 waiting, 1 done (stream must wait on ev), 2 run it yourself, 3 failed
    batch_event *        ev;
    int                  fits;      // checked against the cached plan by the submitting thread: 1 yes, -1 no, 0 not checked
    // A follower sleeps on its OWN condition variable and only the leader that served it wakes it.  One shared variable
    // with notify_all wakes every waiting thread on every arrival: with 64 states that is thousands of futile wake-ups
    // per step, all queueing for the batcher's mutex in front of the leaders.
    std::condition_variable * cv;
};

struct device_batcher {
    std::mutex              mu;
    std::condition_variable cv;                 // the current leader waits here for arrivals
    std::vector<batch_req *> pending;
    bool                    leader_active = false;
    std::vector<batch_event *> free_events;   // events nobody waits on (guarded by mu)
    std::unordered_map<uint64_t, std::shared_ptr<const exec_plan>> plans;      // by signature, fused
    int                     alive = 0;                  // backend instances on this device
    double                  step_ns_ema = 0;            // typical time from "step enqueued" to "next step arrives"

    std::vector<b200_backend_ctx *> members;            // live backend instances on this device
};

static device_batcher g_batchers[B200_MAX_DEVICES];
static int live_backends(int device) { return g_batchers[device].alive; }      // read without the lock: a hint

static void batcher_join(b200_backend_ctx * ctx) {
    device_batcher & B = g_batchers[ctx->device];
    std::lock_guard<std::mutex> lk(B.mu);
    B.members.push_back(ctx);
    B.alive = (int) B.members.size();
}
static void batcher_leave(b200_backend_ctx * ctx) {
    device_batcher & B = g_batchers[ctx->device];
    std::lock_guard<std::mutex> lk(B.mu);
    for (size_t i = 0; i < B.members.size(); ++i) if (B.members[i] == ctx) { B.members.erase(B.members.begin() + i); break; }
    B.alive = (int) B.members.size();
}
static std::atomic<int64_t> g_batched_graphs{0}, g_batches{0}, g_ns_lead_wait{0}, g_ns_lead_prep{0}, g_ns_lead_launch{0};
extern "C" int64_t b200_stat_ns_lead_wait(void)   { return g_ns_lead_wait.load(); }
extern "C" int64_t b200_stat_ns_lead_prep(void)   { return g_ns_lead_prep.load(); }
extern "C" int64_t b200_stat_ns_lead_launch(void) { return g_ns_lead_launch.load(); }
extern "C" int64_t b200_stat_batched_graphs(void) { return g_batched_graphs.load(); }
extern "C" int64_t b200_stat_batches(void)        { return g_batches.load(); }

static bool is_decode_graph(struct ggml_cgraph * g) {
    const int n = ggml_graph_n_nodes(g);
    for (int i = 0; i < n; ++i) {
        const struct ggml_tensor * t = ggml_graph_node(g, i);
        if (is_view_op(t->op)) continue;
        return t->op == GGML_OP_GET_ROWS && t->src[1]->ne[0] <= 8 && n > 64;     // decoder graphs start with the token embedding
    }
    return false;
}

static enum ggml_status finish_status(int e) {
    if (e == 0) return GGML_STATUS_SUCCESS;
    return e == (int) cudaErrorMemoryAllocation ? GGML_STATUS_ALLOC_FAILED : GGML_STATUS_FAILED;
}

static enum ggml_status b200_backend_graph_compute(ggml_backend_t backend, struct ggml_cgraph * cgraph) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return GGML_STATUS_FAILED;
    if (ctx->device < 16 && g_sticky_error[ctx->device].load(std::memory_order_relaxed)) {
        fprintf(stderr, "ggml-b200: an earlier tensor copy on device %d failed: refusing to compute on its data\n", ctx->device);
        return GGML_STATUS_FAILED;
    }
    const int64_t t_enter = now_ns();
    static const bool fuse     = getenv("GGML_B200_NO_FUSION") == nullptr;
    static const bool batching = getenv("GGML_B200_NO_BATCHING") == nullptr;
    static const int  window_us = getenv("GGML_B200_BATCH_WINDOW_US") ? atoi(getenv("GGML_B200_BATCH_WINDOW_US")) : 300;
    static const int  max_group = getenv("GGML_B200_MAX_GROUP") && atoi(getenv("GGML_B200_MAX_GROUP")) > 0 ? atoi(getenv("GGML_B200_MAX_GROUP")) : 12;
    const bool timing = g_timing_on.load() != 0;
    device_batcher & B = g_batchers[ctx->device];

    const int n_nodes = ggml_graph_n_nodes(cgraph);
    int64_t n_compute = 0;
    for (int i = 0; i < n_nodes; ++i) {
        struct ggml_tensor * node = ggml_graph_node(cgraph, i);
        if (is_view_op(node->op) || ggml_is_empty(node)) continue;
        if (!b200_op_supported(node)) {
            fprintf(stderr, "ggml-b200: unsupported node %s (%s) reached graph_compute\n", node->name, ggml_op_name(node->op));
            return GGML_STATUS_FAILED;
        }
        ++n_compute;
    }

    const bool decode_graph = is_decode_graph(cgraph);
    if (decode_graph) tl_last_decode_ctx = ctx;      // b200_last_topk answers for the state this thread stepped last
    // ---- batched path -------------------------------------------------------------------------
    if (batching && fuse && B.alive > 1 && decode_graph) {
        std::condition_variable my_cv;
        batch_req req = { ctx, cgraph, graph_signature(cgraph), 0, nullptr, 0, &my_cv };
        const int64_t t_arrive = now_ns();
        ctx->last_decode_ns = t_arrive;
        {   // every thread checks its own graph against the cached plan, in parallel with the others
            std::shared_ptr<const exec_plan> known;
            {
                std::lock_guard<std::mutex> lk0(B.mu);
                auto pit = B.plans.find(req.sig);
                if (pit != B.plans.end()) known = pit->second;
            }
            if (known) req.fits = graph_fits_plan(*known, cgraph) ? 1 : -1;
        }
        std::unique_lock<std::mutex> lk(B.mu);
        {
            const int64_t t_served = ctx->served_ns.exchange(0);
            if (t_served) {     // one full turn of this state: device time of the step plus the host work between steps
                const double turn = (double) (t_arrive - t_served);
                B.step_ns_ema = B.step_ns_ema == 0 ? turn : 0.8 * B.step_ns_ema + 0.2 * turn;
            }
        }
        B.pending.push_back(&req);
        if (B.leader_active) {
            B.cv.notify_one();                                   // the leader (the only waiter on this variable) may be waiting for this arrival
            my_cv.wait(lk, [&] { return req.state != 0; });
            lk.unlock();
            if (req.state == 1) {
                const bool waited = cuda_ok(cudaStreamWaitEvent(ctx->stream, req.ev->ev, 0), "cudaStreamWaitEvent");
                if (req.ev->refs.fetch_sub(1) == 1) {            // last follower of that step: the event may be reused
                    std::lock_guard<std::mutex> lk2(B.mu);
                    B.free_events.push_back(req.ev);
                }
                if (!waited) return GGML_STATUS_FAILED;
                g_nodes_computed += n_compute;
                g_graphs_computed += 1;
                g_host_ns_compute += now_ns() - t_enter;
                return GGML_STATUS_SUCCESS;
            }
            if (req.state == 3) return GGML_STATUS_FAILED;
            // state 2: structure or aliasing did not fit the group's plan - run alone below
        } else {
            B.leader_active = true;
            // how many states are decoding right now?  those that sent a decode graph within the last 20 ms, or within three
            // turns where a turn takes longer than that (per-operator timing switched on, a device shared with encoders)
            int expected = 0;
            const int64_t now = now_ns();
            int64_t recent_ns = 20 * 1000 * 1000;
            if (3.0 * B.step_ns_ema > (double) recent_ns) recent_ns = (int64_t) (3.0 * B.step_ns_ema);
            for (b200_backend_ctx * c : B.members) if (now - c->last_decode_ns < recent_ns) ++expected;
            if (expected > max_group) expected = max_group;     // larger populations run as several groups whose steps overlap on the device
            // States that were served by an earlier batch come back one turn later.  Waiting for them merges the groups:
            // while they are away the device is busy with their step anyway, so the wait costs nothing when the device
            // is the bottleneck, and one merged group needs one pass over the weights instead of one per group.
            int64_t wait_us = window_us;
            if (B.step_ns_ema > 0) {
                const int64_t turn_us = (int64_t) (1.25 * B.step_ns_ema / 1000.0);
                if (turn_us > wait_us) wait_us = turn_us;
                const int64_t cap_us = timing ? 500000 : 20000;      // with per-operator timing a turn takes tens of milliseconds
                if (wait_us > cap_us) wait_us = cap_us;
            }
            const auto deadline = std::chrono::steady_clock::now() + std::chrono::microseconds(wait_us);
            const int64_t t_w0 = now_ns();
            B.cv.wait_until(lk, deadline, [&] { return (int) B.pending.size() >= expected; });
            g_ns_lead_wait += now_ns() - t_w0;
            const int64_t t_p0 = now_ns();
            std::vector<batch_req *> mine;
            mine.swap(B.pending);                                 // everything that is waiting now (may exceed max_group by a few)
            B.leader_active = false;                              // later arrivals elect their own leader
            batch_event * ev = nullptr;
            if (!B.free_events.empty()) { ev = B.free_events.back(); B.free_events.pop_back(); }
            else {
                ev = new batch_event;
                if (cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); delete ev; ev = nullptr; }
            }
            // plan of the leader's structure (cached by signature)
            std::shared_ptr<const exec_plan> plan_sp;
            {
                auto pit = B.plans.find(req.sig);
                if (pit == B.plans.end()) {
                    if (B.plans.size() > 256) B.plans.clear();
                    auto fresh = std::make_shared<exec_plan>();
                    build_plan(cgraph, *fresh, true);
                    plan_sp = fresh;
                    B.plans[req.sig] = plan_sp;
                    req.fits = 0;                                   // not yet checked against this plan
                } else {
                    plan_sp = pit->second;
                }
            }
            const exec_plan & plan_copy = *plan_sp;
            lk.unlock();

            std::vector<struct ggml_cgraph *> gs;
            std::vector<batch_req *> served;
            int rc = 0;
            auto fits = [&](batch_req * r) { return r->fits != 0 ? r->fits > 0 : graph_fits_plan(plan_copy, r->g); };
            if (fits(&req)) {
                gs.push_back(cgraph);
                for (batch_req * r : mine) {
                    if (r == &req) continue;
                    if (r->sig == req.sig && fits(r)) { gs.push_back(r->g); served.push_back(r); }
                }
                size_t n_ev = 0;
                g_ns_lead_prep += now_ns() - t_p0;
                const int64_t t_l0 = now_ns();
                std::vector<int>    bt_class;
                std::vector<double> bt_work;
                rc = run_plan(ctx, plan_copy, gs.data(), (int) gs.size(), timing, &bt_class, &bt_work, &n_ev);
                if (rc == 0 && (g_topk_k.load() > 0 || g_skip_logits_readback.load())) {
                    std::vector<b200_backend_ctx *> owners;
                    owners.push_back(ctx);
                    for (batch_req * r : served) owners.push_back(r->ctx);
                    rc = logits_side_output(ctx, gs.data(), owners.data(), (int) gs.size());
                }
                g_ns_lead_launch += now_ns() - t_l0;
                if (rc == 0 && timing && !bt_class.empty() && cudaStreamSynchronize(ctx->stream) == cudaSuccess) {
                    std::lock_guard<std::mutex> tl(g_timing_mu);
                    for (size_t k = 0; k < bt_class.size(); ++k) {
                        float ms = 0;
                        cudaEventElapsedTime(&ms, ctx->events[k], ctx->events[k + 1]);
                        g_tc_ms[bt_class[k]] += ms;
                        g_tc_work[bt_class[k]] += bt_work[k];
                        g_tc_count[bt_class[k]] += 1;
                    }
                }
                if (rc == 0 && !served.empty()) {
                    if (!ev) rc = (int) cudaErrorMemoryAllocation;
                    else {
                        ev->refs = (int) served.size();
                        rc = cudaEventRecord(ev->ev, ctx->stream) == cudaSuccess ? 0 : (int) cudaGetLastError();
                    }
                }
                g_batched_graphs += (int64_t) gs.size();
                g_batches += 1;
            } else {
                rc = -1;                                          // leader's own graph does not fit: everybody runs alone
            }
            lk.lock();
            if (ev && (rc != 0 || served.empty())) B.free_events.push_back(ev);      // nobody is going to wait on it
            const int64_t t_done = now_ns();
            if (rc == 0) ctx->served_ns = t_done;
            for (batch_req * r : mine) {
                if (r == &req) continue;
                bool was_served = false;
                for (batch_req * s : served) if (s == r) was_served = true;
                if (was_served) { r->ev = ev; r->state = rc == 0 ? 1 : 3; if (rc == 0) r->ctx->served_ns = t_done; }
                else r->state = 2;
                r->cv->notify_one();                              // under the lock: the request lives on its owner's stack until it sees its state
            }
            lk.unlock();
            if (rc == 0) {
                g_nodes_computed += n_compute;
                g_graphs_computed += 1;
                g_host_ns_compute += now_ns() - t_enter;
                return GGML_STATUS_SUCCESS;
            }
            if (rc > 0) return finish_status(rc);
            // rc == -1: fall through to the plain path
        }
    }

    // ---- plain path: this graph alone ------------------------------------------------------------
    exec_plan plan;
    {
        // plans are cached by structure signature (building one walks the graph with a hash map)
        const uint64_t sig = graph_signature(cgraph) ^ (fuse ? 0 : 0x9e3779b97f4a7c15ull);
        bool have = false;
        {
            std::lock_guard<std::mutex> lk(B.mu);
            auto pit = B.plans.find(sig);
            if (pit != B.plans.end()) { plan = *pit->second; have = true; }
        }
        if (!have) {
            build_plan(cgraph, plan, fuse);
            std::lock_guard<std::mutex> lk(B.mu);
            if (B.plans.size() > 256) B.plans.clear();
            B.plans[sig] = std::make_shared<exec_plan>(plan);
        }
    }
    if (fuse && !graph_fits_plan(plan, cgraph)) build_plan(cgraph, plan, false);     // aliasing hazard somewhere: node by node
    std::vector<int>    t_class;
    std::vector<double> t_work;
    size_t n_ev = 0;
    struct ggml_cgraph * one[1] = { cgraph };
    int e = run_plan(ctx, plan, one, 1, timing, &t_class, &t_work, &n_ev);
    if (e == 0 && decode_graph && (g_topk_k.load() > 0 || g_skip_logits_readback.load())) {
        b200_backend_ctx * owner[1] = { ctx };
        e = logits_side_output(ctx, one, owner, 1);
    }
    if (e != 0) return finish_status(e);
    g_nodes_computed += n_compute;
    g_graphs_computed += 1;
    g_host_ns_compute += now_ns() - t_enter;
    if (timing && !t_class.empty()) {
        if (!cuda_ok(cudaStreamSynchronize(ctx->stream), "timing sync")) return GGML_STATUS_FAILED;
        std::lock_guard<std::mutex> lk(g_timing_mu);
        for (size_t k = 0; k < t_class.size(); ++k) {
            float ms = 0;
            cudaEventElapsedTime(&ms, ctx->events[k], ctx->events[k + 1]);
            g_tc_ms[t_class[k]] += ms;
            g_tc_work[t_class[k]] += t_work[k];
            g_tc_count[t_class[k]] += 1;
        }
    }
    return GGML_STATUS_SUCCESS;
}

static const struct ggml_backend_i b200_backend_iface = {
    /* .get_name           = */ b200_backend_get_name,
    /* .free               = */ b200_backend_free,
    /* .set_tensor_async   = */ nullptr,
    /* .get_tensor_async   = */ nullptr,
    /* .cpy_tensor_async   = */ nullptr,
    /* .synchronize        = */ b200_backend_synchronize,
    /* .graph_plan_create  = */ nullptr,
    /* .graph_plan_free    = */ nullptr,
    /* .graph_plan_update  = */ nullptr,
    /* .graph_plan_compute = */ nullptr,
    /* .graph_compute      = */ b200_backend_graph_compute,
    /* .event_record       = */ nullptr,
    /* .event_wait         = */ nullptr,
};

static ggml_guid_t b200_guid() {
    static ggml_guid guid = {0xb2, 0x00, 0x5a, 0x10, 0x0a, 0x77, 0x68, 0x73, 0x70, 0x72, 0x2d, 0x62, 0x32, 0x30, 0x30, 0x01};
    return &guid;
}

// ---------------------------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------------------------
static const char * b200_dev_get_name(ggml_backend_dev_t dev)        { return ((b200_device_ctx *) dev->context)->name.c_str(); }
static const char * b200_dev_get_description(ggml_backend_dev_t dev) { return ((b200_device_ctx *) dev->context)->description.c_str(); }

static void b200_dev_get_memory(ggml_backend_dev_t dev, size_t * free, size_t * total) {
    b200_device_ctx * ctx = (b200_device_ctx *) dev->context;
    *free = 0; *total = 0;
    if (cudaSetDevice(ctx->device) == cudaSuccess) cudaMemGetInfo(free, total);
}

static enum ggml_backend_dev_type b200_dev_get_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_GPU; }

static void b200_dev_get_props(ggml_backend_dev_t dev, struct ggml_backend_dev_props * props) {
    props->name        = b200_dev_get_name(dev);
    props->description = b200_dev_get_description(dev);
    props->type        = GGML_BACKEND_DEVICE_TYPE_GPU;
    b200_dev_get_memory(dev, &props->memory_free, &props->memory_total);
    props->caps = { /* async */ true, /* host_buffer */ false, /* buffer_from_host_ptr */ false, /* events */ false };
}

static ggml_backend_t b200_dev_init_backend(ggml_backend_dev_t dev, const char *) {
    b200_device_ctx * dctx = (b200_device_ctx *) dev->context;
    if (!cuda_ok(cudaSetDevice(dctx->device), "cudaSetDevice")) return nullptr;
    b200_backend_ctx * ctx = new b200_backend_ctx;
    ctx->device = dctx->device;
    ctx->name   = dctx->name;
    if (!cuda_ok(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking), "cudaStreamCreate")) { delete ctx; return nullptr; }
    if (!cuda_ok(cudaMalloc(&ctx->colq, (size_t) COLQ_MAX_COLS * COLQ_MAX_K + (size_t) COLQ_MAX_COLS * (COLQ_MAX_K / 32) * 4), "cudaMalloc(colq)")) {
        cudaStreamDestroy(ctx->stream); delete ctx; return nullptr;
    }
    if (cudaEventCreateWithFlags(&ctx->sync_event, cudaEventBlockingSync | cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); ctx->sync_event = nullptr; }
    {
        static const bool zero_copy = getenv("GGML_B200_TOPK_DEVICE") == nullptr;
        void * hp = nullptr, * dp = nullptr;
        if (zero_copy && cudaHostAlloc(&hp, 8 * sizeof(b200_topk_result), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess &&
            cudaHostGetDevicePointer(&dp, hp, 0) == cudaSuccess) {
            memset(hp, 0, 8 * sizeof(b200_topk_result));
            ctx->topk_host = (b200_topk_result *) hp;
            ctx->topk = (b200_topk_result *) dp;
        } else {
            cudaGetLastError();
            if (hp) cudaFreeHost(hp);
            if (cudaMalloc((void **) &ctx->topk, 8 * sizeof(b200_topk_result)) != cudaSuccess) { cudaGetLastError(); ctx->topk = nullptr; }
        }
    }
    // activation scratch of the many-column products, sized here for Whisper's largest product (1500 columns of 5120
    // values) so that graph_compute does not allocate on its usual path; it still grows on demand for larger graphs
    ensure_scratch(ctx, (size_t) 1536 * 5120 + (size_t) 1536 * (5120 / 32) * 4);
    batcher_join(ctx);
    return new ggml_backend{ b200_guid(), b200_backend_iface, dev, ctx };
}

static ggml_backend_buffer_type_t b200_dev_get_buffer_type(ggml_backend_dev_t dev) {
    return &((b200_device_ctx *) dev->context)->buft;
}

static bool b200_op_supported(const struct ggml_tensor * op) {
    const struct ggml_tensor * s0 = op->src[0];
    const struct ggml_tensor * s1 = op->src[1];
    switch (op->op) {
        case GGML_OP_NONE: case GGML_OP_RESHAPE: case GGML_OP_VIEW: case GGML_OP_PERMUTE: case GGML_OP_TRANSPOSE:
            return true;
        case GGML_OP_MUL_MAT:
            if (op->type != GGML_TYPE_F32 || op->nb[0] != 4) return false;
            if (is_quant(s0->type)) {
                return s0->view_src == nullptr && ggml_is_contiguous(s0) && s0->ne[2] == 1 && s0->ne[3] == 1 &&
                       s1->type == GGML_TYPE_F32 && s1->nb[0] == 4 && s1->ne[2] == 1 && s1->ne[3] == 1 &&
                       s1->ne[0] % 32 == 0 && (s1->nb[1] % 16) == 0;
            }
            if (s0->type == GGML_TYPE_F16) {
                return s0->nb[0] == 2 && ((s1->type == GGML_TYPE_F32 && s1->nb[0] == 4) || (s1->type == GGML_TYPE_F16 && s1->nb[0] == 2)) &&
                       s1->ne[2] % s0->ne[2] == 0 && s1->ne[3] % s0->ne[3] == 0 && s1->ne[2] * s1->ne[3] <= 65535;
            }
            return false;
        case GGML_OP_FLASH_ATTN_EXT: {
            const struct ggml_tensor * k = op->src[1], * v = op->src[2], * mask = op->src[3];
            float max_bias, softcap;
            memcpy(&max_bias, (const float *) op->op_params + 1, sizeof(float));
            memcpy(&softcap,  (const float *) op->op_params + 2, sizeof(float));
            return s0->type == GGML_TYPE_F32 && k->type == GGML_TYPE_F16 && v->type == GGML_TYPE_F16 &&
                   s0->ne[0] == 64 && k->ne[0] == 64 && v->ne[0] == 64 && s0->ne[3] == 1 && k->ne[3] == 1 && v->ne[3] == 1 &&
                   k->ne[2] == s0->ne[2] && v->ne[2] == s0->ne[2] && k->ne[1] == v->ne[1] &&
                   s0->nb[0] == 4 && k->nb[0] == 2 && v->nb[0] == 2 && max_bias == 0.0f && softcap == 0.0f &&
                   (!mask || (mask->type == GGML_TYPE_F16 && mask->nb[0] == 2 && mask->ne[0] >= k->ne[1] && mask->ne[1] >= s0->ne[1]));
        }
        case GGML_OP_NORM:
            return s0->type == GGML_TYPE_F32 && s0->nb[0] == 4 && op->nb[0] == 4;
        case GGML_OP_ADD:
        case GGML_OP_MUL:
            return s0->type == GGML_TYPE_F32 && s1->type == GGML_TYPE_F32 && op->type == GGML_TYPE_F32 && ggml_can_repeat(s1, s0);
        case GGML_OP_SCALE:
            return s0->type == GGML_TYPE_F32 && ggml_is_contiguous(s0) && ggml_is_contiguous(op);
        case GGML_OP_UNARY:
            return ggml_get_unary_op(op) == GGML_UNARY_OP_GELU && s0->type == GGML_TYPE_F32 && ggml_is_contiguous(s0) && ggml_is_contiguous(op);
        case GGML_OP_CPY:
        case GGML_OP_DUP:
        case GGML_OP_CONT: {
            const enum ggml_type a = s0->type, b = op->type;
            return (a == GGML_TYPE_F32 && (b == GGML_TYPE_F32 || b == GGML_TYPE_F16)) ||
                   (a == GGML_TYPE_F16 && (b == GGML_TYPE_F32 || b == GGML_TYPE_F16)) || (a == GGML_TYPE_I32 && b == GGML_TYPE_I32);
        }
        case GGML_OP_GET_ROWS:
            if (s1->type != GGML_TYPE_I32 || s1->ne[1] != 1 || s1->ne[2] != 1 || !ggml_is_contiguous(s1)) return false;
            if (is_quant(s0->type)) return s0->view_src == nullptr && ggml_is_contiguous(s0) && s0->ne[2] == 1 && s0->ne[3] == 1;
            return (s0->type == GGML_TYPE_F16 || s0->type == GGML_TYPE_F32) && s0->ne[2] == 1 && s0->ne[3] == 1;
        case GGML_OP_IM2COL: {
            const int32_t * p = (const int32_t *) op->op_params;
            return p[6] == 0 && op->type == GGML_TYPE_F16 && s1->type == GGML_TYPE_F32 && s1->nb[0] == 4 && s1->ne[2] == 1 && s1->ne[3] == 1;
        }
        case GGML_OP_SOFT_MAX: {
            float max_bias;
            memcpy(&max_bias, (const float *) op->op_params + 1, sizeof(float));
            return max_bias == 0.0f && s0->type == GGML_TYPE_F32 && ggml_is_contiguous(s0) && ggml_is_contiguous(op) &&
                   (!s1 || ((s1->type == GGML_TYPE_F32 || s1->type == GGML_TYPE_F16) && ggml_is_contiguous(s1)));
        }
        case GGML_OP_CONCAT:
            return s0->type == GGML_TYPE_F32 && s1->type == GGML_TYPE_F32;
        default:
            return false;
    }
}

static bool b200_dev_supports_op(ggml_backend_dev_t, const struct ggml_tensor * op) { return b200_op_supported(op); }

static bool b200_dev_supports_buft(ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    return buft == &((b200_device_ctx *) dev->context)->buft;
}

static const struct ggml_backend_device_i b200_device_iface = {
    /* .get_name             = */ b200_dev_get_name,
    /* .get_description      = */ b200_dev_get_description,
    /* .get_memory           = */ b200_dev_get_memory,
    /* .get_type             = */ b200_dev_get_type,
    /* .get_props            = */ b200_dev_get_props,
    /* .init_backend         = */ b200_dev_init_backend,
    /* .get_buffer_type      = */ b200_dev_get_buffer_type,
    /* .get_host_buffer_type = */ nullptr,
    /* .buffer_from_host_ptr = */ nullptr,
    /* .supports_op          = */ b200_dev_supports_op,
    /* .supports_buft        = */ b200_dev_supports_buft,
    /* .offload_op           = */ nullptr,
    /* .event_new            = */ nullptr,
    /* .event_free           = */ nullptr,
    /* .event_synchronize    = */ nullptr,
};

// ---------------------------------------------------------------------------------------------
// registry
// ---------------------------------------------------------------------------------------------
struct b200_reg_ctx {
    std::vector<ggml_backend_device *> devices;
};

static const char * b200_reg_get_name(ggml_backend_reg_t) { return "B200"; }
static size_t b200_reg_get_device_count(ggml_backend_reg_t reg) { return ((b200_reg_ctx *) reg->context)->devices.size(); }
static ggml_backend_dev_t b200_reg_get_device(ggml_backend_reg_t reg, size_t index) {
    b200_reg_ctx * ctx = (b200_reg_ctx *) reg->context;
    GGML_ASSERT(index < ctx->devices.size());
    return ctx->devices[index];
}

static struct ggml_backend_feature * b200_get_features(ggml_backend_reg_t) {
    static struct ggml_backend_feature features[] = {
        { "ARCH", "sm_100a" },
        { "CPU_PARITY", "avx2-fma-f16c" },
        { nullptr, nullptr },
    };
    return features;
}

extern "C" {
GGML_BACKEND_API void b200_logits_side_output(int top_k, int skip_readback) {
    g_topk_k = top_k < 0 ? 0 : (top_k > B200_TOPK_MAX ? B200_TOPK_MAX : top_k);
    g_skip_logits_readback = (skip_readback != 0 && top_k > 0) ? 1 : 0;
}
GGML_BACKEND_API int b200_last_topk(int row, b200_topk_result * out) {
    b200_backend_ctx * ctx = tl_last_decode_ctx;
    if (!ctx || !out || !ctx->topk || row < 0 || row >= ctx->topk_rows) return B200_ERR_ARG;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return (int) cudaGetLastError();
    // the side output was enqueued on the stream that ran the graph; this instance's stream is ordered behind it
    cudaError_t e;
    if (ctx->topk_host) {      // written by the kernel into host memory: visible once the stream is known to be idle
        e = cudaStreamQuery(ctx->stream);
        if (e == cudaErrorNotReady) { cudaGetLastError(); e = stream_wait_blocking(ctx->stream); }
        if (e == cudaSuccess) memcpy(out, ctx->topk_host + row, sizeof(*out));
    } else {
        e = cudaMemcpyAsync(out, ctx->topk + row, sizeof(*out), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = stream_wait_blocking(ctx->stream);
    }
    if (e != cudaSuccess) { cudaGetLastError(); return (int) e; }
    g_d2h_bytes += (int64_t) sizeof(*out);
    return 0;
}
}

static void * b200_reg_get_proc_address(ggml_backend_reg_t, const char * name) {
    if (strcmp(name, "ggml_backend_get_features") == 0) return (void *) b200_get_features;
    if (strcmp(name, "b200_logits_side_output") == 0) return (void *) b200_logits_side_output;
    if (strcmp(name, "b200_last_topk") == 0)          return (void *) b200_last_topk;
    if (strcmp(name, "b200_stat_nodes") == 0)  return (void *) b200_stat_nodes;
    if (strcmp(name, "b200_stat_graphs") == 0) return (void *) b200_stat_graphs;
    if (strcmp(name, "b200_stat_h2d") == 0)    return (void *) b200_stat_h2d;
    if (strcmp(name, "b200_stat_d2h") == 0)    return (void *) b200_stat_d2h;
    if (strcmp(name, "b200_stat_host_ns_compute") == 0) return (void *) b200_stat_host_ns_compute;
    if (strcmp(name, "b200_stat_host_ns_sync") == 0)    return (void *) b200_stat_host_ns_sync;
    if (strcmp(name, "b200_stat_batched_graphs") == 0)  return (void *) b200_stat_batched_graphs;
    if (strcmp(name, "b200_stat_batches") == 0)         return (void *) b200_stat_batches;
    if (strcmp(name, "b200_stat_ns_lead_wait") == 0)    return (void *) b200_stat_ns_lead_wait;
    if (strcmp(name, "b200_stat_ns_lead_prep") == 0)    return (void *) b200_stat_ns_lead_prep;
    if (strcmp(name, "b200_stat_ns_lead_launch") == 0)  return (void *) b200_stat_ns_lead_launch;
    if (strcmp(name, "b200_launch_count") == 0) return (void *) b200_launch_count;
    if (strcmp(name, "b200_timing_enable") == 0)  return (void *) b200_timing_enable;
    if (strcmp(name, "b200_timing_reset") == 0)   return (void *) b200_timing_reset;
    if (strcmp(name, "b200_timing_classes") == 0) return (void *) b200_timing_classes;
    if (strcmp(name, "b200_timing_name") == 0)    return (void *) b200_timing_name;
    if (strcmp(name, "b200_timing_get") == 0)     return (void *) b200_timing_get;
    return nullptr;
}

static const struct ggml_backend_reg_i b200_reg_iface = {
    /* .get_name         = */ b200_reg_get_name,
    /* .get_device_count = */ b200_reg_get_device_count,
    /* .get_device       = */ b200_reg_get_device,
    /* .get_proc_address = */ b200_reg_get_proc_address,
};

static int b200_visible_devices() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n > B200_MAX_DEVICES ? B200_MAX_DEVICES : n;
}

extern "C" {

GGML_BACKEND_API int ggml_backend_score(void) {
    // 0 = "not supported on this system": without a CUDA device the plugin refuses to load,
    // it never computes on the host.
    return b200_visible_devices() > 0 ? 100 : 0;
}

GGML_BACKEND_API ggml_backend_reg_t ggml_backend_init(void) {
    static std::mutex mu;
    static ggml_backend_reg reg;
    static bool initialised = false;
    std::lock_guard<std::mutex> lk(mu);
    if (!initialised) {
        b200_reg_ctx * ctx = new b200_reg_ctx;
        const int n = b200_visible_devices();
        for (int i = 0; i < n; ++i) {
            cudaDeviceProp prop;
            if (cudaGetDeviceProperties(&prop, i) != cudaSuccess) continue;
            if (prop.major != 10) {
                fprintf(stderr, "ggml-b200: device %d (%s, sm_%d%d) is not sm_100: skipped\n", i, prop.name, prop.major, prop.minor);
                continue;
            }
            b200_device_ctx * dctx = new b200_device_ctx;
            dctx->device      = i;
            dctx->name        = "B200_" + std::to_string(i);
            dctx->description = prop.name;
            dctx->buft_name   = dctx->name;
            ggml_backend_device * dev = new ggml_backend_device{ b200_device_iface, &reg, dctx };
            dctx->buft = { { b200_buft_get_name, b200_buft_alloc_buffer, b200_buft_get_alignment, nullptr, nullptr, b200_buft_is_host }, dev, dctx };
            ctx->devices.push_back(dev);
        }
        reg = ggml_backend_reg{ GGML_BACKEND_API_VERSION, b200_reg_iface, ctx };
        initialised = true;
    }
    return &reg;
}

}
