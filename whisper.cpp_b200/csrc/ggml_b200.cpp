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
#include <mutex>
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
enum b200_timing_class { TC_MMQ_VEC = 0, TC_MMQ_GEMM, TC_MM_F16, TC_FATTN, TC_NORM, TC_BINARY, TC_SCALE, TC_GELU, TC_CPY,
                         TC_GET_ROWS, TC_IM2COL, TC_SOFT_MAX, TC_CONCAT, TC_COUNT };
static const char * const g_tc_names[TC_COUNT] = { "mul_mat_vec_q", "mul_mat_q", "mul_mat_f16", "flash_attn_ext", "norm", "binary",
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

// ---------------------------------------------------------------------------------------------
// buffer
// ---------------------------------------------------------------------------------------------
struct b200_buffer_ctx {
    int    device;
    void * base;
};

static void b200_buffer_free(ggml_backend_buffer_t buffer) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    cudaFree(ctx->base);
    delete ctx;
}

static void * b200_buffer_get_base(ggml_backend_buffer_t buffer) {
    return ((b200_buffer_ctx *) buffer->context)->base;
}

static void b200_buffer_memset_tensor(ggml_backend_buffer_t buffer, struct ggml_tensor * tensor, uint8_t value, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    cuda_ok(cudaMemsetAsync((char *) tensor->data + offset, value, size, cudaStreamPerThread), "memset_tensor");
    cuda_ok(cudaStreamSynchronize(cudaStreamPerThread), "memset_tensor sync");
}

// Block-quantised tensors live in device memory as planes (see b200_whisper.h); set/get translate.
static void b200_buffer_set_tensor(ggml_backend_buffer_t buffer, struct ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    g_h2d_bytes += (int64_t) size;
    if (is_quant(tensor->type)) {
        const size_t  bs = ggml_type_size(tensor->type);
        const int64_t nb_total = (int64_t) (ggml_nbytes(tensor) / bs);
        GGML_ASSERT(tensor->view_src == nullptr && "ggml-b200: views of block-quantised tensors are not supported");
        GGML_ASSERT(offset % bs == 0 && size % bs == 0);
        const int64_t first = (int64_t) (offset / bs), count = (int64_t) (size / bs);
        // repack into a host image of the touched plane ranges, then copy each range
        const size_t qsz = tensor->type == GGML_TYPE_Q5_0 ? 16 : 32;
        std::vector<uint8_t> qs(count * qsz), qh(tensor->type == GGML_TYPE_Q5_0 ? count * 4 : 0), d(count * 2);
        const uint8_t * src = (const uint8_t *) data;
        for (int64_t i = 0; i < count; ++i) {
            const uint8_t * b = src + bs * i;
            memcpy(&d[2 * i], b, 2);
            if (tensor->type == GGML_TYPE_Q5_0) {
                memcpy(&qh[4 * i], b + 2, 4);
                memcpy(&qs[16 * i], b + 6, 16);
            } else {
                memcpy(&qs[32 * i], b + 2, 32);
            }
        }
        char * base = (char *) tensor->data;
        cudaStream_t st = cudaStreamPerThread;
        bool ok = cuda_ok(cudaMemcpyAsync(base + qsz * first, qs.data(), qs.size(), cudaMemcpyHostToDevice, st), "set_tensor qs");
        if (tensor->type == GGML_TYPE_Q5_0) {
            ok = ok && cuda_ok(cudaMemcpyAsync(base + 16 * nb_total + 4 * first, qh.data(), qh.size(), cudaMemcpyHostToDevice, st), "set_tensor qh");
            ok = ok && cuda_ok(cudaMemcpyAsync(base + 20 * nb_total + 2 * first, d.data(), d.size(), cudaMemcpyHostToDevice, st), "set_tensor d");
        } else {
            ok = ok && cuda_ok(cudaMemcpyAsync(base + 32 * nb_total + 2 * first, d.data(), d.size(), cudaMemcpyHostToDevice, st), "set_tensor d");
        }
        cuda_ok(cudaStreamSynchronize(st), "set_tensor sync");
        GGML_ASSERT(ok);
        return;
    }
    bool ok = cuda_ok(cudaMemcpyAsync((char *) tensor->data + offset, data, size, cudaMemcpyHostToDevice, cudaStreamPerThread), "set_tensor");
    ok = ok && cuda_ok(cudaStreamSynchronize(cudaStreamPerThread), "set_tensor sync");
    GGML_ASSERT(ok);
}

static void b200_buffer_get_tensor(ggml_backend_buffer_t buffer, const struct ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
    g_d2h_bytes += (int64_t) size;
    if (is_quant(tensor->type)) {
        const size_t  bs = ggml_type_size(tensor->type);
        const int64_t nb_total = (int64_t) (ggml_nbytes(tensor) / bs);
        GGML_ASSERT(tensor->view_src == nullptr);
        GGML_ASSERT(offset % bs == 0 && size % bs == 0);
        const int64_t first = (int64_t) (offset / bs), count = (int64_t) (size / bs);
        const size_t qsz = tensor->type == GGML_TYPE_Q5_0 ? 16 : 32;
        std::vector<uint8_t> qs(count * qsz), qh(tensor->type == GGML_TYPE_Q5_0 ? count * 4 : 0), d(count * 2);
        const char * base = (const char *) tensor->data;
        cudaStream_t st = cudaStreamPerThread;
        bool ok = cuda_ok(cudaMemcpyAsync(qs.data(), base + qsz * first, qs.size(), cudaMemcpyDeviceToHost, st), "get_tensor qs");
        if (tensor->type == GGML_TYPE_Q5_0) {
            ok = ok && cuda_ok(cudaMemcpyAsync(qh.data(), base + 16 * nb_total + 4 * first, qh.size(), cudaMemcpyDeviceToHost, st), "get_tensor qh");
            ok = ok && cuda_ok(cudaMemcpyAsync(d.data(), base + 20 * nb_total + 2 * first, d.size(), cudaMemcpyDeviceToHost, st), "get_tensor d");
        } else {
            ok = ok && cuda_ok(cudaMemcpyAsync(d.data(), base + 32 * nb_total + 2 * first, d.size(), cudaMemcpyDeviceToHost, st), "get_tensor d");
        }
        ok = ok && cuda_ok(cudaStreamSynchronize(st), "get_tensor sync");
        GGML_ASSERT(ok);
        uint8_t * dst = (uint8_t *) data;
        for (int64_t i = 0; i < count; ++i) {
            uint8_t * b = dst + bs * i;
            memcpy(b, &d[2 * i], 2);
            if (tensor->type == GGML_TYPE_Q5_0) {
                memcpy(b + 2, &qh[4 * i], 4);
                memcpy(b + 6, &qs[16 * i], 16);
            } else {
                memcpy(b + 2, &qs[32 * i], 32);
            }
        }
        return;
    }
    bool ok = cuda_ok(cudaMemcpyAsync(data, (const char *) tensor->data + offset, size, cudaMemcpyDeviceToHost, cudaStreamPerThread), "get_tensor");
    ok = ok && cuda_ok(cudaStreamSynchronize(cudaStreamPerThread), "get_tensor sync");
    GGML_ASSERT(ok);
}

static void b200_buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    cudaSetDevice(ctx->device);
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
};

static const char * b200_backend_get_name(ggml_backend_t backend) {
    return ((b200_backend_ctx *) backend->context)->name.c_str();
}

static void b200_backend_free(ggml_backend_t backend) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (cudaEvent_t e : ctx->events) cudaEventDestroy(e);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    delete backend;
}

static void b200_backend_synchronize(ggml_backend_t backend) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    cudaSetDevice(ctx->device);
    const int64_t t0 = now_ns();
    cuda_ok(cudaStreamSynchronize(ctx->stream), "synchronize");
    g_host_ns_sync += now_ns() - t0;
}

static bool ensure_scratch(b200_backend_ctx * ctx, size_t size) {
    if (ctx->scratch_size >= size) return true;
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
                const size_t q_bytes = (size_t) N * K, d_bytes = (size_t) N * (K / 32) * 4;
                const size_t q_pad = (q_bytes + 255) & ~(size_t) 255;
                if (!ensure_scratch(ctx, q_pad + d_bytes)) return (int) cudaErrorMemoryAllocation;
                int8_t * xq = (int8_t *) ctx->scratch;
                float *  xd = (float *) ((char *) ctx->scratch + q_pad);
                int e = b200_quantize_q8_0((const float *) s1->data, N, K, nb1[1], xq, xd, st);
                if (e) return e;
                return b200_mul_mat_q((int) s0->type, s0->data, nb_total, M, K, xq, xd, N, (float *) node->data, nbd[1] / 4, st);
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
// node-sequence fusion.  A fused launch evaluates the same single-precision operations in the same
// order as the node sequence it replaces, so the bits that reach memory do not change; what goes
// away is the round trip of the intermediate through HBM and the extra launches.
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

// NORM -> MUL(gamma) -> ADD(beta) starting at node i; returns the index of the ADD node or -1
static int match_layer_norm(struct ggml_cgraph * g, const graph_info & gi, int i, const struct ggml_tensor ** gamma, const struct ggml_tensor ** beta) {
    const int n = ggml_graph_n_nodes(g);
    struct ggml_tensor * nrm = ggml_graph_node(g, i);
    if (i + 2 >= n || !only_feeds(gi, nrm, i)) return -1;
    struct ggml_tensor * mul = ggml_graph_node(g, i + 1);
    struct ggml_tensor * add = ggml_graph_node(g, i + 2);
    if (mul->op != GGML_OP_MUL || add->op != GGML_OP_ADD || mul->src[0] != nrm || add->src[0] != mul || !only_feeds(gi, mul, i + 1)) return -1;
    const struct ggml_tensor * ga = mul->src[1], * be = add->src[1], * x = nrm->src[0];
    auto vec_ok = [&](const struct ggml_tensor * v) {
        return v->type == GGML_TYPE_F32 && v->ne[0] == x->ne[0] && v->ne[1] == 1 && v->ne[2] == 1 && v->ne[3] == 1 && v->nb[0] == 4;
    };
    if (!vec_ok(ga) || !vec_ok(be) || !ready_before(gi, ga, i) || !ready_before(gi, be, i)) return -1;
    if (x->ne[2] != 1 || x->ne[3] != 1 || x->nb[0] != 4 || add->nb[0] != 4 || !ggml_are_same_shape(x, add)) return -1;
    *gamma = ga; *beta = be;
    return i + 2;
}

// MUL_MAT (quantised weights, <= 8 columns) followed by ADD / SCALE / GELU nodes and an optional F32->F16 CPY.
// Fills ep, *last = index of the last fused node, *out = tensor whose memory receives the result.
static void match_vec_epilogue(struct ggml_cgraph * g, const graph_info & gi, int i, b200_epilogue * ep, int * last, struct ggml_tensor ** out,
                               std::vector<char> & fused, const struct ggml_tensor ** operands) {
    const int n = ggml_graph_n_nodes(g);
    struct ggml_tensor * cur = ggml_graph_node(g, i);
    const int64_t M = cur->ne[0], N = cur->ne[1];
    int cur_pos = i;
    ep->n_steps = 0; ep->store_f16 = 0;
    *last = i; *out = cur;
    for (int j = i + 1; j < n && ep->n_steps < 4; ++j) {
        struct ggml_tensor * t = ggml_graph_node(g, j);
        if (is_view_op(t->op)) {
            if (t->src[0] == cur || t->view_src == cur) break;      // someone looks at cur itself
            continue;
        }
        if (!only_feeds(gi, cur, cur_pos)) break;
        b200_ep_step st = {0, nullptr, 0, 0.0f};
        if (t->op == GGML_OP_ADD && (t->src[0] == cur || t->src[1] == cur) && t->type == GGML_TYPE_F32) {
            const struct ggml_tensor * o = t->src[0] == cur ? t->src[1] : t->src[0];
            if (o == cur || o->type != GGML_TYPE_F32 || o->nb[0] != 4 || o->ne[0] != M || o->ne[2] != 1 || o->ne[3] != 1) break;
            if (o->ne[1] != 1 && o->ne[1] != N) break;
            if (!ggml_are_same_shape(t, cur) || !ready_before(gi, o, i)) break;
            st.kind = B200_EP_ADD; st.ptr = (const float *) o->data; st.stride_n = (o->ne[1] == 1) ? 0 : (int64_t) o->nb[1] / 4;
            operands[ep->n_steps] = o;
        } else if (t->op == GGML_OP_SCALE && t->src[0] == cur) {
            st.kind = B200_EP_SCALE;
            memcpy(&st.scalar, t->op_params, sizeof(float));
        } else if (t->op == GGML_OP_UNARY && t->src[0] == cur && ggml_get_unary_op(t) == GGML_UNARY_OP_GELU) {
            st.kind = B200_EP_GELU;
        } else if (t->op == GGML_OP_CPY && t->src[0] == cur && t->type == GGML_TYPE_F16 && ggml_is_contiguous(t) &&
                   ggml_nelements(t) == M * N && ggml_is_contiguous(cur)) {
            ep->store_f16 = 1;
            fused[j] = 1;
            *last = j; *out = t;
            return;
        } else {
            break;
        }
        if (t->nb[0] != 4) break;
        ep->step[ep->n_steps++] = st;
        fused[j] = 1;
        cur = t; cur_pos = j;
        *last = j; *out = t;
    }
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

static enum ggml_status b200_backend_graph_compute(ggml_backend_t backend, struct ggml_cgraph * cgraph) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return GGML_STATUS_FAILED;
    const int64_t t_enter = now_ns();
    const int n_nodes = ggml_graph_n_nodes(cgraph);
    int64_t done = 0;
    const bool timing = g_timing_on.load() != 0;
    std::vector<int>    t_class;
    std::vector<double> t_work;
    size_t n_ev = 0;
    auto next_event = [&]() -> cudaEvent_t {
        if (n_ev == ctx->events.size()) { cudaEvent_t e; cudaEventCreate(&e); ctx->events.push_back(e); }
        return ctx->events[n_ev++];
    };
    static const bool fuse = getenv("GGML_B200_NO_FUSION") == nullptr;
    graph_info gi;
    std::vector<char> fused(n_nodes, 0);
    if (fuse) analyse_graph(cgraph, gi);
    for (int i = 0; i < n_nodes; ++i) {
        struct ggml_tensor * node = ggml_graph_node(cgraph, i);
        if (is_view_op(node->op) || ggml_is_empty(node)) continue;
        if (fused[i]) { ++done; continue; }
        if (!b200_op_supported(node)) {
            fprintf(stderr, "ggml-b200: unsupported node %s (%s) reached graph_compute\n", node->name, ggml_op_name(node->op));
            return GGML_STATUS_FAILED;
        }
        if (timing) {
            double work = 0;
            t_class.push_back(node_class(node, &work));
            t_work.push_back(work);
            cudaEventRecord(next_event(), ctx->stream);
        }
        int e = -1;
        if (fuse && node->op == GGML_OP_NORM) {
            const struct ggml_tensor * ga = nullptr, * be = nullptr;
            const int last = match_layer_norm(cgraph, gi, i, &ga, &be);
            struct ggml_tensor * out = last > 0 ? ggml_graph_node(cgraph, last) : nullptr;
            const struct ggml_tensor * x = node->src[0];
            // rows are read and written by the same lanes, so exact in-place is fine; a shifted overlap is not
            const bool alias_ok = out && (!overlaps(out, x) || (out->data == x->data && out->nb[1] == x->nb[1]));
            if (last > 0 && alias_ok && b200_op_supported(ggml_graph_node(cgraph, i + 1)) && b200_op_supported(out)) {
                float eps;
                memcpy(&eps, node->op_params, sizeof(float));
                e = b200_layer_norm((const float *) x->data, (const float *) ga->data, (const float *) be->data, (float *) out->data,
                                    x->ne[0], x->ne[1], (int64_t) x->nb[1], (int64_t) out->nb[1], eps, (void *) ctx->stream);
                fused[i + 1] = 1; fused[last] = 1;
            }
        } else if (fuse && node->op == GGML_OP_MUL_MAT && is_quant(node->src[0]->type) && node->src[1]->ne[1] <= 8) {
            b200_epilogue ep;
            int last = i;
            struct ggml_tensor * out = node;
            const struct ggml_tensor * operands[4] = {nullptr, nullptr, nullptr, nullptr};
            match_vec_epilogue(cgraph, gi, i, &ep, &last, &out, fused, operands);
            const struct ggml_tensor * s0 = node->src[0], * s1 = node->src[1];
            bool hazard = out != node && overlaps(out, s1);
            for (int k = 0; k < ep.n_steps; ++k) {
                // an added tensor may share memory with the result only element for element (same thread reads then writes)
                if (operands[k] && overlaps(out, operands[k]) && !(operands[k]->data == out->data && operands[k]->nb[1] == out->nb[1])) hazard = true;
            }
            if (hazard) {
                // the allocator placed the final tensor over the activations, which every CTA still reads: run unfused
                for (int j = i + 1; j <= last; ++j) fused[j] = 0;
                ep.n_steps = 0; ep.store_f16 = 0; out = node;
            }
            const int64_t nb_total = (int64_t) (ggml_nbytes(s0) / ggml_type_size(s0->type));
            const int64_t ldd = ep.store_f16 ? node->ne[0] : (int64_t) out->nb[1] / 4;
            e = b200_mul_mat_vec_q_ep((int) s0->type, s0->data, nb_total, s0->ne[1], s0->ne[0], (const float *) s1->data, (int64_t) s1->nb[1],
                                      s1->ne[1], out->data, ldd, &ep, (void *) ctx->stream);
        }
        if (e == -1) e = compute_node(ctx, node);
        if (timing) cudaEventRecord(next_event(), ctx->stream);
        if (e != 0) {
            fprintf(stderr, "ggml-b200: node %d %s (%s) failed with code %d (%s)\n", i, node->name, ggml_op_name(node->op), e,
                    e < 10000 ? cudaGetErrorString((cudaError_t) e) : "argument error");
            return e == (int) cudaErrorMemoryAllocation ? GGML_STATUS_ALLOC_FAILED : GGML_STATUS_FAILED;
        }
        ++done;
    }
    g_nodes_computed += done;
    g_graphs_computed += 1;
    g_host_ns_compute += now_ns() - t_enter;
    if (timing && !t_class.empty()) {
        if (!cuda_ok(cudaStreamSynchronize(ctx->stream), "timing sync")) return GGML_STATUS_FAILED;
        std::lock_guard<std::mutex> lk(g_timing_mu);
        for (size_t k = 0; k < t_class.size(); ++k) {
            float ms = 0;
            cudaEventElapsedTime(&ms, ctx->events[2 * k], ctx->events[2 * k + 1]);
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

static void * b200_reg_get_proc_address(ggml_backend_reg_t, const char * name) {
    if (strcmp(name, "ggml_backend_get_features") == 0) return (void *) b200_get_features;
    if (strcmp(name, "b200_stat_nodes") == 0)  return (void *) b200_stat_nodes;
    if (strcmp(name, "b200_stat_graphs") == 0) return (void *) b200_stat_graphs;
    if (strcmp(name, "b200_stat_h2d") == 0)    return (void *) b200_stat_h2d;
    if (strcmp(name, "b200_stat_d2h") == 0)    return (void *) b200_stat_d2h;
    if (strcmp(name, "b200_stat_host_ns_compute") == 0) return (void *) b200_stat_host_ns_compute;
    if (strcmp(name, "b200_stat_host_ns_sync") == 0)    return (void *) b200_stat_host_ns_sync;
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
