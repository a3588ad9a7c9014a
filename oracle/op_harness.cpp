// Test infrastructure, not product code.
// Runs ONE ggml operator, built exactly as src/whisper.cpp builds it, on a named ggml backend device
// ("CPU" = the reference's own CPU backend, "B200_0" = the plugin under test) and returns the result.
// Compiled against the reference's ggml headers and linked to its unmodified libggml*.so
// (oracle/Makefile), so the CPU side IS the reference implementation of each operator.
#include <dlfcn.h>
#include "ggml.h"
#include "ggml-alloc.h"
#include "ggml-backend.h"
#include "ggml-cpu.h"

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

extern "C" {

int oph_load_backend(const char * path) {
    ggml_backend_reg_t reg = ggml_backend_load(path);
    return reg ? (int) ggml_backend_reg_dev_count(reg) : 0;
}

// ggml_quantize_chunk of the reference (ggml/src/ggml.c:6498): f32 rows -> block bytes
int64_t oph_quantize(int type, const float * src, void * dst, int64_t nrows, int64_t n_per_row) {
    return (int64_t) ggml_quantize_chunk((enum ggml_type) type, src, dst, 0, nrows, n_per_row, nullptr);
}

// to_float of the reference type traits (dequantize_row_*): block bytes -> f32
int oph_dequantize(int type, const void * src, float * dst, int64_t n) {
    static bool tables_ready = false;      // ggml_init fills the f16 -> f32 table that ggml-base's to_float uses
    if (!tables_ready) { struct ggml_init_params ip = { 0, nullptr, false }; ggml_free(ggml_init(ip)); tables_ready = true; }
    const struct ggml_type_traits * tr = ggml_get_type_traits((enum ggml_type) type);
    if (!tr || !tr->to_float) return -1;
    tr->to_float(src, dst, n);
    return 0;
}

// from_float of the CPU type traits (quantize_row_q8_0 SIMD variant for type 8)
int oph_cpu_from_float(int type, const float * src, void * dst, int64_t n) {
    const struct ggml_type_traits_cpu * tr = ggml_get_type_traits_cpu((enum ggml_type) type);
    if (!tr || !tr->from_float) return -1;
    tr->from_float(src, dst, n);
    return 0;
}

struct run_ctx {
    ggml_backend_t        backend = nullptr;
    ggml_context *        ctx     = nullptr;
    ggml_backend_buffer_t buf     = nullptr;
};

static ggml_backend_t init_backend(const char * dev_name, int threads) {
    ggml_backend_dev_t dev = ggml_backend_dev_by_name(dev_name);
    if (!dev) return nullptr;
    ggml_backend_t b = ggml_backend_dev_init(dev, nullptr);
    if (b && ggml_backend_is_cpu(b)) ggml_backend_cpu_set_n_threads(b, threads);
    return b;
}

// op ids
enum { OP_MUL_MAT = 1, OP_MUL_MAT_CONV, OP_FLASH_ATTN, OP_NORM, OP_ADD, OP_MUL, OP_SCALE, OP_GELU, OP_CPY_F16, OP_CONT_T,
       OP_GET_ROWS, OP_IM2COL, OP_SOFT_MAX, OP_CONCAT, OP_KQ_NOFA, OP_KQV_NOFA, OP_CPY_F16_T, OP_ROUNDTRIP, OP_MM_TWICE };

// p: integer parameters, f: float parameters, in: input buffers (host), out: result buffer (host).
// Returns number of bytes written to out, or a negative error.
int64_t oph_run(const char * dev_name, int op, const int64_t * p, const float * f, const void ** in, void * out, int64_t out_cap, int threads) {
    ggml_backend_t backend = init_backend(dev_name, threads);
    if (!backend) return -1;
    struct ggml_init_params ip = { ggml_tensor_overhead() * 64 + ggml_graph_overhead(), nullptr, true };
    ggml_context * ctx = ggml_init(ip);
    ggml_tensor * src[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t src_bytes[4] = {0, 0, 0, 0};
    ggml_tensor * res = nullptr;

    switch (op) {
        case OP_MUL_MAT: {          // p: wtype, K, M, N
            src[0] = ggml_new_tensor_2d(ctx, (enum ggml_type) p[0], p[1], p[2]);
            src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[1], p[3]);
            res = ggml_mul_mat(ctx, src[0], src[1]);
        } break;
        case OP_MUL_MAT_CONV: {     // conv stem product: both f16 (whisper.cpp:2019-2027 via ggml_conv_1d); p: K, M(=OW), N(=OC)
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F16, p[0], p[1]);
            src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F16, p[0], p[2]);
            res = ggml_mul_mat(ctx, src[0], src[1]);
        } break;
        case OP_FLASH_ATTN: {       // p: n_q, n_kv, H, has_mask, kv_rows(>=n_kv) ; f: scale
            const int64_t n_q = p[0], n_kv = p[1], H = p[2], d = 64 * H, kv_rows = p[4];
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, d, n_q);                  // Qcur [d, n_q]
            src[1] = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, d * kv_rows);             // K cache
            src[2] = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, d * kv_rows);             // V cache
            ggml_tensor * Q = ggml_permute(ctx, ggml_reshape_3d(ctx, src[0], 64, H, n_q), 0, 2, 1, 3);
            ggml_tensor * K = ggml_view_3d(ctx, src[1], 64, n_kv, H, ggml_element_size(src[1]) * d, ggml_element_size(src[1]) * 64, 0);
            ggml_tensor * V = ggml_view_3d(ctx, src[2], 64, n_kv, H, ggml_element_size(src[2]) * d, ggml_element_size(src[2]) * 64, 0);
            ggml_tensor * M = nullptr;
            if (p[3]) {
                src[3] = ggml_new_tensor_2d(ctx, GGML_TYPE_F16, n_kv, GGML_PAD(n_q, GGML_KQ_MASK_PAD));
                M = src[3];
            }
            res = ggml_flash_attn_ext(ctx, Q, K, V, M, f[0], 0.0f, 0.0f);
        } break;
        case OP_NORM: {             // p: ne0, ne1 ; f: eps
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            res = ggml_norm(ctx, src[0], f[0]);
        } break;
        case OP_ADD: case OP_MUL: { // p: a ne0, ne1, b ne0, ne1
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[2], p[3]);
            res = op == OP_ADD ? ggml_add(ctx, src[0], src[1]) : ggml_mul(ctx, src[0], src[1]);
        } break;
        case OP_SCALE: {
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            res = ggml_scale(ctx, src[0], f[0]);
        } break;
        case OP_GELU: {
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            res = ggml_gelu(ctx, src[0]);
        } break;
        case OP_CPY_F16: {          // f32 [ne0, ne1] -> f16 1-D view at element offset p[2] of a buffer of p[3] elements
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            src[1] = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, p[3]);
            ggml_tensor * v = ggml_view_1d(ctx, src[1], p[0] * p[1], p[2] * ggml_element_size(src[1]));
            res = ggml_cpy(ctx, src[0], v);
        } break;
        case OP_CPY_F16_T: {        // transposed V store of the non-flash path (whisper.cpp:2337-2347): f32 [d, n] -> f16 [n_ctx, d] strided
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            src[1] = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, p[0] * p[2]);
            ggml_tensor * v = ggml_view_2d(ctx, src[1], p[1], p[0], p[2] * ggml_element_size(src[1]), 0);
            res = ggml_cpy(ctx, ggml_transpose(ctx, src[0]), v);
        } break;
        case OP_CONT_T: {           // cont(transpose(x)) as in whisper.cpp:2080-2084
            src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]);
            res = ggml_cont(ctx, ggml_transpose(ctx, src[0]));
        } break;
        case OP_GET_ROWS: {         // p: type, ne0, n_rows_table, n_ids
            src[0] = ggml_new_tensor_2d(ctx, (enum ggml_type) p[0], p[1], p[2]);
            src[1] = ggml_new_tensor_1d(ctx, GGML_TYPE_I32, p[3]);
            res = ggml_get_rows(ctx, src[0], src[1]);
        } break;
        case OP_IM2COL: {           // conv_1d_ph front half: kernel f16 [3, IC, OC], x f32 [IW, IC]; p: IC, OC, IW, stride
            src[0] = ggml_new_tensor_3d(ctx, GGML_TYPE_F16, 3, p[0], p[1]);
            src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[2], p[0]);
            res = ggml_im2col(ctx, src[0], src[1], (int) p[3], 0, 1, 0, 1, 0, false, GGML_TYPE_F16);
        } break;
        case OP_SOFT_MAX: {         // p: ne0, ne1, ne2, mask(0 none, 1 f32, 2 f16) ; f: scale
            src[0] = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, p[0], p[1], p[2]);
            ggml_tensor * M = nullptr;
            if (p[3]) { src[1] = ggml_new_tensor_2d(ctx, p[3] == 2 ? GGML_TYPE_F16 : GGML_TYPE_F32, p[0], GGML_PAD(p[1], GGML_KQ_MASK_PAD)); M = src[1]; }
            res = ggml_soft_max_ext(ctx, src[0], M, f[0], 0.0f);
        } break;
        case OP_CONCAT: {           // p: ne0, ne1a, ne1b, dim(=1) or along 0
            if (p[3] == 1) { src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[1]); src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[0], p[2]); }
            else           { src[0] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[1], p[0]); src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[2], p[0]); }
            res = ggml_concat(ctx, src[0], src[1], (int) p[3]);
        } break;
        case OP_KQ_NOFA: {          // non-flash scores (whisper.cpp:2175-2186): K f16 [64, n_kv, H] view, Q f32 [64, n_q, H] permuted
            const int64_t n_q = p[0], n_kv = p[1], H = p[2], d = 64 * H;
            src[0] = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, d * n_kv);
            src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, d, n_q);
            ggml_tensor * K = ggml_view_3d(ctx, src[0], 64, n_kv, H, ggml_element_size(src[0]) * d, ggml_element_size(src[0]) * 64, 0);
            ggml_tensor * Q = ggml_permute(ctx, ggml_reshape_3d(ctx, src[1], 64, H, n_q), 0, 2, 1, 3);
            res = ggml_mul_mat(ctx, K, Q);
        } break;
        case OP_KQV_NOFA: {         // non-flash P*V (whisper.cpp:2190-2200): V f16 [n_kv, 64, H] view of a transposed store, P f32 [n_kv, n_q, H]
            const int64_t n_q = p[0], n_kv = p[1], H = p[2], n_ctx = p[3];
            src[0] = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, 64 * H * n_ctx);
            src[1] = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, n_kv, n_q, H);
            ggml_tensor * V = ggml_view_3d(ctx, src[0], n_kv, 64, H, n_ctx * ggml_element_size(src[0]), n_ctx * ggml_element_size(src[0]) * 64, 0);
            res = ggml_mul_mat(ctx, V, src[1]);
        } break;
        case OP_MM_TWICE: {         // two products on the same activations, p: wtype, K, M, N, overwrite.  With overwrite the
                                    // activations are scaled IN PLACE between the products (the second product must see the new values:
                                    // a backend that keeps a converted copy of the activations has to notice the write)
            src[0] = ggml_new_tensor_2d(ctx, (enum ggml_type) p[0], p[1], p[2]);
            src[1] = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, p[1], p[3]);
            ggml_tensor * y1 = ggml_mul_mat(ctx, src[0], src[1]);
            ggml_tensor * x2 = p[4] ? ggml_scale_inplace(ctx, src[1], 0.5f) : src[1];
            ggml_tensor * y2 = ggml_mul_mat(ctx, src[0], x2);
            res = ggml_add(ctx, y1, ggml_scale(ctx, y2, 3.0f));
        } break;
        case OP_ROUNDTRIP: {        // set_tensor then get_tensor of a weight tensor; p: type, ne0, ne1
            src[0] = ggml_new_tensor_2d(ctx, (enum ggml_type) p[0], p[1], p[2]);
            res = nullptr;
        } break;
        default:
            ggml_free(ctx); ggml_backend_free(backend);
            return -2;
    }

    ggml_cgraph * gf = nullptr;
    if (res) {
        gf = ggml_new_graph(ctx);
        ggml_build_forward_expand(gf, res);
    }
    ggml_backend_buffer_t buf = ggml_backend_alloc_ctx_tensors(ctx, backend);
    if (!buf) { ggml_free(ctx); ggml_backend_free(backend); return -3; }
    for (int i = 0; i < 4; ++i) {
        if (src[i] && in[i]) ggml_backend_tensor_set(src[i], in[i], 0, ggml_nbytes(src[i]));
        else if (src[i]) ggml_backend_tensor_memset(src[i], 0, 0, ggml_nbytes(src[i]));
    }
    (void) src_bytes;
    int64_t written = -4;
    if (res) {
        if (!ggml_backend_supports_op(backend, res)) { written = -5; }
        else if (ggml_backend_graph_compute(backend, gf) == GGML_STATUS_SUCCESS) {
            // for CPY nodes the interesting bytes are the destination buffer
            ggml_tensor * o = res;
            if (op == OP_CPY_F16 || op == OP_CPY_F16_T) o = src[1];
            const int64_t n = (int64_t) ggml_nbytes(o);
            if (n <= out_cap) { ggml_backend_tensor_get(o, out, 0, n); written = n; } else written = -6;
        }
    } else {
        const int64_t n = (int64_t) ggml_nbytes(src[0]);
        if (n <= out_cap) { ggml_backend_tensor_get(src[0], out, 0, n); written = n; } else written = -6;
    }
    ggml_backend_buffer_free(buf);
    ggml_free(ctx);
    ggml_backend_free(backend);
    return written;
}


// Plan reuse of the plugin: two graphs with the same operators, types and shapes in the same order.  In the first the
// product feeds only the addition (a fusion candidate); in the second (variant 1) the last node reads the PRODUCT instead of
// the sum, so the product has two consumers and must be written to memory.  Calls the plugin's test hook
// b200_plan_probe(plan_graph, candidate) from the already loaded plugin library; no device work.
// Returns the hook's value, or -10 (hook not found), -11 (set-up failed).
int oph_plan_probe(const char * plugin_path, int variant) {
    void * h = dlopen(plugin_path, RTLD_NOW | RTLD_LOCAL);
    if (!h) return -10;
    typedef int (*probe_fn)(ggml_cgraph *, ggml_cgraph *);
    probe_fn probe = (probe_fn) dlsym(h, "b200_plan_probe");
    if (!probe) return -10;
    ggml_backend_t cpu = init_backend("CPU", 1);
    if (!cpu) return -11;
    struct ggml_init_params ip = { ggml_tensor_overhead() * 64 + 2 * ggml_graph_overhead(), nullptr, true };
    ggml_context * ctx = ggml_init(ip);
    ggml_cgraph * g[2];
    for (int v = 0; v < 2; ++v) {
        ggml_tensor * w = ggml_new_tensor_2d(ctx, GGML_TYPE_Q5_0, 256, 64);
        ggml_tensor * x = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, 256, 1);
        ggml_tensor * b = ggml_new_tensor_1d(ctx, GGML_TYPE_F32, 64);
        ggml_tensor * y = ggml_mul_mat(ctx, w, x);
        ggml_tensor * z = ggml_add(ctx, y, b);
        ggml_tensor * r = ggml_scale(ctx, (v == 1 && variant == 1) ? y : z, 2.0f);
        g[v] = ggml_new_graph(ctx);
        if (v == 1 && variant == 1) ggml_build_forward_expand(g[v], z);      // keep the node order: product, sum, scale
        ggml_build_forward_expand(g[v], r);
    }
    ggml_backend_buffer_t buf = ggml_backend_alloc_ctx_tensors(ctx, cpu);
    int rc = buf ? probe(g[0], g[1]) : -11;
    if (buf) ggml_backend_buffer_free(buf);
    ggml_free(ctx);
    ggml_backend_free(cpu);
    return rc;
}

// Error paths of a backend device (no abort, an error value instead):
//  oph_try_alloc: 1 if the device's buffer type hands out a buffer of `size` bytes (freed again), 0 if it returns NULL.
int oph_try_alloc(const char * dev_name, int64_t size) {
    ggml_backend_dev_t dev = ggml_backend_dev_by_name(dev_name);
    if (!dev) return -1;
    ggml_backend_buffer_t buf = ggml_backend_buft_alloc_buffer(ggml_backend_dev_buffer_type(dev), (size_t) size);
    if (!buf) return 0;
    ggml_backend_buffer_free(buf);
    return 1;
}

//  oph_unsupported_status: ggml_status of graph_compute for a graph that holds an operator the device does not support
//  (ggml_sqr), handed to the backend directly, past the scheduler that would never send it there (GGML_STATUS_FAILED is -1,
//  GGML_STATUS_ALLOC_FAILED -2, GGML_STATUS_SUCCESS 0).  -11/-12: set-up failed, -13: the device claims to support the operator.
int oph_unsupported_status(const char * dev_name) {
    ggml_backend_t backend = init_backend(dev_name, 1);
    if (!backend) return -11;
    struct ggml_init_params ip = { ggml_tensor_overhead() * 8 + ggml_graph_overhead(), nullptr, true };
    ggml_context * ctx = ggml_init(ip);
    ggml_tensor * a = ggml_new_tensor_1d(ctx, GGML_TYPE_F32, 64);
    ggml_tensor * r = ggml_sqr(ctx, a);
    int rc;
    if (ggml_backend_dev_supports_op(ggml_backend_get_device(backend), r)) {
        rc = -13;
    } else {
        ggml_backend_buffer_t buf = ggml_backend_alloc_ctx_tensors(ctx, backend);
        if (!buf) {
            rc = -12;
        } else {
            ggml_cgraph * g = ggml_new_graph(ctx);
            ggml_build_forward_expand(g, r);
            rc = (int) ggml_backend_graph_compute(backend, g);
            ggml_backend_buffer_free(buf);
        }
    }
    ggml_free(ctx);
    ggml_backend_free(backend);
    return rc;
}

}
