/*
 * b200_whisper.h - C ABI of the sm_100a kernels behind the ggml backend plugin (libggml-b200.so).
 *
 * Two libraries:
 *   libb200_kernels.so  exports every b200_* function below (plain pointers and sizes, no ggml types).
 *   libggml-b200.so     exports ggml_backend_init / ggml_backend_score, the entry points that ggml's
 *                       dynamic loader binds (ggml/src/ggml-backend-impl.h:215-218, looked up by
 *                       ggml/src/ggml-backend-reg.cpp:236-253).  Its graph_compute maps every node of a
 *                       whisper graph onto the functions declared here.
 *
 * Every function returns 0 on success or a cudaError_t value (B200_ERR_* for argument errors).  Device
 * pointers are plain CUDA device pointers on the current device.  `stream` is a cudaStream_t passed
 * as void* (NULL = legacy default stream).  Nothing here synchronises the stream.
 *
 * Arithmetic contract: each kernel reproduces the operation order of the AVX2/FMA/F16C build of the
 * reference CPU backend (lane-wise partial sums, FMA placement, F16 round trips), so results are
 * expected to be bit-identical to it, not merely close.
 */
#ifndef B200_WHISPER_H
#define B200_WHISPER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ERR_ARG      10001   /* unsupported shape / type / alignment */
#define B200_ERR_NO_DEVICE 10002  /* no CUDA device: the library never falls back to the CPU */

/* ggml type ids used at this boundary (ggml/include/ggml.h:354-387) */
#define B200_TYPE_F32  0
#define B200_TYPE_F16  1
#define B200_TYPE_Q5_0 6
#define B200_TYPE_Q8_0 8
#define B200_TYPE_I32  26

/* ---- block formats ---------------------------------------------------------------------------
 * ggml stores 32 weights per block: block_q5_0 = {f16 d; u8 qh[4]; u8 qs[16]} (22 B),
 * block_q8_0 = {f16 d; i8 qs[32]} (34 B)  (ggml/src/ggml-common.h:187-214).  Neither size allows
 * aligned vector loads, so device memory holds the same bytes as three (two) planes of one tensor:
 *   Q5_0: qs[nb][16] | qh[nb] (u32) | d[nb] (f16)         Q8_0: qs[nb][32] | d[nb] (f16)
 * Total size is unchanged (22*nb / 34*nb bytes).  These run on the host and allocate nothing. */
int b200_blocks_to_planes(int type, const void * blocks, void * planes, int64_t nb_total,
                          int64_t nb_first, int64_t nb_count);   /* replaces nothing: layout helper */
int b200_planes_to_blocks(int type, const void * planes, void * blocks, int64_t nb_total,
                          int64_t nb_first, int64_t nb_count);
/* The same conversions on the device: `blocks_dev` holds nb_count raw ggml blocks (as read from a model file,
 * src/whisper.cpp:1874-1960, or produced by the quantize tool), `planes_dev` is the whole tensor's plane storage.
 * The plugin's set_tensor / get_tensor use them: one upload of the file's bytes plus one launch per weight tensor. */
int b200_blocks_to_planes_device(int type, const void * blocks_dev, void * planes_dev, int64_t nb_total, int64_t nb_first,
                                 int64_t nb_count, void * stream);
int b200_planes_to_blocks_device(int type, const void * planes_dev, void * blocks_dev, int64_t nb_total, int64_t nb_first,
                                 int64_t nb_count, void * stream);

/* dequantize_row_q5_0 / dequantize_row_q8_0 (ggml/src/ggml-quants.c:296-320, 349-362) on planes. */
int b200_dequantize(int type, const void * planes, int64_t nb_total, int64_t nb_first, int64_t nb_count,
                    float * out, void * stream);

/* quantize_row_q8_0, AVX2 variant (ggml/src/ggml-cpu/ggml-cpu-quants.c:808-866): rows of f32 ->
 * int8 qs[n_rows][k] and the f16-rounded scale widened to f32, d[n_rows][k/32]. */
int b200_quantize_q8_0(const float * x, int64_t n_rows, int64_t k, int64_t row_stride_bytes,
                       int8_t * qs, float * d, void * stream);

/* ggml_compute_forward_mul_mat for Q5_0 / Q8_0 weights (ggml/src/ggml-cpu/ggml-cpu.c:1266-1458 with
 * ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_q8_0_q8_0, ggml-cpu-quants.c:3076-3100, 3869-3886):
 * dst[n*dst_stride + m] = sum_k W[m][k] * X[n][k], activations already quantised by
 * b200_quantize_q8_0.  w_planes covers the WHOLE weight tensor (nb_total blocks). */
int b200_mul_mat_q(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                   const int8_t * xq, const float * xd, int64_t N,
                   float * dst, int64_t dst_stride, void * stream);

/* Same contract for 1..8 activation columns given as f32 (row stride in bytes): quantisation of the
 * activations is fused, no scratch is needed.  The batch-1 / beam decode path. */
int b200_mul_mat_vec_q(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                       const float * x, int64_t x_stride_bytes, int64_t N,
                       float * dst, int64_t dst_stride, void * stream);

/* Fused form of the above for the decode step: the product value passes through up to four steps, in the
 * order given, before it is stored - the ADD / SCALE / UNARY(GELU) / CPY nodes that follow a MUL_MAT node in
 * the whisper decoder graph (src/whisper.cpp:2533-2830), evaluated with the same single-precision
 * operations, so the stored bits equal those of the unfused node sequence.
 *   B200_EP_ADD   v = v + ptr[m + n*stride_n]   (stride_n = 0: bias broadcast over columns)
 *   B200_EP_SCALE v = v * scalar
 *   B200_EP_GELU  v = gelu_table(v)
 * store_f16 != 0 stores round-to-nearest-even f16 (the F32->F16 CPY into the KV cache) instead of f32. */
#define B200_EP_ADD   1
#define B200_EP_SCALE 2
#define B200_EP_GELU  3
typedef struct { int kind; const float * ptr; int64_t stride_n; float scalar; } b200_ep_step;
typedef struct { int n_steps; b200_ep_step step[4]; int store_f16; } b200_epilogue;
int b200_mul_mat_vec_q_ep(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                          const float * x, int64_t x_stride_bytes, int64_t N,
                          void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream);

/* b200_mul_mat_q with the same epilogue steps applied to every product value (encoder and prompt path). */
int b200_mul_mat_q_ep(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                      const int8_t * xq, const float * xd, int64_t N,
                      void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream);

/* The same kernel with every column described on its own: column n reads x (K floats, 16-byte aligned), writes
 * dst (M f32, or M f16 when store_f16) and adds add[s] (M floats) at epilogue step s when kind[s] == B200_EP_ADD.
 * This is how single-token decode steps of several whisper_states that run in lock-step share one pass over
 * the weights (up to 8 columns per launch).  No counterpart in the reference, which decodes state by state. */
typedef struct { const float * x; void * dst; const float * add[4]; } b200_gemv_col;
typedef struct { int n_steps; int kind[4]; float scalar[4]; int store_f16; } b200_gemv_ep;
int b200_mul_mat_vec_q_cols(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                            const b200_gemv_col * cols, int n_cols, const b200_gemv_ep * ep, void * stream);

/* Up to 32 columns per launch, quantised beforehand: b200_quantize_cols gathers columns that live at unrelated
 * addresses (K floats each) into xq[n_cols][K] / xd[n_cols][K/32]; b200_mul_mat_cols_q multiplies them with the
 * weights (cols[n].x is ignored, dst/add as above).  A CTA keeps a few weight rows in shared memory for all
 * columns, so the weights are read once for the whole group.  No counterpart in the reference. */
int b200_quantize_cols(const float * const * x_cols, int n_cols, int64_t K, int8_t * xq, float * xd, void * stream);
int b200_mul_mat_cols_q(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                        const int8_t * xq, const float * xd, const b200_gemv_col * cols, int n_cols,
                        const b200_gemv_ep * ep, void * stream);

/* Up to three b200_mul_mat_cols_q products on the SAME quantised columns in one launch (the Q, K and V projections of
 * a decoder layer): job i has its own weights (w_planes[i], nb_total[i], M[i] rows; all jobs share K and the type), its own
 * outputs cols[i][0..n_cols) and its own epilogue ep[i] (ep or ep[i] may be NULL).  No counterpart in the reference. */
int b200_mul_mat_cols_q_multi(int wtype, int n_jobs, const void * const * w_planes, const int64_t * nb_total, const int64_t * M,
                              int64_t K, const int8_t * xq, const float * xd, const b200_gemv_col * const * cols, int n_cols,
                              const b200_gemv_ep * const * ep, void * stream);

/* The same product (ggml_compute_forward_mul_mat with ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_q8_0_q8_0, same bits)
 * for many columns on the tensor pipe.  The integer lane sums of the AVX2 dot product are exact in an f16 MMA with
 * f32 accumulation, the per-block float chain is replayed as in b200_mul_mat_q.  Operands are repacked once:
 *   b200_mma_pack_weights: planes -> h[nb_total][16] u32 (the block's 32 integers as f16 pairs, pair 4r+t stored at
 *                          position 4t+r) and d[nb_total] f32; 68 bytes per block, both 16-byte aligned.  No
 *                          counterpart in the reference (layout helper, done once per weight tensor).
 *   b200_mma_quantize:     quantize_row_q8_0 (ggml-cpu-quants.c:808-866) writing the same integers in that format.
 *   b200_mul_mat_mma_ep:   dst[n*dst_stride + m] with the epilogue steps of b200_mul_mat_q_ep; K % 128 == 0. */
int b200_mma_pack_weights(int wtype, const void * w_planes, int64_t nb_total, void * h, float * d, void * stream);
int b200_mma_quantize(const float * x, int64_t n_rows, int64_t k, int64_t row_stride_bytes, void * h, float * d, void * stream);
int b200_mul_mat_mma_ep(const void * wh, const float * wd, int64_t M, int64_t K,
                        const void * xh, const float * xd, int64_t N,
                        void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream);

/* The same product once more (ggml_compute_forward_mul_mat, ggml/src/ggml-cpu/ggml-cpu.c:1266-1458, with
 * ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_q8_0_q8_0, ggml-cpu-quants.c:3076-3100, 3869-3886; same bits) on the
 * fifth-generation tensor cores: tcgen05.mma with a fresh tensor-memory accumulator per 32-block gives the eight
 * exact integer lane sums of every (row, column, block), epilogue warps drain tensor memory into the reference's
 * float chain.  Arguments as b200_mul_mat_q_ep: weights as planes (no repacked copy is needed, Q5_0 is unpacked in
 * the shared-memory stage), activations quantised by b200_quantize_q8_0.  Any M, N >= 1, K % 32 == 0.
 * b200_mul_mat_tc_status: 0, or the code of a device-side wait that ran out in an earlier launch (the launch then
 * returned without finishing its tiles); synchronises with the device. */
int b200_mul_mat_tc_ep(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                       const int8_t * xq, const float * xd, int64_t N,
                       void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream);
int b200_mul_mat_tc_status(void);
/* The same with every column described on its own (cols[n].dst / cols[n].add as in b200_mul_mat_cols_q, cols[n].x is
 * ignored; at most 64 columns): single-token decode steps of many whisper_states in one pass over the weights.  No
 * counterpart in the reference, which decodes state by state. */
int b200_mul_mat_tc_cols(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                         const int8_t * xq, const float * xd, const b200_gemv_col * cols, int n_cols,
                         const b200_gemv_ep * ep, void * stream);

/* NORM -> MUL(gamma) -> ADD(beta) in one pass (ops.cpp:3109-3158 followed by binary-ops.cpp:50-137), each of the
 * three roundings kept: y = ((x - mean) * rstd) * gamma + beta. */
int b200_layer_norm(const float * x, const float * gamma, const float * beta, float * y, int64_t ne00, int64_t nrows,
                    int64_t x_row_stride_bytes, int64_t y_row_stride_bytes, float eps, void * stream);

/* No counterpart in the reference.  b200_mul_mat_q needs the activations quantised into scratch memory that
 * the caller allocates.  Some callers cannot allocate device memory at the point where they need a product:
 * code that runs inside another framework's memory plan (all device memory handed out up front), hosts that
 * forbid the implicit device-wide synchronisation of cudaMalloc/cudaFree on a latency-critical path, or a
 * plugin callback that is only given input and output pointers.  For them this entry point does the same
 * work - quantise N rows of f32 activations (row stride in bytes), then the Q5_0/Q8_0 product - with the
 * scratch held in a fixed device array that is part of this library's image (b200_static_scratch_bytes()
 * bytes, resident on every GPU that loads the library until the process exits).  It calls no allocator.
 *  - N*K + 4*N*K/32 bytes (plus padding to 256) must fit; otherwise B200_ERR_TOO_LARGE is returned.  All
 *    arguments (NULL pointers, alignment, strides, weight extent) are checked first: an error return means nothing
 *    was launched.
 *  - The first call on each device looks up the array's device address (with that device current); make that
 *    first call outside any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents.  Every byte a call reads is
 *    written by that same call first, so nothing needs clearing, but two calls that may overlap on the GPU
 *    (different streams, no ordering between them) race on it. */
#define B200_ERR_TOO_LARGE 10003
int64_t b200_static_scratch_bytes(void);
int b200_mul_mat_q_static(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                          const float * x, int64_t x_stride_bytes, int64_t N,
                          float * dst, int64_t dst_stride, void * stream);

/* mul_mat with F16 src0 (ggml_vec_dot_f16, ggml/src/ggml-cpu/vec.cpp:128-167): src1 is f32 (rounded
 * to f16 first, ggml-cpu.c:1329-1362) or f16.  Strides in bytes; src0 [K, M, ne02, ne03],
 * src1 [K, N, ne12, ne13] with ne12 % ne02 == 0, dst f32 contiguous [M, N, ne12, ne13]. */
int b200_mul_mat_f16(const void * src0, const int64_t * ne0, const int64_t * nb0,
                     const void * src1, int src1_type, const int64_t * ne1, const int64_t * nb1,
                     float * dst, const int64_t * nbd, void * stream);

/* ggml_compute_forward_flash_attn_ext_f16 (ggml/src/ggml-cpu/ops.cpp:6638-6851) for head size 64,
 * F16 K/V, optional F16 mask; the running F16 accumulator and its rounding order are kept.
 * q f32 [64, n_q, n_head] (strides nbq1, nbq2 bytes), k/v f16 [64, n_kv, n_head], mask f16
 * [n_kv, >=n_q] or NULL, dst f32 [64, n_head, n_q] contiguous. */
int b200_flash_attn_ext(const float * q, int64_t nbq1, int64_t nbq2,
                        const void * k, int64_t nbk1, int64_t nbk2,
                        const void * v, int64_t nbv1, int64_t nbv2,
                        const void * mask, int64_t nbm1,
                        float * dst, int64_t n_q, int64_t n_kv, int64_t n_head, float scale, void * stream);

/* The decode-shaped form of the above, one entry per query row (at most 32): each row has its own query, K/V
 * views, mask row, output and key count, so rows of different whisper_states (different KV caches, different
 * lengths) go out in one launch.  dst receives [n_head][64] f32 per row.  No counterpart in the reference. */
typedef struct { const float * q; const void * k; const void * v; const void * mask; float * dst; int64_t n_kv; } b200_fa_row;
int b200_flash_attn_decode_rows(const b200_fa_row * rows, int n_rows, int64_t n_head, int64_t nbq2, int64_t nbk1, int64_t nbk2,
                                int64_t nbv1, int64_t nbv2, float scale, void * stream);
/* The same, and additionally every output row quantised as b200_quantize_cols would do it afterwards (row i ->
 * xq[i][n_head*64], xd[i][n_head*2]): saves the separate quantisation launch before the output projection. */
int b200_flash_attn_decode_rows_q(const b200_fa_row * rows, int n_rows, int64_t n_head, int64_t nbq2, int64_t nbk1, int64_t nbk2,
                                  int64_t nbv1, int64_t nbv2, float scale, int8_t * xq, float * xd, void * stream);

/* ggml_compute_forward_norm_f32 (ops.cpp:3109-3158): rows of ne00 f32, row strides in bytes. */
int b200_norm(const float * x, float * y, int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
              const int64_t * nbx, const int64_t * nby, float eps, void * stream);

/* b200_layer_norm for rows that live at unrelated addresses (at most 64; rows of several decoder states). */
typedef struct { const float * x; float * y; } b200_ln_row;
int b200_layer_norm_rows(const b200_ln_row * rows, int n_rows, const float * gamma, const float * beta, int64_t ne00, float eps, void * stream);
/* The same, and additionally every output row quantised as b200_quantize_cols would do it afterwards (row i ->
 * xq[i][ne00], xd[i][ne00/32]; ne00 a multiple of 32): saves the separate quantisation launch before the products that
 * consume the rows.  No counterpart in the reference beyond quantize_row_q8_0 itself. */
int b200_layer_norm_rows_q(const b200_ln_row * rows, int n_rows, const float * gamma, const float * beta, int64_t ne00, float eps,
                           int8_t * xq, float * xd, void * stream);

/* ADD (op 0) / MUL (op 1) with ggml broadcasting of src1 (ggml/src/ggml-cpu/binary-ops.cpp:50-137). */
int b200_binary(int op, const float * a, const int64_t * nea, const int64_t * nba,
                const float * b, const int64_t * neb, const int64_t * nbb,
                float * dst, const int64_t * nbd, void * stream);

/* SCALE (ops.cpp:3840) and GELU via the F16 lookup table (vec.h:443-457) on contiguous f32. */
int b200_scale(const float * x, float * y, int64_t n, float s, void * stream);
int b200_gelu(const float * x, float * y, int64_t n, void * stream);

/* CPY / DUP / CONT (ops.cpp:26-1183): f32->f32, f32->f16, f16->f16, f16->f32, any strides,
 * same element count, element order = row-major over ne. */
int b200_cpy(const void * src, int src_type, const int64_t * nes, const int64_t * nbs,
             void * dst, int dst_type, const int64_t * ned, const int64_t * nbd, void * stream);

/* GET_ROWS (ops.cpp:4146-4313): rows selected by i32 ids from a Q5_0/Q8_0 (planes), F16 or F32
 * table [ne00, n_table_rows] -> f32 [ne00, n_ids] contiguous. */
int b200_get_rows(int type, const void * table, int64_t nb_total_or_row_stride, int64_t ne00,
                  const int32_t * ids, int64_t n_ids, float * dst, void * stream);

/* Side output for the host sampler (whisper_process_logits / whisper_sample_token / whisper_sample_token_topk,
 * src/whisper.cpp:5015-5430, which scan a full row of n_vocab logits per decoder and step): per row of n values the k
 * largest with their indices (ties: lower index first, as the reference's forward scan with `>` resolves them), the
 * maximum and log(sum(exp(x - max))) + max.  rows[i] / out[i] are device pointers, at most 64 rows per call. */
#define B200_TOPK_MAX 8
typedef struct { int32_t n, k; float max, logsumexp; int32_t ids[B200_TOPK_MAX]; float vals[B200_TOPK_MAX]; } b200_topk_result;
int b200_topk_rows(const float * const * rows, b200_topk_result * const * out, int n_rows, int64_t n, int k, void * stream);

/* IM2COL 1-D, F16 output (ops.cpp:5784-5855): x f32 [IW, IC] (row stride bytes) ->
 * dst f16 [IC*KW, OW]. */
int b200_im2col_1d_f16(const float * x, int64_t x_stride_bytes, int64_t IW, int64_t IC, int64_t KW,
                       int64_t OW, int s0, int p0, int d0, void * dst, void * stream);

/* SOFT_MAX with optional mask and scale (ops.cpp:4641-4737, max_bias = 0): rows of ne00 f32. */
int b200_soft_max(const float * x, const void * mask, int mask_type, int64_t mask_nb1, int64_t mask_ne1,
                  float * y, int64_t ne00, int64_t nrows, int64_t ne01, float scale, void * stream);

/* CONCAT along dim (ops.cpp:2403-2604), f32, contiguous dst. */
int b200_concat(const float * a, const int64_t * nea, const int64_t * nba,
                const float * b, const int64_t * neb, const int64_t * nbb,
                float * dst, const int64_t * ned, const int64_t * nbd, int dim, void * stream);

/* log_mel_spectrogram (src/whisper.cpp:3008-3271): 16 kHz mono f32 PCM -> log-mel [n_mel][n_len]
 * on the device; out_host receives n_mel*n_len floats (n_len = (n_samples + 480000 padding)/160).
 * The result feeds whisper_set_mel_with_state (include/whisper.h:278-293). */
int b200_log_mel(int device, const float * pcm_host, int64_t n_samples, const float * filters_host,
                 int n_mel, float * out_host, int64_t out_capacity, int * n_len, int * n_len_org);

/* Same front-end with persistent device buffers, tables and a private stream, for repeated use
 * (one plan per host thread).  b200_mel_compute is synchronous: on return out_host holds
 * [n_mel][n_len] floats.  No counterpart in the reference (its mel runs on host threads). */
void * b200_mel_create(int device, const float * filters_host, int n_mel);
int    b200_mel_compute(void * plan, const float * pcm_host, int64_t n_samples, float * out_host, int64_t out_capacity,
                        int * n_len, int * n_len_org);
void   b200_mel_destroy(void * plan);

/* ---- optional entry points of the plugin (libggml-b200.so), obtained with
 * ggml_backend_reg_get_proc_address(ggml_backend_reg_by_name("B200"), name)  (ggml/include/ggml-backend.h:190):
 *
 *   void b200_logits_side_output(int top_k, int skip_readback)
 *       top_k > 0: after every decoder graph (its last node is the logits product, src/whisper.cpp:2830) the plugin also
 *       leaves b200_topk_rows of every logits row in a small device buffer of the backend instance that ran the graph.
 *       skip_readback != 0: ggml_backend_tensor_get on a logits tensor returns at once without copying - for callers
 *       that sample from the side output only; whisper_get_logits() then holds stale data.  Default: off, off.
 *   int b200_last_topk(int row, b200_topk_result * out)
 *       side output of logits row `row` of the last decoder graph computed on the CALLING thread (whisper_decode is
 *       synchronous, so that is the state the thread just stepped); waits for that graph, copies one result to the host.
 *       Returns 0, or B200_ERR_ARG when there is no such row.
 * No counterpart in the reference, which samples from the full row on the host.
 *
 * A plain exported symbol of the plugin for tests (no device work, needs no GPU):
 *   int b200_plan_probe(struct ggml_cgraph * plan_graph, struct ggml_cgraph * candidate)
 *       builds the fused execution plan of plan_graph and checks candidate against it the way a cached plan is checked
 *       before reuse: -1 when the two graphs' signatures differ, else bit 0 = candidate may run on the plan, bit 1 = the
 *       plan fuses at least one pair of nodes. */

/* Library info: number of kernel launches issued so far by this process (all entry points). */
int64_t b200_launch_count(void);
const char * b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_WHISPER_H */
