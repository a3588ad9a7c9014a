/*
 * TEST INFRASTRUCTURE - CPU restatement of the whisper.cpp hot-path arithmetic.
 *
 * Plain scalar C that restates, operation by operation, what the reference's CPU backend computes in
 * its AVX2/FMA/F16C build (the build pinned by oracle/Makefile).  It exists so that parity tests have a
 * checker that needs neither the reference tree nor a GPU.  It is pinned against the real reference:
 * tests/test_oracle_cpu.py compares every function here with outputs of the unmodified reference
 * libraries (live when oracle/_ref exists, and always against the committed vectors in tests/golden/
 * that tests/golden/make_golden.py produced from those libraries).
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may load this library.
 * Compile with -ffp-contract=off: every fused multiply-add below is written out as fmaf().
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

static inline float h2f(uint16_t h) { f16 v; memcpy(&v, &h, 2); return (float) v; }
static inline uint16_t f2h(float f) { f16 v = (f16) f; uint16_t h; memcpy(&h, &v, 2); return h; }   /* round to nearest even */
static inline float rf16(float f) { return (float) (f16) f; }

/* ---- block formats (ggml/src/ggml-common.h:187-214) -------------------------------------------- */
/* dequantize_row_q5_0, ggml/src/ggml-quants.c:296-320 */
void orc_dequantize_q5_0(const uint8_t * blocks, float * y, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i) {
        const uint8_t * b = blocks + 22 * i;
        uint16_t dh; uint32_t qh;
        memcpy(&dh, b, 2); memcpy(&qh, b + 2, 4);
        const float d = h2f(dh);
        for (int j = 0; j < 16; ++j) {
            const uint8_t xh_0 = ((qh >> (j + 0)) << 4) & 0x10;
            const uint8_t xh_1 = ((qh >> (j + 12))) & 0x10;
            const int32_t x0 = ((b[6 + j] & 0x0F) | xh_0) - 16;
            const int32_t x1 = ((b[6 + j] >> 4) | xh_1) - 16;
            y[i * 32 + j] = x0 * d;
            y[i * 32 + j + 16] = x1 * d;
        }
    }
}

/* dequantize_row_q8_0, ggml/src/ggml-quants.c:349-362 */
void orc_dequantize_q8_0(const uint8_t * blocks, float * y, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i) {
        const uint8_t * b = blocks + 34 * i;
        uint16_t dh; memcpy(&dh, b, 2);
        const float d = h2f(dh);
        for (int j = 0; j < 32; ++j) y[i * 32 + j] = ((const int8_t *) b)[2 + j] * d;
    }
}

/* quantize_row_q8_0, AVX2 branch, ggml/src/ggml-cpu/ggml-cpu-quants.c:808-866:
 * d = amax/127 (stored f16), q = round-to-nearest-even(x * (127/amax)). */
void orc_quantize_row_q8_0(const float * x, int8_t * qs, float * d_out, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) { const float a = fabsf(x[i * 32 + j]); if (a > amax) amax = a; }
        const float d = amax / 127.f;
        const float id = (amax != 0.0f) ? 127.f / amax : 0.0f;
        d_out[i] = h2f(f2h(d));
        for (int j = 0; j < 32; ++j) qs[i * 32 + j] = (int8_t) lrintf(x[i * 32 + j] * id);   /* default rounding mode = nearest even */
    }
}

/* signed weights of one Q5_0 block, as bytes_from_nibbles_32 | ~bits<<4 builds them (ggml-cpu-quants.c:3086-3089) */
static void q5_block_to_i8(const uint8_t * b, int8_t * w) {
    uint32_t qh; memcpy(&qh, b + 2, 4);
    for (int j = 0; j < 16; ++j) {
        w[j]      = (int8_t) (((b[6 + j] & 0x0F) | (((qh >> j) & 1u) << 4)) - 16);
        w[j + 16] = (int8_t) (((b[6 + j] >> 4)   | (((qh >> (j + 16)) & 1u) << 4)) - 16);
    }
}

/* ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_q8_0_q8_0, AVX2 branches (ggml-cpu-quants.c:3076-3100, 3869-3886):
 * eight float lanes; lane j of a block = sum of products of elements 4j..4j+3 (maddubs + madd), converted to
 * float; acc[j] = fma(d_w*d_x, lane, acc[j]); final hsum_float_8 (:49-55). */
static float vec_dot_q_q8(int wtype, const uint8_t * wblocks, const int8_t * xq, const float * xd, int64_t nb) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t ib = 0; ib < nb; ++ib) {
        int8_t wbuf[32];
        const int8_t * w;
        uint16_t dh;
        if (wtype == 6) { const uint8_t * b = wblocks + 22 * ib; memcpy(&dh, b, 2); q5_block_to_i8(b, wbuf); w = wbuf; }
        else            { const uint8_t * b = wblocks + 34 * ib; memcpy(&dh, b, 2); w = (const int8_t *) (b + 2); }
        const float d = h2f(dh) * xd[ib];
        for (int j = 0; j < 8; ++j) {
            int32_t s = 0;
            for (int t = 0; t < 4; ++t) s += (int32_t) w[4 * j + t] * (int32_t) xq[ib * 32 + 4 * j + t];
            acc[j] = fmaf(d, (float) s, acc[j]);
        }
    }
    float r0 = acc[4] + acc[0], r1 = acc[5] + acc[1], r2 = acc[6] + acc[2], r3 = acc[7] + acc[3];
    r0 = r0 + r2; r1 = r1 + r3;
    return r0 + r1;
}

/* ggml_compute_forward_mul_mat for quantised src0 (ggml-cpu.c:1266-1458): src1 rows are quantised to Q8_0
 * first, then dst[n][m] = vec_dot(W row m, X row n).  W = ggml block bytes [M][K/32]. */
void orc_mul_mat_q(int wtype, const uint8_t * w, int64_t M, int64_t K, const float * x, int64_t N, float * dst) {
    const int64_t nb = K / 32, bs = wtype == 6 ? 22 : 34;
    int8_t * xq = (int8_t *) malloc((size_t) K);
    float *  xd = (float *) malloc((size_t) nb * sizeof(float));
    for (int64_t n = 0; n < N; ++n) {
        orc_quantize_row_q8_0(x + n * K, xq, xd, K);
        for (int64_t m = 0; m < M; ++m) dst[n * M + m] = vec_dot_q_q8(wtype, w + m * nb * bs, xq, xd, nb);
    }
    free(xq); free(xd);
}

/* ggml_vec_dot_f16, AVX2/F16C (ggml/src/ggml-cpu/vec.cpp:128-167, simd-mappings.h:236-332): 32 running sums,
 * element k joins sum k%32 by fma; reduce: s0+=s2, s1+=s3, s0+=s1, halves folded, two hadds; tail in double. */
static float vec_dot_f16(const uint16_t * x, const uint16_t * y, int64_t n) {
    float sum[32];
    for (int i = 0; i < 32; ++i) sum[i] = 0.0f;
    const int64_t np = n & ~(int64_t) 31;
    for (int64_t i = 0; i < np; i += 32)
        for (int l = 0; l < 32; ++l) sum[l] = fmaf(h2f(x[i + l]), h2f(y[i + l]), sum[l]);
    float v[8];
    for (int p = 0; p < 8; ++p) { const float a = sum[p] + sum[16 + p], b = sum[8 + p] + sum[24 + p]; v[p] = a + b; }
    const float t0 = v[0] + v[4], t1 = v[1] + v[5], t2 = v[2] + v[6], t3 = v[3] + v[7];
    double sumf = (double) ((t0 + t1) + (t2 + t3));
    for (int64_t i = np; i < n; ++i) sumf += (double) (h2f(x[i]) * h2f(y[i]));
    return (float) sumf;
}

/* mul_mat with F16 src0: src1 (f32) is converted to f16 row by row (ggml-cpu.c:1329-1362), then vec_dot_f16. */
void orc_mul_mat_f16(const uint16_t * w, int64_t M, int64_t K, const float * x, int64_t N, float * dst) {
    uint16_t * xr = (uint16_t *) malloc((size_t) K * 2);
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) xr[k] = f2h(x[n * K + k]);
        for (int64_t m = 0; m < M; ++m) dst[n * M + m] = vec_dot_f16(w + m * K, xr, K);
    }
    free(xr);
}

/* ggml_compute_forward_norm_f32, ggml/src/ggml-cpu/ops.cpp:3109-3158 */
void orc_norm(const float * x, float * y, int64_t ne0, int64_t nrows, float eps) {
    for (int64_t r = 0; r < nrows; ++r) {
        const float * xp = x + r * ne0; float * yp = y + r * ne0;
        double sum = 0.0;
        for (int64_t i = 0; i < ne0; ++i) sum += (double) xp[i];
        const float mean = (float) (sum / ne0);
        double sum2 = 0.0;
        for (int64_t i = 0; i < ne0; ++i) { const float v = xp[i] - mean; yp[i] = v; sum2 += (double) (v * v); }
        const float variance = (float) (sum2 / ne0);
        const float scale = 1.0f / sqrtf(variance + eps);
        for (int64_t i = 0; i < ne0; ++i) yp[i] = yp[i] * scale;
    }
}

/* ggml_vec_gelu_f32 through the f16 table (ggml/src/ggml-cpu/vec.h:428-457, table ggml-cpu.c:3398-3421).
 * The table entry is evaluated with the same expression; the reference's compiler contracts a*b+c forms, which
 * -ffp-contract=off forbids here, so the contracted form is spelled out: inner = fma(c*x, x, 1) and
 * outer = 0.5*x*(1+tanh(.)) (verified against the reference for all 65536 inputs by the oracle tests). */
static float gelu_entry(float x, int variant) {
    const float A = 0.044715f, S = 0.79788456080286535587989211986876f;
    float inner;
    if (variant == 0) inner = 1.0f + A * x * x;
    else              inner = fmaf(A * x, x, 1.0f);
    const float t = tanhf(S * x * inner);
    return 0.5f * x * (1.0f + t);
}
static int g_gelu_variant = 1;
void orc_set_gelu_variant(int v) { g_gelu_variant = v; }
void orc_gelu(const float * x, float * y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        if (x[i] <= -10.0f) y[i] = 0.0f;
        else if (x[i] >= 10.0f) y[i] = x[i];
        else y[i] = h2f(f2h(gelu_entry(h2f(f2h(x[i])), g_gelu_variant)));
    }
}

/* ggml_compute_forward_flash_attn_ext_f16, F16 K/V (ggml/src/ggml-cpu/ops.cpp:6638-6851); q [n_q][H][64] f32 (already the
 * permuted view's rows), k/v [n_kv][H][64] f16, mask [>=n_q][n_kv] f16 or NULL, dst [n_q][H][64]. */
void orc_flash_attn(const float * q, const uint16_t * k, const uint16_t * v, const uint16_t * mask, float * dst,
                    int64_t n_q, int64_t n_kv, int64_t H, float scale) {
    for (int64_t iq = 0; iq < n_q; ++iq) for (int64_t h = 0; h < H; ++h) {
        uint16_t Q16[64], VKQ16[64];
        for (int d = 0; d < 64; ++d) { Q16[d] = f2h(q[(iq * H + h) * 64 + d]); VKQ16[d] = 0; }
        float S = 0.0f, M = -INFINITY;
        for (int64_t ic = 0; ic < n_kv; ++ic) {
            const float mv = mask ? h2f(mask[iq * n_kv + ic]) : 0.0f;
            if (mv == -INFINITY) continue;
            float s = vec_dot_f16(k + (ic * H + h) * 64, Q16, 64);
            s = s * scale;
            s += mv;
            const float Mold = M;
            float ms = 1.0f, vs = 1.0f;
            const uint16_t * vr = v + (ic * H + h) * 64;
            if (s > M) {
                M = s;
                ms = expf(Mold - M);
                for (int d = 0; d < 64; ++d) VKQ16[d] = f2h(h2f(VKQ16[d]) * ms);         /* ggml_vec_scale_f16 */
            } else {
                vs = expf(s - M);
            }
            for (int d = 0; d < 64; ++d) VKQ16[d] = f2h(fmaf(h2f(vr[d]), vs, h2f(VKQ16[d])));   /* ggml_vec_mad_f16 */
            S = fmaf(S, ms, vs);       /* "S*ms + vs", contracted by the reference's compiler */
        }
        const float S_inv = 1.0f / S;
        for (int d = 0; d < 64; ++d) dst[(iq * H + h) * 64 + d] = h2f(VKQ16[d]) * S_inv;
    }
}

/* ggml_v_expf, AVX2 (ggml/src/ggml-cpu/vec.h:603-640), one element */
static float v_expf(float x) {
    const float r = 0x1.8p23f;
    const float z = fmaf(x, 0x1.715476p+0f, r);
    const float n = z - r;
    const float b = fmaf(-n, 0x1.7f7d1cp-20f, fmaf(-n, 0x1.62e4p-1f, x));
    uint32_t zb; memcpy(&zb, &z, 4);
    const uint32_t e = zb << 23;
    uint32_t kb = e + 0x3f800000u; float k; memcpy(&k, &kb, 4);
    const int c = fabsf(n) > 126.0f;
    const float u = b * b;
    const float j = fmaf(fmaf(fmaf(0x1.0e4020p-7f, b, 0x1.573e2ep-5f), u, fmaf(0x1.555e66p-3f, b, 0x1.fffdb6p-2f)), u, 0x1.ffffecp-1f * b);
    if (!c) return fmaf(j, k, k);
    const uint32_t g = (n <= 0.0f) ? 0x82000000u : 0u;
    uint32_t s1b = g + 0x7f000000u, s2b = e - g; float s1, s2; memcpy(&s1, &s1b, 4); memcpy(&s2, &s2b, 4);
    if (fabsf(n) > 192.0f) return s1 * s1;
    return fmaf(s2, j, s2) * s1;
}

/* ggml_compute_forward_soft_max_f32 (ops.cpp:4641-4737) + ggml_vec_soft_max_f32 AVX2 (vec.cpp:194-245); mask row = row % ne01 */
void orc_soft_max(const float * x, const float * mask_f32, const uint16_t * mask_f16, float * y, int64_t ne0, int64_t nrows, int64_t ne01, float scale) {
    float * wp = (float *) malloc((size_t) ne0 * sizeof(float));
    for (int64_t r = 0; r < nrows; ++r) {
        const float * sp = x + r * ne0; float * dp = y + r * ne0;
        for (int64_t i = 0; i < ne0; ++i) wp[i] = sp[i] * scale;
        if (mask_f32) for (int64_t i = 0; i < ne0; ++i) wp[i] += mask_f32[(r % ne01) * ne0 + i];
        if (mask_f16) for (int64_t i = 0; i < ne0; ++i) wp[i] += h2f(mask_f16[(r % ne01) * ne0 + i]);
        float mx = -INFINITY;
        for (int64_t i = 0; i < ne0; ++i) if (wp[i] > mx) mx = wp[i];
        double sum = 0.0;
        int64_t i = 0;
        for (; i + 7 < ne0; i += 8) {
            float val[8];
            for (int t = 0; t < 8; ++t) { val[t] = v_expf(wp[i + t] - mx); dp[i + t] = val[t]; }
            const float a0 = val[4] + val[0], a1 = val[5] + val[1], a2 = val[6] + val[2], a3 = val[7] + val[3];
            const float b0 = a0 + a2, b1 = a1 + a3;
            sum += (double) (b0 + b1);
        }
        for (; i < ne0; ++i) { const float val = expf(wp[i] - mx); sum += (double) val; dp[i] = val; }
        const float inv = (float) (1.0 / sum);
        for (int64_t t = 0; t < ne0; ++t) dp[t] = dp[t] * inv;
    }
    free(wp);
}

/* ggml_compute_forward_im2col_f16, 1-D (ops.cpp:5784-5855): x f32 [IC][IW] -> dst f16 [OW][IC*KW] */
void orc_im2col_1d(const float * x, int64_t IW, int64_t IC, int64_t KW, int64_t OW, int s0, int p0, int d0, uint16_t * dst) {
    for (int64_t iow = 0; iow < OW; ++iow) for (int64_t iic = 0; iic < IC; ++iic) for (int64_t ikw = 0; ikw < KW; ++ikw) {
        const int64_t iiw = iow * s0 + ikw * d0 - p0;
        dst[iow * IC * KW + iic * KW + ikw] = (iiw < 0 || iiw >= IW) ? 0 : f2h(x[iic * IW + iiw]);
    }
}

/* ---- log-mel (src/whisper.cpp:3008-3271; that file is built without FMA) -------------------------- */
static float g_sin[400], g_cos[400], g_hann[400];
static int g_mel_init = 0;
static void mel_init(void) {
    if (g_mel_init) return;
    for (int i = 0; i < 400; i++) {
        double theta = (2 * M_PI * i) / 400;
        g_sin[i] = sinf(theta); g_cos[i] = cosf(theta);
        g_hann[i] = 0.5 * (1.0 - cosf((2.0 * M_PI * i) / 400));
    }
    g_mel_init = 1;
}
static void dft(const float * in, int N, float * out) {
    const int step = 400 / N;
    for (int k = 0; k < N; k++) {
        float re = 0, im = 0;
        for (int n = 0; n < N; n++) { int idx = (k * n * step) % 400; re += in[n] * g_cos[idx]; im -= in[n] * g_sin[idx]; }
        out[k * 2 + 0] = re; out[k * 2 + 1] = im;
    }
}
static void fft(float * in, int N, float * out) {
    if (N == 1) { out[0] = in[0]; out[1] = 0; return; }
    const int half_N = N / 2;
    if (N - half_N * 2 == 1) { dft(in, N, out); return; }
    float * even = in + N;
    for (int i = 0; i < half_N; ++i) even[i] = in[2 * i];
    float * even_fft = out + 2 * N;
    fft(even, half_N, even_fft);
    float * odd = even;
    for (int i = 0; i < half_N; ++i) odd[i] = in[2 * i + 1];
    float * odd_fft = even_fft + N;
    fft(odd, half_N, odd_fft);
    const int step = 400 / N;
    for (int k = 0; k < half_N; k++) {
        int idx = k * step;
        float re = g_cos[idx], im = -g_sin[idx];
        float re_odd = odd_fft[2 * k + 0], im_odd = odd_fft[2 * k + 1];
        out[2 * k + 0] = even_fft[2 * k + 0] + re * re_odd - im * im_odd;
        out[2 * k + 1] = even_fft[2 * k + 1] + re * im_odd + im * re_odd;
        out[2 * (k + half_N) + 0] = even_fft[2 * k + 0] - re * re_odd + im * im_odd;
        out[2 * (k + half_N) + 1] = even_fft[2 * k + 1] - re * im_odd - im * re_odd;
    }
}
/* returns n_len; mel = [n_mel][n_len] */
int orc_log_mel(const float * pcm, int64_t n_samples, const float * filters, int n_mel, float * mel, int64_t cap) {
    mel_init();
    const int64_t pad1 = 16000 * 30, pad2 = 200;
    const int64_t n_padded = n_samples + pad1 + 2 * pad2;
    const int n_len = (int) ((n_padded - 400) / 160);
    if ((int64_t) n_mel * n_len > cap) return -1;
    float * sp = (float *) calloc((size_t) n_padded, sizeof(float));
    memcpy(sp + pad2, pcm, (size_t) n_samples * sizeof(float));
    for (int64_t i = 0; i < pad2; ++i) sp[i] = pcm[pad2 - i];
    const int64_t n_valid = n_samples + pad2;
    float fft_in[800], fft_out[3200];
    int i = 0;
    const int n_frames = (int) (n_valid / 160 + 1) < n_len ? (int) (n_valid / 160 + 1) : n_len;
    for (; i < n_frames; ++i) {
        const int64_t offset = (int64_t) i * 160;
        memset(fft_in, 0, sizeof(fft_in));
        const int64_t lim = n_valid - offset < 400 ? n_valid - offset : 400;
        for (int64_t j = 0; j < lim; j++) fft_in[j] = g_hann[j] * sp[offset + j];
        fft(fft_in, 400, fft_out);
        for (int j = 0; j < 201; j++) fft_out[j] = (fft_out[2 * j + 0] * fft_out[2 * j + 0] + fft_out[2 * j + 1] * fft_out[2 * j + 1]);
        for (int j = 0; j < n_mel; j++) {
            double sum = 0.0;
            int k = 0;
            for (k = 0; k < 201 - 3; k += 4) {
                sum += fft_out[k + 0] * filters[j * 201 + k + 0] + fft_out[k + 1] * filters[j * 201 + k + 1] +
                       fft_out[k + 2] * filters[j * 201 + k + 2] + fft_out[k + 3] * filters[j * 201 + k + 3];
            }
            for (; k < 201; k++) sum += fft_out[k] * filters[j * 201 + k];
            sum = log10(sum > 1e-10 ? sum : 1e-10);
            mel[(int64_t) j * n_len + i] = sum;
        }
    }
    const double fill = log10(1e-10);
    for (; i < n_len; ++i) for (int j = 0; j < n_mel; j++) mel[(int64_t) j * n_len + i] = fill;
    double mmax = -1e20;
    for (int64_t t = 0; t < (int64_t) n_mel * n_len; t++) if (mel[t] > mmax) mmax = mel[t];
    mmax -= 8.0;
    for (int64_t t = 0; t < (int64_t) n_mel * n_len; t++) {
        if (mel[t] < mmax) mel[t] = mmax;
        mel[t] = (mel[t] + 4.0) / 4.0;
    }
    free(sp);
    return n_len;
}
