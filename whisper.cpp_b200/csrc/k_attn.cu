// Attention kernels that keep the arithmetic order of the reference CPU backend:
//  * flash_attn_ext with F16 K/V (ggml/src/ggml-cpu/ops.cpp:6638-6851): scores by the f16 dot
//    product order of vec.cpp:128-167, one key after the other through the online softmax, the V
//    accumulator held in F16 and rounded after every key (vec.h:180-197, 295-322), exp() as glibc's
//    expf (table of 2^(i/32) + degree-3 polynomial in double);
//  * soft_max (ops.cpp:4641-4737) with the vectorised exp of vec.h:603-640 and its 8-wide sums.
#include "b200_common.cuh"
#include <stdlib.h>
#include <math.h>
#include <mutex>

// ---- glibc expf -----------------------------------------------------------------------------
__constant__ uint64_t c_exp2f_tab[32];

static void ensure_exp_table() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64 || done[dev]) return;
    uint64_t tab[32];
    for (int i = 0; i < 32; ++i) {
        const double v = (double) exp2l((long double) i / 32.0L);
        uint64_t bits;
        memcpy(&bits, &v, 8);
        tab[i] = bits - ((uint64_t) i << 47);
    }
    cudaMemcpyToSymbol(c_exp2f_tab, tab, sizeof(tab));
    done[dev] = true;
}

// tab: the 32-entry 2^(i/32) table in SHARED memory (every lane indexes it differently; the same lookup in constant
// memory is serialised per distinct address)
__device__ __forceinline__ float expf_glibc(float x, const uint64_t * tab) {
    const uint32_t ux = __float_as_uint(x);
    const uint32_t abstop = (ux >> 20) & 0x7ffu;
    if (abstop >= 0x42bu) {                       // |x| >= 88
        if (ux == 0xff800000u) return 0.0f;       // -inf
        if (abstop >= 0x7f8u) return x + x;       // nan, +inf
        if (x > 0x1.62e42ep6f) return __int_as_float(0x7f800000);
        if (x < -0x1.9fe368p6f) return 0.0f;
    }
    const double InvLn2N = 0x1.71547652b82fep+0 * 32.0;
    const double Shift   = 0x1.8p+52;
    const double C0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double C1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double C2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double xd = (double) x;
    double z  = __dmul_rn(InvLn2N, xd);
    double kd = __dadd_rn(z, Shift);
    const uint64_t ki = (uint64_t) __double_as_longlong(kd);
    kd = __dadd_rn(kd, -Shift);
    const double r = __dadd_rn(z, -kd);
    uint64_t t = tab[ki & 31];
    t += ki << 47;
    const double s = __longlong_as_double((long long) t);
    z = __fma_rn(C0, r, C1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(C2, r, 1.0);
    y = __fma_rn(z, r2, y);
    y = __dmul_rn(y, s);
    return (float) y;
}

// ---- flash attention ------------------------------------------------------------------------
// Many query rows (encoder, prompts): a warp owns FA_R consecutive query rows of one head.  Per 32 keys: every lane
// loads one key row once and scores it against the FA_R queries with the exact reduction tree, a prefix maximum per
// query tells each key the running maximum it meets, exp() runs in parallel, then the 64-wide F16 accumulators
// (two dims per lane, FA_R independent chains) are updated key by key.  HAS_SKIP = a mask is present or the key count
// is not a multiple of 32; without it the per-key "skipped" handling is compiled out.
// RELAXED (measurement switch GGML_B200_RELAXED=1, off by default): what a tensor-core attention would do instead - the
// softmax weights rounded to F16 once, the V accumulator kept in f32 - to measure how far that moves the model outputs.
// MIXED: the key/query products use the mixed-precision FMA of sm_100 (two f16 factors, f32 addend and result: the
// same value as converting both factors first, the products of two f16 numbers being exact in f32), which drops the
// f16 -> f32 conversions of the keys and halves the shared-memory reads of the queries.
#define FA_R 4
__device__ __forceinline__ void fma_f16x2_f32(float & a0, float & a1, uint32_t kw, uint32_t qw) {
    asm("{\n\t.reg .b16 kl, kh, ql, qh;\n\t"
        "mov.b32 {kl, kh}, %2;\n\t"
        "mov.b32 {ql, qh}, %3;\n\t"
        "fma.rn.f32.f16 %0, kl, ql, %0;\n\t"
        "fma.rn.f32.f16 %1, kh, qh, %1;\n\t}"
        : "+f"(a0), "+f"(a1) : "r"(kw), "r"(qw));
}
template <bool S_FMA, bool HAS_SKIP, bool RELAXED, bool MIXED>
__global__ void __launch_bounds__(128, 5)
k_flash_attn_ext(const char * __restrict__ q, int64_t nbq1, int64_t nbq2,
                 const char * __restrict__ k, int64_t nbk1, int64_t nbk2,
                 const char * __restrict__ v, int64_t nbv1, int64_t nbv2,
                 const char * __restrict__ mask, int64_t nbm1,
                 float * __restrict__ dst, int64_t n_q, int64_t n_kv, int64_t n_head, float scale) {
    __shared__ __align__(16) float Qs[4][MIXED ? 1 : FA_R][64];
    __shared__ __align__(16) __half Qh[4][MIXED ? FA_R : 1][64];
    __shared__ __align__(16) float MS[4][FA_R][32];
    __shared__ __align__(16) float VS[4][FA_R][32];
    __shared__ uint64_t s_exp_tab[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row0 = ((int64_t) blockIdx.x * 4 + warp) * FA_R;
    const int64_t h    = blockIdx.y;
    if (row0 >= n_q) return;
    s_exp_tab[lane] = c_exp2f_tab[lane];      // every warp writes the same 32 values; visible to this warp after its __syncwarp
    const int n_rows = (int) min((int64_t) FA_R, n_q - row0);

#pragma unroll
    for (int r = 0; r < FA_R; ++r) {
        const int64_t iq = min(row0 + r, n_q - 1);             // rows past the end repeat the last one and are not stored
        const float * qp = (const float *) (q + iq * nbq1 + h * nbq2);
        if (MIXED) {
            Qh[warp][r][lane]      = __float2half_rn(qp[lane]);
            Qh[warp][r][lane + 32] = __float2half_rn(qp[lane + 32]);
        } else {
            Qs[warp][r][lane]      = round_f16(qp[lane]);
            Qs[warp][r][lane + 32] = round_f16(qp[lane + 32]);
        }
    }
    __syncwarp();

    const char * kh = k + h * nbk2;
    const char * vh = v + h * nbv2;

    float M[FA_R], S[FA_R], a0[FA_R], a1[FA_R];
#pragma unroll
    for (int r = 0; r < FA_R; ++r) { M[r] = -INFINITY; S[r] = 0.0f; a0[r] = 0.0f; a1[r] = 0.0f; }

    for (int64_t ic0 = 0; ic0 < n_kv; ic0 += 32) {
        const int64_t ic = ic0 + lane;
        const bool valid = !HAS_SKIP || ic < n_kv;
        uint4 kreg[8];
        if (valid) {
            const uint4 * kp = (const uint4 *) (kh + ic * nbk1);
#pragma unroll
            for (int c = 0; c < 8; ++c) kreg[c] = kp[c];
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) kreg[c] = make_uint4(0, 0, 0, 0);
        }
        unsigned evt_any = 0;
#pragma unroll
        for (int r = 0; r < FA_R; ++r) {
            float mv = 0.0f;
            bool skip = !valid;
            if (HAS_SKIP && mask && valid) {
                const int64_t iq = min(row0 + r, n_q - 1);
                mv = __half2float(((const __half *) (mask + iq * nbm1))[ic]);
                skip = (mv == -INFINITY);
            }
            float s = -INFINITY;
            if (!skip) {
                float acc[32];
                if (MIXED) {
#pragma unroll
                    for (int p = 0; p < 32; ++p) acc[p] = 0.0f;
                }
#pragma unroll
                for (int step = 0; step < 2; ++step) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint4 kv = kreg[step * 4 + c];
                        if (MIXED) {
                            const uint4 qv = *(const uint4 *) &Qh[warp][r][step * 32 + c * 8];
                            float * a = &acc[c * 8];
                            fma_f16x2_f32(a[0], a[1], kv.x, qv.x);
                            fma_f16x2_f32(a[2], a[3], kv.y, qv.y);
                            fma_f16x2_f32(a[4], a[5], kv.z, qv.z);
                            fma_f16x2_f32(a[6], a[7], kv.w, qv.w);
                            continue;
                        }
                        const float4 qa = *(const float4 *) &Qs[warp][r][step * 32 + c * 8];
                        const float4 qb = *(const float4 *) &Qs[warp][r][step * 32 + c * 8 + 4];
                        const float2 k0 = __half22float2(*(const __half2 *) &kv.x);
                        const float2 k1 = __half22float2(*(const __half2 *) &kv.y);
                        const float2 k2 = __half22float2(*(const __half2 *) &kv.z);
                        const float2 k3 = __half22float2(*(const __half2 *) &kv.w);
                        float * a = &acc[c * 8];
                        if (step == 0) {
                            a[0] = __fmaf_rn(k0.x, qa.x, 0.0f); a[1] = __fmaf_rn(k0.y, qa.y, 0.0f);
                            a[2] = __fmaf_rn(k1.x, qa.z, 0.0f); a[3] = __fmaf_rn(k1.y, qa.w, 0.0f);
                            a[4] = __fmaf_rn(k2.x, qb.x, 0.0f); a[5] = __fmaf_rn(k2.y, qb.y, 0.0f);
                            a[6] = __fmaf_rn(k3.x, qb.z, 0.0f); a[7] = __fmaf_rn(k3.y, qb.w, 0.0f);
                        } else {
                            a[0] = __fmaf_rn(k0.x, qa.x, a[0]); a[1] = __fmaf_rn(k0.y, qa.y, a[1]);
                            a[2] = __fmaf_rn(k1.x, qa.z, a[2]); a[3] = __fmaf_rn(k1.y, qa.w, a[3]);
                            a[4] = __fmaf_rn(k2.x, qb.x, a[4]); a[5] = __fmaf_rn(k2.y, qb.y, a[5]);
                            a[6] = __fmaf_rn(k3.x, qb.z, a[6]); a[7] = __fmaf_rn(k3.y, qb.w, a[7]);
                        }
                    }
                }
                float y[8];
#pragma unroll
                for (int p = 0; p < 8; ++p)
                    y[p] = __fadd_rn(__fadd_rn(acc[p], acc[16 + p]), __fadd_rn(acc[8 + p], acc[24 + p]));
                const float t0 = __fadd_rn(y[0], y[4]), t1 = __fadd_rn(y[1], y[5]);
                const float t2 = __fadd_rn(y[2], y[6]), t3 = __fadd_rn(y[3], y[7]);
                s = __fadd_rn(__fadd_rn(t0, t1), __fadd_rn(t2, t3));
                s = __fmul_rn(s, scale);
                s = __fadd_rn(s, mv);
            }
            // running maximum seen by each key (exclusive prefix over non-skipped keys; skipped keys carry -inf)
            float pm = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, pm, o);
                if (lane >= o) pm = fmaxf(pm, t);
            }
            float ex = __shfl_up_sync(0xffffffffu, pm, 1);
            if (lane == 0) ex = -INFINITY;
            const float Mprev  = fmaxf(M[r], ex);
            const bool  newmax = !skip && (s > Mprev);
            float e = 1.0f;
            if (!skip) e = expf_glibc(newmax ? __fadd_rn(Mprev, -s) : __fadd_rn(s, -Mprev), s_exp_tab);
            MS[warp][r][lane] = newmax ? e : 1.0f;
            VS[warp][r][lane] = skip ? -0.0f : (newmax ? 1.0f : e);
            if (__ballot_sync(0xffffffffu, newmax)) evt_any |= 1u << r;
            M[r] = fmaxf(M[r], __shfl_sync(0xffffffffu, pm, 31));
        }
        __syncwarp();

        // V rows of the 32 keys (two dims per lane), shared by the FA_R chains: four keys at a time, the next four are
        // requested while these are used.  The loop is kept rolled (two groups per trip): the fully unrolled form is
        // tens of kilobytes of code and the warps then wait for instruction fetch.
        auto load4 = [&](int i0, __half2 (&v)[4]) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (!HAS_SKIP || ic0 + i0 + u < n_kv) v[u] = *(const __half2 *) (vh + (ic0 + i0 + u) * nbv1 + lane * 4);
                else                                  v[u] = __floats2half2_rn(0.0f, 0.0f);
            }
        };
        auto use4 = [&](int i0, const __half2 (&v)[4]) {
            float4 vs4[FA_R];
#pragma unroll
            for (int r = 0; r < FA_R; ++r) vs4[r] = *(const float4 *) &VS[warp][r][i0];
            if (evt_any == 0) {            // no row met a new maximum in this block: ms == 1 everywhere
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 vf = __half22float2(v[u]);
#pragma unroll
                    for (int r = 0; r < FA_R; ++r) {
                        const float vs = u == 0 ? vs4[r].x : u == 1 ? vs4[r].y : u == 2 ? vs4[r].z : vs4[r].w;
                        float vx = vf.x, vy = vf.y;
                        if (HAS_SKIP && __float_as_uint(vs) == 0x80000000u) { vx = 0.0f; vy = 0.0f; }    // skipped key: exact no-op
                        S[r] = __fadd_rn(S[r], vs);          // ms == 1: fma(S, 1, vs) == S + vs
                        if (RELAXED) { const float p = round_f16(vs); a0[r] = __fmaf_rn(vx, p, a0[r]); a1[r] = __fmaf_rn(vy, p, a1[r]); }
                        else {
                            const float2 t = __half22float2(__floats2half2_rn(__fmaf_rn(vx, vs, a0[r]), __fmaf_rn(vy, vs, a1[r])));
                            a0[r] = t.x; a1[r] = t.y;
                        }
                    }
                }
                return;
            }
            float4 ms4[FA_R];
#pragma unroll
            for (int r = 0; r < FA_R; ++r) ms4[r] = *(const float4 *) &MS[warp][r][i0];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float2 vf = __half22float2(v[u]);
#pragma unroll
                for (int r = 0; r < FA_R; ++r) {
                    const float vs = u == 0 ? vs4[r].x : u == 1 ? vs4[r].y : u == 2 ? vs4[r].z : vs4[r].w;
                    const float ms = u == 0 ? ms4[r].x : u == 1 ? ms4[r].y : u == 2 ? ms4[r].z : ms4[r].w;
                    float vx = vf.x, vy = vf.y;
                    if (HAS_SKIP && __float_as_uint(vs) == 0x80000000u) { vx = 0.0f; vy = 0.0f; }
                    if ((evt_any >> r) & 1u) {
                        if (ms != 1.0f) {
                            if (RELAXED) { a0[r] = __fmul_rn(a0[r], ms); a1[r] = __fmul_rn(a1[r], ms); }
                            else {
                                const float2 t = __half22float2(__floats2half2_rn(__fmul_rn(a0[r], ms), __fmul_rn(a1[r], ms)));
                                a0[r] = t.x; a1[r] = t.y;
                            }
                        }
                        S[r] = S_FMA ? __fmaf_rn(S[r], ms, vs) : __fadd_rn(__fmul_rn(S[r], ms), vs);
                    } else {
                        S[r] = __fadd_rn(S[r], vs);
                    }
                    if (RELAXED) { const float p = round_f16(vs); a0[r] = __fmaf_rn(vx, p, a0[r]); a1[r] = __fmaf_rn(vy, p, a1[r]); }
                    else {
                        const float2 t = __half22float2(__floats2half2_rn(__fmaf_rn(vx, vs, a0[r]), __fmaf_rn(vy, vs, a1[r])));
                        a0[r] = t.x; a1[r] = t.y;
                    }
                }
            }
        };
        __half2 va[4], vb4[4];
        load4(0, va);
#pragma unroll 1
        for (int i0 = 0; i0 < 32; i0 += 8) {
            load4(i0 + 4, vb4);
            use4(i0, va);
            if (i0 + 8 < 32) load4(i0 + 8, va);
            use4(i0 + 4, vb4);
        }
        __syncwarp();
    }

#pragma unroll
    for (int r = 0; r < FA_R; ++r) {
        if (r < n_rows) {
            const float S_inv = __fdiv_rn(1.0f, S[r]);
            float2 o;
            o.x = __fmul_rn(a0[r], S_inv);
            o.y = __fmul_rn(a1[r], S_inv);
            *(float2 *) (dst + ((row0 + r) * n_head + h) * 64 + lane * 2) = o;
        }
    }
}

// Few query rows (token-by-token decode, beams, several decoder states stepping together): one CTA per
// (query row, head).  The work of the kernel above is split by role so that the sequential part is as short as
// possible: all threads score the keys, a block scan gives every key the running maximum it meets, exp() runs in
// parallel, then 64 threads (one per output dim) replay the F16 accumulation key by key while one more thread
// replays the running sum.  Every query row carries its own K/V/mask/output pointers and key count.
#define FA_DEC_THREADS 128
#define FA_DEC_MAX_KV  8192
#define FA_DEC_CHUNK   64
#define FA_DEC_MAX_ROWS 32
struct FaRow {
    const char * q;        // 64 f32 per head, head stride nbq2
    const char * k;        // f16 [64, n_kv, H], strides nbk1, nbk2
    const char * v;
    const char * mask;     // f16 row of this query (n_kv entries) or NULL
    float *      dst;      // [H][64] f32 of this query row
    int          n_kv;
};
struct FaRows {
    FaRow r[FA_DEC_MAX_ROWS];
    int64_t nbq2, nbk1, nbk2, nbv1, nbv2;
    float scale;
};

// STAGES buffers of FA_DEC_CHUNK keys: STAGES - 1 chunks are in flight ahead of the one in use (3: small enough for all
// CTAs of 32 rows x 20 heads to be resident at once; 6 was measured and changes nothing, the CTA is bound by its chains)
#ifdef FA_DEC_PROFILE
__device__ long long g_fa_prof[8];
#define FA_PROF(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g_fa_prof[i] = clock64(); } while (0)
extern "C" int b200_fa_prof_read(long long * out) { return (int) cudaMemcpyFromSymbol(out, g_fa_prof, sizeof(g_fa_prof)); }
#else
#define FA_PROF(i) do { } while (0)
#endif
template <bool S_FMA, int STAGES>
__global__ void __launch_bounds__(FA_DEC_THREADS)
k_flash_attn_decode(FaRows rows, int max_kv, int8_t * __restrict__ xq, float * __restrict__ xd) {
    extern __shared__ __align__(16) float fa_smem[];
    // heads of one query row are neighbours in launch order: they walk the same K/V rows (d_model wide, 128 bytes per
    // head) at about the same time, which keeps the DRAM pages they share open
    const FaRow & R = rows.r[blockIdx.y];
    const int n_kv = R.n_kv;
    float * Qs  = fa_smem;                 // [64]
    float * sc  = Qs + 64;                 // [n_kv] scores, later vs (-0.0f marks a skipped key)
    float * msv = sc + max_kv;             // [n_kv] ms (1 unless a new maximum)
    unsigned char * evt = (unsigned char *) (msv + max_kv);                 // [n_kv/8] group contains a new maximum
    __half * Vs = (__half *) (fa_smem + ((64 + 2 * max_kv + (max_kv + 31) / 32 + 3) & ~3));   // [STAGES][FA_DEC_CHUNK][64], 16-byte aligned
    __shared__ float seg_max[FA_DEC_THREADS];
    __shared__ float s_S;
    __shared__ uint64_t s_exp_tab[32];
    const int tid = threadIdx.x;
    const int64_t h = blockIdx.x;
    const int64_t nbk1 = rows.nbk1, nbv1 = rows.nbv1;
    const float scale = rows.scale;
    chain_wait();                          // Q, and for self-attention the newest K/V rows, come from the kernels before this one
    FA_PROF(0);

    if (tid < 64) Qs[tid] = round_f16(*(const float *) (R.q + h * rows.nbq2 + tid * 4));
    if (tid >= 96) s_exp_tab[tid - 96] = c_exp2f_tab[tid - 96];
    for (int g = tid; g < (n_kv + 7) / 8; g += FA_DEC_THREADS) evt[g] = 0;
    __syncthreads();

    const char * kh = R.k + h * rows.nbk2;
    const char * vh = R.v + h * rows.nbv2;
    const __half * mp = (const __half *) R.mask;

    // scores: K is streamed through shared memory in chunks of FA_DEC_CHUNK keys (the buffers V uses later), copied
    // asynchronously in 16-byte pieces that are contiguous in global memory; the eight pieces of a key row are stored
    // XOR-swizzled by the key index so that the threads of a warp, one key each, read them without bank conflicts.
    // Warps 0..1 score chunk c while chunks c+1 and c+2 are in flight.
    {
        const int n_chunks = (n_kv + FA_DEC_CHUNK - 1) / FA_DEC_CHUNK;
        auto fetch_k = [&](int c) {
            const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);      // kn <= 0 beyond the last chunk: empty group
            const unsigned base = (unsigned) __cvta_generic_to_shared(Vs + (size_t) (c % STAGES) * FA_DEC_CHUNK * 64);
            for (int t = tid; t < kn * 8; t += FA_DEC_THREADS) {
                const int key = t >> 3, pc = t & 7;
                const char * src = kh + (int64_t) (k0 + key) * nbk1 + pc * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(base + key * 128 + ((pc ^ (key & 7)) << 4)), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // one group is committed per prologue slot and per iteration (empty beyond the last chunk), so chunk c is always
        // followed by exactly STAGES - 2 younger groups when it is waited for
#pragma unroll
        for (int c = 0; c < STAGES - 1; ++c) fetch_k(c);
        for (int c = 0; c < n_chunks; ++c) {
            const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
            asm volatile("cp.async.wait_group %0;" :: "n"(STAGES - 2) : "memory");
            __syncthreads();
            fetch_k(c + STAGES - 1);
            if (tid < kn) {
                const int ic = k0 + tid;
                float mv = 0.0f;
                if (mp) mv = __half2float(mp[ic]);
                float s = -INFINITY;
                const bool skip = (mv == -INFINITY);
                if (!skip) {
                    float acc[32];
                    const char * krow = (const char *) (Vs + (size_t) (c % STAGES) * FA_DEC_CHUNK * 64) + tid * 128;
#pragma unroll
                    for (int step = 0; step < 2; ++step) {
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            const uint4 kv = *(const uint4 *) (krow + (((step * 4 + cc) ^ (tid & 7)) << 4));
                            const float4 qa = *(const float4 *) &Qs[step * 32 + cc * 8];
                            const float4 qb = *(const float4 *) &Qs[step * 32 + cc * 8 + 4];
                            const float2 k0v = __half22float2(*(const __half2 *) &kv.x);
                            const float2 k1v = __half22float2(*(const __half2 *) &kv.y);
                            const float2 k2v = __half22float2(*(const __half2 *) &kv.z);
                            const float2 k3v = __half22float2(*(const __half2 *) &kv.w);
                            float * a = &acc[cc * 8];
                            if (step == 0) {
                                a[0] = __fmaf_rn(k0v.x, qa.x, 0.0f); a[1] = __fmaf_rn(k0v.y, qa.y, 0.0f);
                                a[2] = __fmaf_rn(k1v.x, qa.z, 0.0f); a[3] = __fmaf_rn(k1v.y, qa.w, 0.0f);
                                a[4] = __fmaf_rn(k2v.x, qb.x, 0.0f); a[5] = __fmaf_rn(k2v.y, qb.y, 0.0f);
                                a[6] = __fmaf_rn(k3v.x, qb.z, 0.0f); a[7] = __fmaf_rn(k3v.y, qb.w, 0.0f);
                            } else {
                                a[0] = __fmaf_rn(k0v.x, qa.x, a[0]); a[1] = __fmaf_rn(k0v.y, qa.y, a[1]);
                                a[2] = __fmaf_rn(k1v.x, qa.z, a[2]); a[3] = __fmaf_rn(k1v.y, qa.w, a[3]);
                                a[4] = __fmaf_rn(k2v.x, qb.x, a[4]); a[5] = __fmaf_rn(k2v.y, qb.y, a[5]);
                                a[6] = __fmaf_rn(k3v.x, qb.z, a[6]); a[7] = __fmaf_rn(k3v.y, qb.w, a[7]);
                            }
                        }
                    }
                    float y[8];
#pragma unroll
                    for (int pp = 0; pp < 8; ++pp)
                        y[pp] = __fadd_rn(__fadd_rn(acc[pp], acc[16 + pp]), __fadd_rn(acc[8 + pp], acc[24 + pp]));
                    const float t0 = __fadd_rn(y[0], y[4]), t1 = __fadd_rn(y[1], y[5]);
                    const float t2 = __fadd_rn(y[2], y[6]), t3 = __fadd_rn(y[3], y[7]);
                    s = __fadd_rn(__fadd_rn(t0, t1), __fadd_rn(t2, t3));
                    s = __fmul_rn(s, scale);
                    s = __fadd_rn(s, mv);
                }
                sc[ic]  = s;                       // -inf for skipped keys: never a new maximum
                msv[ic] = skip ? -1.0f : 1.0f;     // temporary skip mark
            }
        }
    }
    __syncthreads();

    FA_PROF(1);
    // V takes over the buffers: its first two chunks are requested now and arrive while the maxima and exponentials
    // below are computed
    const int n_chunks = (n_kv + FA_DEC_CHUNK - 1) / FA_DEC_CHUNK;
    auto fetch = [&](int c) {
        const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
        const unsigned base = (unsigned) __cvta_generic_to_shared(Vs + (size_t) (c % STAGES) * FA_DEC_CHUNK * 64);
        for (int t = tid; t < kn * 8; t += FA_DEC_THREADS) {
            const char * src = vh + (int64_t) (k0 + (t >> 3)) * nbv1 + (t & 7) * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(base + t * 16), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int c = 0; c < STAGES - 1; ++c) fetch(c);

    // contiguous segment per thread: segment maxima, exclusive block scan, then the per-key pass
    const int seg = (n_kv + FA_DEC_THREADS - 1) / FA_DEC_THREADS;
    const int i0 = min(n_kv, tid * seg), i1 = min(n_kv, i0 + seg);
    float m = -INFINITY;
    for (int i = i0; i < i1; ++i) m = fmaxf(m, sc[i]);
    seg_max[tid] = m;
    __syncthreads();
    if (tid < 32) {                        // exclusive prefix maximum over the segment maxima
        float carry = -INFINITY;
        for (int base = 0; base < FA_DEC_THREADS; base += 32) {
            const float x = seg_max[base + tid];
            float inc = x;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, inc, o);
                if (tid >= o) inc = fmaxf(inc, t);
            }
            float exc = __shfl_up_sync(0xffffffffu, inc, 1);
            if (tid == 0) exc = -INFINITY;
            seg_max[base + tid] = fmaxf(carry, exc);
            carry = fmaxf(carry, __shfl_sync(0xffffffffu, inc, 31));
        }
    }
    __syncthreads();
    {
        // the running maximum is a cheap sequential chain; the exponentials (double precision inside) do not depend on
        // each other, so four keys are taken at a time with the branches turned into selects
        float M = seg_max[tid];
        int i = i0;
        for (; i + 4 <= i1; i += 4) {
            float arg[4], e[4];
            bool skipk[4], newmax[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float s = sc[i + u];
                skipk[u]  = msv[i + u] < 0.0f;
                newmax[u] = !skipk[u] && s > M;
                arg[u] = newmax[u] ? __fadd_rn(M, -s) : __fadd_rn(s, -M);
                if (skipk[u]) arg[u] = 0.0f;
                if (newmax[u]) M = s;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) e[u] = expf_glibc(arg[u], s_exp_tab);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (skipk[u])       { msv[i + u] = 1.0f; sc[i + u] = -0.0f; }               // skipped: ms = 1, vs = -0
                else if (newmax[u]) { msv[i + u] = e[u]; sc[i + u] = 1.0f; evt[(i + u) >> 3] = 1; }
                else                { sc[i + u] = e[u]; }
            }
        }
        for (; i < i1; ++i) {
            if (msv[i] < 0.0f) { msv[i] = 1.0f; sc[i] = -0.0f; continue; }
            const float s = sc[i];
            if (s > M) { msv[i] = expf_glibc(__fadd_rn(M, -s), s_exp_tab); sc[i] = 1.0f; M = s; evt[i >> 3] = 1; }
            else       { sc[i] = expf_glibc(__fadd_rn(s, -M), s_exp_tab); }
        }
    }
    __syncthreads();

    FA_PROF(2);
    // V is streamed through shared memory in chunks of FA_DEC_CHUNK keys, STAGES buffers: chunks c+1 and c+2 are
    // being copied asynchronously while warps 0..1 (one thread per output dim) replay the F16 accumulation over chunk c
    // and one thread of warp 2 replays the running sum.  The buffers are kept small so that every (row, head) CTA of 32
    // rows x 20 heads is resident at once (no second wave).  Keys are taken eight at a time with all operands in registers; only groups that
    // contain a new maximum take the path that rescales the accumulator.
    {
        float a = 0.0f, S = 0.0f;
        for (int c = 0; c < n_chunks; ++c) {
            const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
            // chunk c has landed (at most the group of chunk c+1 may still be in flight); the barrier also says that
            // everybody is done with chunk c-1, whose buffer chunk c+2 reuses
            asm volatile("cp.async.wait_group %0;" :: "n"(STAGES - 2) : "memory");
            __syncthreads();
            fetch(c + STAGES - 1);
            if (tid < 64) {
                const __half * vb = Vs + (size_t) (c % STAGES) * FA_DEC_CHUNK * 64 + tid;
                int i = 0;
                // Common case, a full chunk without a new maximum: straight-line blocks of dependent steps, so that the
                // compiler can place the shared-memory loads and conversions of later keys into the latency gaps of the chain
                // (a warp issues in order; with loops or branches in between it would wait for the loads instead).
                if (kn == FA_DEC_CHUNK && *(const unsigned long long *) &evt[k0 >> 3] == 0ull) {
                    // blocks of 16 steps: long enough to hide the loads, short enough to stay in the instruction cache
#pragma unroll 1
                    for (int ub = 0; ub < FA_DEC_CHUNK; ub += 16) {
#pragma unroll
                        for (int u = 0; u < 16; ++u) {
                            const float vsu = sc[k0 + ub + u];
                            float vvu = __half2float(vb[(ub + u) * 64]);
                            if (__float_as_uint(vsu) == 0x80000000u) vvu = 0.0f;     // skipped key: exact no-op whatever V holds
                            a = round_f16(__fmaf_rn(vvu, vsu, a));
                        }
                    }
                    i = FA_DEC_CHUNK;
                }
                for (; i + 8 <= kn; i += 8) {
                    float vs[8], vv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        vs[u] = sc[k0 + i + u];
                        vv[u] = __half2float(vb[(i + u) * 64]);
                        if (__float_as_uint(vs[u]) == 0x80000000u) vv[u] = 0.0f;
                    }
                    if (!evt[(k0 + i) >> 3]) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) a = round_f16(__fmaf_rn(vv[u], vs[u], a));
                    } else {
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float ms = msv[k0 + i + u];
                            if (ms != 1.0f) a = round_f16(__fmul_rn(a, ms));
                            a = round_f16(__fmaf_rn(vv[u], vs[u], a));
                        }
                    }
                }
                for (; i < kn; ++i) {
                    const float ms = msv[k0 + i], vs1 = sc[k0 + i];
                    float vv1 = __half2float(vb[i * 64]);
                    if (__float_as_uint(vs1) == 0x80000000u) vv1 = 0.0f;
                    if (ms != 1.0f) a = round_f16(__fmul_rn(a, ms));
                    a = round_f16(__fmaf_rn(vv1, vs1, a));
                }
            } else if (tid == 64) {
                int i = 0;
                for (; i + 8 <= kn; i += 8) {
                    float ms[8], vs[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) { ms[u] = msv[k0 + i + u]; vs[u] = sc[k0 + i + u]; }
#pragma unroll
                    for (int u = 0; u < 8; ++u) S = S_FMA ? __fmaf_rn(S, ms[u], vs[u]) : __fadd_rn(__fmul_rn(S, ms[u]), vs[u]);
                }
                for (; i < kn; ++i) S = S_FMA ? __fmaf_rn(S, msv[k0 + i], sc[k0 + i]) : __fadd_rn(__fmul_rn(S, msv[k0 + i]), sc[k0 + i]);
            }
        }
        FA_PROF(3);
        if (tid < 64) Qs[tid] = a;         // Qs is free now
        if (tid == 64) s_S = S;
    }
    __syncthreads();
    if (tid < 64) {
        const float o = __fmul_rn(Qs[tid], __fdiv_rn(1.0f, s_S));
        R.dst[h * 64 + tid] = o;
        // optional second output: this head's two 32-blocks of the row quantised as quantize_row_q8_0 does it, in the
        // layout of b200_quantize_cols (row = blockIdx.y), for the projection that consumes the row next
        if (xq != nullptr) {
            float amax = fabsf(o);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            const float id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
            const size_t kk = (size_t) gridDim.x * 64;
            xq[blockIdx.y * kk + h * 64 + tid] = (int8_t) __float2int_rn(__fmul_rn(o, id));
            if ((tid & 31) == 0) xd[blockIdx.y * (kk >> 5) + h * 2 + (tid >> 5)] = round_f16(__fdiv_rn(amax, 127.f));
        }
    }
}

// Streaming form of the kernel above for launches whose CTAs are all resident with the larger buffers.  Four warps,
// four roles: warp 0 replays the F16 accumulation (two output dims per lane, so two independent chains fill each
// other's latency) and the running sum over chunk c; warp 1 issues and awaits every cp.async; warps 2..3 score chunk
// c+1 (one key per thread, running maximum carried from chunk to chunk, exponentials).  The sequential chain is the
// only thing on the critical path.  K and V arrive through separate three-stage rings of FA_DEC_CHUNK keys.
template <bool S_FMA>
__global__ void __launch_bounds__(FA_DEC_THREADS)
k_flash_attn_decode_stream(FaRows rows, int max_kv, int8_t * __restrict__ xq, float * __restrict__ xd) {
    extern __shared__ __align__(16) float fa_smem[];
    const FaRow & R = rows.r[blockIdx.y];
    const int n_kv = R.n_kv;
    float * Qs  = fa_smem;                 // [64]
    float * sc  = Qs + 64;                 // [n_kv] vs (-0.0f marks a skipped key)
    float * msv = sc + max_kv;             // [n_kv] ms (1 unless a new maximum)
    unsigned char * evt = (unsigned char *) (msv + max_kv);                 // [n_kv/8] group contains a new maximum
    __half * Vs = (__half *) (fa_smem + ((64 + 2 * max_kv + (max_kv + 31) / 32 + 3) & ~3));   // [3][FA_DEC_CHUNK][64], 16-byte aligned
    __half * Ks = Vs + 3 * FA_DEC_CHUNK * 64;                                                 // [3][FA_DEC_CHUNK][64], swizzled pieces
    __shared__ float s_tot[2];             // maxima of the two scorer warps over the chunk in hand
    __shared__ uint64_t s_exp_tab[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t h = blockIdx.x;
    const int64_t nbk1 = rows.nbk1, nbv1 = rows.nbv1;
    const float scale = rows.scale;
    chain_wait();                          // Q, and for self-attention the newest K/V rows, come from the kernels before this one

    __half * Qh = (__half *) Qs;           // the query as f16: the scores use the mixed-precision FMA (f16 factors, f32 sum)
    if (tid < 64) Qh[tid] = __float2half_rn(*(const float *) (R.q + h * rows.nbq2 + tid * 4));
    if (tid >= 96) s_exp_tab[tid - 96] = c_exp2f_tab[tid - 96];
    for (int g = tid; g < (max_kv + 7) / 8; g += FA_DEC_THREADS) evt[g] = 0;

    const char * kh = R.k + h * rows.nbk2;
    const char * vh = R.v + h * rows.nbv2;
    const __half * mp = (const __half *) R.mask;
    const int n_chunks = (n_kv + FA_DEC_CHUNK - 1) / FA_DEC_CHUNK;

    // ---- warp 1: copies.  Lane l moves piece (l & 7) of keys (l >> 3) + 4 i, i = 0..15, of a chunk: source addresses
    // advance by a constant per copy and per chunk, destinations are immediates (K pieces XOR-swizzled by the key).
    const char * cp_k = kh + (int64_t) (lane >> 3) * nbk1 + (lane & 7) * 16;
    const char * cp_v = vh + (int64_t) (lane >> 3) * nbv1 + (lane & 7) * 16;
    const unsigned ks_u = (unsigned) __cvta_generic_to_shared(Ks), vs_u = (unsigned) __cvta_generic_to_shared(Vs);
    auto fetch_k = [&](int c) {            // nothing beyond the last chunk
        const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
        const unsigned base = ks_u + (unsigned) (c % 3) * FA_DEC_CHUNK * 128;
        const char * src = cp_k + (int64_t) k0 * nbk1;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int key = (lane >> 3) + 4 * i;
            if (key < kn)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(base + key * 128 + (((lane & 7) ^ (key & 7)) << 4)), "l"(src + (int64_t) (4 * i) * nbk1) : "memory");
        }
    };
    auto fetch_v = [&](int c) {
        const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
        const unsigned base = vs_u + (unsigned) (c % 3) * FA_DEC_CHUNK * 128;
        const char * src = cp_v + (int64_t) k0 * nbv1;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int key = (lane >> 3) + 4 * i;
            if (key < kn)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(base + key * 128 + ((lane & 7) << 4)), "l"(src + (int64_t) (4 * i) * nbv1) : "memory");
        }
    };

    // ---- warps 2..3: scores
    float m_carry = -INFINITY;             // maximum over all earlier chunks
    auto score_chunk = [&](int c) {        // thread j = tid - 64 scores key k0 + j
        const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
        const int j = tid - 64, ic = k0 + j;
        float s = -INFINITY;
        bool skip = true;
        if (j < kn) {
            float mv = 0.0f;
            if (mp) mv = __half2float(mp[ic]);
            skip = (mv == -INFINITY);
            if (!skip) {
                float acc[32];
#pragma unroll
                for (int pp = 0; pp < 32; ++pp) acc[pp] = 0.0f;
                const char * krow = (const char *) (Ks + (size_t) (c % 3) * FA_DEC_CHUNK * 64) + j * 128;
#pragma unroll
                for (int step = 0; step < 2; ++step) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const uint4 kv = *(const uint4 *) (krow + (((step * 4 + cc) ^ (j & 7)) << 4));
                        const uint4 qv = *(const uint4 *) (Qh + step * 32 + cc * 8);
                        float * a = &acc[cc * 8];
                        fma_f16x2_f32(a[0], a[1], kv.x, qv.x);
                        fma_f16x2_f32(a[2], a[3], kv.y, qv.y);
                        fma_f16x2_f32(a[4], a[5], kv.z, qv.z);
                        fma_f16x2_f32(a[6], a[7], kv.w, qv.w);
                    }
                }
                float y[8];
#pragma unroll
                for (int pp = 0; pp < 8; ++pp)
                    y[pp] = __fadd_rn(__fadd_rn(acc[pp], acc[16 + pp]), __fadd_rn(acc[8 + pp], acc[24 + pp]));
                const float t0 = __fadd_rn(y[0], y[4]), t1 = __fadd_rn(y[1], y[5]);
                const float t2 = __fadd_rn(y[2], y[6]), t3 = __fadd_rn(y[3], y[7]);
                s = __fadd_rn(__fadd_rn(t0, t1), __fadd_rn(t2, t3));
                s = __fmul_rn(s, scale);
                s = __fadd_rn(s, mv);
            }
        }
        // running maximum met by each key: earlier chunks (m_carry), warp 2's keys for warp 3, earlier lanes of the own warp
        float pm = s;                      // -inf for skipped keys and beyond the end
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float tt = __shfl_up_sync(0xffffffffu, pm, o);
            if (lane >= o) pm = fmaxf(pm, tt);
        }
        float ex = __shfl_up_sync(0xffffffffu, pm, 1);
        if (lane == 0) ex = -INFINITY;
        if (lane == 31) s_tot[warp - 2] = pm;
        asm volatile("bar.sync 1, 64;" ::: "memory");               // the two scorer warps only
        const float tot2 = s_tot[0], tot3 = s_tot[1];
        float m_before = fmaxf(m_carry, ex);
        if (warp == 3) m_before = fmaxf(m_before, tot2);
        if (j < kn) {
            if (skip)              { msv[ic] = 1.0f; sc[ic] = -0.0f; }                  // skipped: ms = 1, vs = -0
            else if (s > m_before) { msv[ic] = expf_glibc(__fadd_rn(m_before, -s), s_exp_tab); sc[ic] = 1.0f; evt[ic >> 3] = 1; }
            else                   { msv[ic] = 1.0f; sc[ic] = expf_glibc(__fadd_rn(s, -m_before), s_exp_tab); }
        }
        m_carry = fmaxf(m_carry, fmaxf(tot2, tot3));
    };

    // Copy groups (warp 1): P0 = {K0, V0}, P1 = {K1, V1, K2}, then group c = {V(c+2), K(c+3)} committed in iteration c.
    // A wait by warp 1 followed by the CTA barrier publishes the data to the other warps.
    if (warp == 1) {
        fetch_k(0); fetch_v(0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        fetch_k(1); fetch_v(1); fetch_k(2);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
    }
    __syncthreads();                       // K0 has landed; Qs, the table and the cleared flags are visible
    if (warp >= 2) score_chunk(0);

    float a0 = 0.0f, a1 = 0.0f, S = 0.0f;  // warp 0: dims 2*lane, 2*lane + 1
#ifdef FA_DEC_PROFILE
    long long p_wait = 0, p_work = 0, p_t0, p_t1, p_start = clock64();
    const bool p_me = blockIdx.x == 0 && blockIdx.y == 0 && lane == 0;
#endif
    for (int c = 0; c < n_chunks; ++c) {
        const int k0 = c * FA_DEC_CHUNK, kn = min(FA_DEC_CHUNK, n_kv - k0);
#ifdef FA_DEC_PROFILE
        p_t0 = clock64();
#endif
        if (warp == 1) {                   // V(c) and K(c+1) have landed when at most the newest group is pending (all for c == 0)
            if (c == 0) asm volatile("cp.async.wait_group 0;" ::: "memory");
            else        asm volatile("cp.async.wait_group 1;" ::: "memory");
        }
        __syncthreads();                   // scores of chunk c are written; chunk c-1 is consumed (its V stage and K(c)'s stage are free)
#ifdef FA_DEC_PROFILE
        p_t1 = clock64(); p_wait += p_t1 - p_t0;
#endif
        if (warp == 1) {
            fetch_v(c + 2); fetch_k(c + 3);
            asm volatile("cp.async.commit_group;" ::: "memory");
        } else if (warp >= 2) {
            if (c + 1 < n_chunks) score_chunk(c + 1);
        } else {
            const __half2 * vb = (const __half2 *) (Vs + (size_t) (c % 3) * FA_DEC_CHUNK * 64) + lane;      // key u: vb[u * 32]
            auto step = [&](float vs, float ms, float2 v, bool rescale) {
                if (__float_as_uint(vs) == 0x80000000u) { v.x = 0.0f; v.y = 0.0f; }      // skipped key: exact no-op whatever V holds
                if (rescale && ms != 1.0f) {
                    const float2 r = __half22float2(__floats2half2_rn(__fmul_rn(a0, ms), __fmul_rn(a1, ms)));
                    a0 = r.x; a1 = r.y;
                }
                const float2 t = __half22float2(__floats2half2_rn(__fmaf_rn(v.x, vs, a0), __fmaf_rn(v.y, vs, a1)));
                a0 = t.x; a1 = t.y;
                if (rescale) S = S_FMA ? __fmaf_rn(S, ms, vs) : __fadd_rn(__fmul_rn(S, ms), vs);
                else         S = __fadd_rn(S, vs);             // ms == 1: fma(S, 1, vs) and S*1 + vs are both S + vs
            };
            int i = 0;
            // a full chunk without a new maximum: one straight-line block of 64 dependent steps, so that the loads and
            // conversions of later keys are placed into the latency gaps of the two chains (a warp issues in order)
            if (kn == FA_DEC_CHUNK && *(const unsigned long long *) &evt[k0 >> 3] == 0ull) {
                // blocks of 16 steps: long enough to hide the loads, short enough to stay in the instruction cache
#pragma unroll 1
                for (int ub = 0; ub < FA_DEC_CHUNK; ub += 16) {
#pragma unroll
                    for (int u4 = 0; u4 < 4; ++u4) {
                        const float4 vs4 = *(const float4 *) &sc[k0 + ub + u4 * 4];
                        step(vs4.x, 1.0f, __half22float2(vb[(ub + u4 * 4 + 0) * 32]), false);
                        step(vs4.y, 1.0f, __half22float2(vb[(ub + u4 * 4 + 1) * 32]), false);
                        step(vs4.z, 1.0f, __half22float2(vb[(ub + u4 * 4 + 2) * 32]), false);
                        step(vs4.w, 1.0f, __half22float2(vb[(ub + u4 * 4 + 3) * 32]), false);
                    }
                }
                i = FA_DEC_CHUNK;
            }
            for (; i + 8 <= kn; i += 8) {  // a chunk with new maxima (or the last, short one): groups of eight keys
                float vs[8];
                float2 vv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) { vs[u] = sc[k0 + i + u]; vv[u] = __half22float2(vb[(i + u) * 32]); }
                if (!evt[(k0 + i) >> 3]) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) step(vs[u], 1.0f, vv[u], false);
                } else {
#pragma unroll
                    for (int u = 0; u < 8; ++u) step(vs[u], msv[k0 + i + u], vv[u], true);
                }
            }
            for (; i < kn; ++i) step(sc[k0 + i], msv[k0 + i], __half22float2(vb[i * 32]), true);
        }
#ifdef FA_DEC_PROFILE
        p_work += clock64() - p_t1;
#endif
    }
#ifdef FA_DEC_PROFILE
    if (p_me && warp < 3) { g_fa_prof[warp * 2] = p_wait; g_fa_prof[warp * 2 + 1] = p_work; if (warp == 0) g_fa_prof[6] = clock64() - p_start; }
#endif
    if (warp == 0) {
        const float S_inv = __fdiv_rn(1.0f, S);
        float2 o;
        o.x = __fmul_rn(a0, S_inv);
        o.y = __fmul_rn(a1, S_inv);
        *(float2 *) (R.dst + h * 64 + lane * 2) = o;
        if (xq != nullptr) {               // second output, as in the kernel above: lanes 0..15 hold block 2h, lanes 16..31 block 2h+1
            float amax = fmaxf(fabsf(o.x), fabsf(o.y));
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            const float id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
            const size_t kk = (size_t) gridDim.x * 64;
            char2 q;
            q.x = (signed char) __float2int_rn(__fmul_rn(o.x, id));
            q.y = (signed char) __float2int_rn(__fmul_rn(o.y, id));
            *(char2 *) (xq + blockIdx.y * kk + h * 64 + lane * 2) = q;
            if ((lane & 15) == 0) xd[blockIdx.y * (kk >> 5) + h * 2 + (lane >> 4)] = round_f16(__fdiv_rn(amax, 127.f));
        }
    }
}

static size_t fa_dec_smem(int max_kv, int stages) {
    return (size_t) ((64 + 2 * max_kv + (max_kv + 31) / 32 + 3) & ~3) * sizeof(float) + (size_t) stages * FA_DEC_CHUNK * 64 * sizeof(__half);
}

static bool g_fa_s_fma = true;

static int launch_fa_decode(const FaRows & rows, int n_rows, int64_t n_head, int8_t * xq, float * xd, cudaStream_t st) {
    int max_kv = 1;
    for (int i = 0; i < n_rows; ++i) max_kv = max(max_kv, rows.r[i].n_kv);
    max_kv = (max_kv + 7) & ~7;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(k_flash_attn_decode<true, 3>,  cudaFuncAttributeMaxDynamicSharedMemorySize, (int) fa_dec_smem(FA_DEC_MAX_KV, 3));
        cudaFuncSetAttribute(k_flash_attn_decode<false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) fa_dec_smem(FA_DEC_MAX_KV, 3));
        cudaFuncSetAttribute(k_flash_attn_decode_stream<true>,  cudaFuncAttributeMaxDynamicSharedMemorySize, (int) fa_dec_smem(FA_DEC_MAX_KV, 6));
        cudaFuncSetAttribute(k_flash_attn_decode_stream<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) fa_dec_smem(FA_DEC_MAX_KV, 6));
        attr_done[dev] = true;
    }
    dim3 grid((unsigned) n_head, (unsigned) n_rows);
    // the streaming kernel needs two rings (six chunk buffers): three CTAs per SM; larger launches keep to the small one
    static const bool no_stream = getenv("B200_FA_NO_STREAM") != nullptr;
    if (!no_stream && (int64_t) n_head * n_rows <= 3 * 148) {
        if (g_fa_s_fma) launch_chained(k_flash_attn_decode_stream<true>,  grid, dim3(FA_DEC_THREADS), fa_dec_smem(max_kv, 6), st, rows, max_kv, xq, xd);
        else            launch_chained(k_flash_attn_decode_stream<false>, grid, dim3(FA_DEC_THREADS), fa_dec_smem(max_kv, 6), st, rows, max_kv, xq, xd);
        B200_RETURN_LAST();
    }
    if (g_fa_s_fma) launch_chained(k_flash_attn_decode<true, 3>,  grid, dim3(FA_DEC_THREADS), fa_dec_smem(max_kv, 3), st, rows, max_kv, xq, xd);
    else            launch_chained(k_flash_attn_decode<false, 3>, grid, dim3(FA_DEC_THREADS), fa_dec_smem(max_kv, 3), st, rows, max_kv, xq, xd);
    B200_RETURN_LAST();
}

extern "C" int b200_flash_attn_decode_rows_q(const b200_fa_row * rows, int n_rows, int64_t n_head, int64_t nbq2, int64_t nbk1, int64_t nbk2,
                                             int64_t nbv1, int64_t nbv2, float scale, int8_t * xq, float * xd, void * stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > FA_DEC_MAX_ROWS || n_head <= 0 || n_head > 65535) return B200_ERR_ARG;
    if ((nbk1 & 15) || (nbk2 & 15) || (nbv1 & 15) || (nbv2 & 15) || (nbq2 & 3)) return B200_ERR_ARG;
    ensure_exp_table();
    FaRows r;
    memset(&r, 0, sizeof(r));
    r.nbq2 = nbq2; r.nbk1 = nbk1; r.nbk2 = nbk2; r.nbv1 = nbv1; r.nbv2 = nbv2; r.scale = scale;
    for (int i = 0; i < n_rows; ++i) {
        if (rows[i].n_kv <= 0 || rows[i].n_kv > FA_DEC_MAX_KV) return B200_ERR_ARG;
        if (((uintptr_t) rows[i].k & 15) || ((uintptr_t) rows[i].v & 15) || ((uintptr_t) rows[i].q & 3)) return B200_ERR_ARG;
        r.r[i].q = (const char *) rows[i].q; r.r[i].k = (const char *) rows[i].k; r.r[i].v = (const char *) rows[i].v;
        r.r[i].mask = (const char *) rows[i].mask; r.r[i].dst = rows[i].dst; r.r[i].n_kv = (int) rows[i].n_kv;
    }
    return launch_fa_decode(r, n_rows, n_head, xq, xd, as_stream(stream));
}

extern "C" int b200_flash_attn_decode_rows(const b200_fa_row * rows, int n_rows, int64_t n_head, int64_t nbq2, int64_t nbk1, int64_t nbk2,
                                           int64_t nbv1, int64_t nbv2, float scale, void * stream) {
    return b200_flash_attn_decode_rows_q(rows, n_rows, n_head, nbq2, nbk1, nbk2, nbv1, nbv2, scale, nullptr, nullptr, stream);
}

// The host compiler of the reference contracts "S*ms + vs" into one FMA (GNU mode, -mfma).
extern "C" void b200_set_fa_sum_fma(int on) { g_fa_s_fma = on != 0; }

extern "C" int b200_flash_attn_ext(const float * q, int64_t nbq1, int64_t nbq2,
                                   const void * k, int64_t nbk1, int64_t nbk2,
                                   const void * v, int64_t nbv1, int64_t nbv2,
                                   const void * mask, int64_t nbm1,
                                   float * dst, int64_t n_q, int64_t n_kv, int64_t n_head, float scale, void * stream) {
    if (n_q <= 0 || n_head <= 0) return 0;
    if (n_kv <= 0 || n_head > 65535) return B200_ERR_ARG;
    if (((uintptr_t) k & 15) || (nbk1 & 15) || (nbk2 & 15) || ((uintptr_t) v & 3) || (nbv1 & 3) || (nbv2 & 3)) return B200_ERR_ARG;
    if (((uintptr_t) q & 3) || (nbq1 & 3) || (nbq2 & 3) || ((uintptr_t) dst & 7)) return B200_ERR_ARG;
    ensure_exp_table();
    if (n_q <= FA_DEC_MAX_ROWS && n_kv <= FA_DEC_MAX_KV && !((uintptr_t) v & 15) && !(nbv1 & 15) && !(nbv2 & 15)) {
        FaRows r;
        memset(&r, 0, sizeof(r));
        r.nbq2 = nbq2; r.nbk1 = nbk1; r.nbk2 = nbk2; r.nbv1 = nbv1; r.nbv2 = nbv2; r.scale = scale;
        for (int i = 0; i < (int) n_q; ++i) {
            r.r[i].q = (const char *) q + i * nbq1; r.r[i].k = (const char *) k; r.r[i].v = (const char *) v;
            r.r[i].mask = mask ? (const char *) mask + i * nbm1 : nullptr;
            r.r[i].dst = dst + (int64_t) i * n_head * 64; r.r[i].n_kv = (int) n_kv;
        }
        return launch_fa_decode(r, (int) n_q, n_head, nullptr, nullptr, as_stream(stream));
    }
    dim3 grid((unsigned) ((n_q + 4 * FA_R - 1) / (4 * FA_R)), (unsigned) n_head);
    const bool has_skip = mask != nullptr || (n_kv % 32) != 0;
    static const bool relaxed = getenv("GGML_B200_RELAXED") != nullptr && atoi(getenv("GGML_B200_RELAXED")) != 0;
    static const bool mixed = getenv("B200_FA_MIXED") == nullptr || atoi(getenv("B200_FA_MIXED")) != 0;
#define FA_LAUNCH(SF, HS, RX) if (mixed) k_flash_attn_ext<SF, HS, RX, true><<<grid, 128, 0, as_stream(stream)>>>((const char *) q, nbq1, nbq2, (const char *) k, nbk1, nbk2, \
            (const char *) v, nbv1, nbv2, (const char *) mask, nbm1, dst, n_q, n_kv, n_head, scale); \
        else k_flash_attn_ext<SF, HS, RX, false><<<grid, 128, 0, as_stream(stream)>>>((const char *) q, nbq1, nbq2, (const char *) k, nbk1, nbk2, \
            (const char *) v, nbv1, nbv2, (const char *) mask, nbm1, dst, n_q, n_kv, n_head, scale)
    if (relaxed)         { if (has_skip) FA_LAUNCH(true, true, true); else FA_LAUNCH(true, false, true); }
    else if (g_fa_s_fma) { if (has_skip) FA_LAUNCH(true, true, false); else FA_LAUNCH(true, false, false); }
    else                 { if (has_skip) FA_LAUNCH(false, true, false); else FA_LAUNCH(false, false, false); }
#undef FA_LAUNCH
    B200_RETURN_LAST();
}

// ---- soft_max -------------------------------------------------------------------------------
__device__ __forceinline__ float v_expf_avx2(float x) {     // vec.h:603-640, one element
    const float r = 0x1.8p23f;
    const float z = __fmaf_rn(x, 0x1.715476p+0f, r);
    const float n = __fadd_rn(z, -r);
    const float b = __fmaf_rn(-n, 0x1.7f7d1cp-20f, __fmaf_rn(-n, 0x1.62e4p-1f, x));
    const uint32_t e = __float_as_uint(z) << 23;
    const float kf = __uint_as_float(e + 0x3f800000u);
    const bool  c = fabsf(n) > 126.0f;
    const float u = __fmul_rn(b, b);
    const float j = __fmaf_rn(__fmaf_rn(__fmaf_rn(0x1.0e4020p-7f, b, 0x1.573e2ep-5f), u,
                                        __fmaf_rn(0x1.555e66p-3f, b, 0x1.fffdb6p-2f)),
                              u, __fmul_rn(0x1.ffffecp-1f, b));
    if (!c) return __fmaf_rn(j, kf, kf);
    const uint32_t g = (n <= 0.0f) ? 0x82000000u : 0u;
    const float s1 = __uint_as_float(g + 0x7f000000u);
    const float s2 = __uint_as_float(e - g);
    if (fabsf(n) > 192.0f) return __fmul_rn(s1, s1);
    return __fmul_rn(__fmaf_rn(s2, j, s2), s1);
}

// one warp per row; mask row = (row % ne01), f16 or f32
__global__ void __launch_bounds__(128)
k_soft_max(const float * __restrict__ x, const char * __restrict__ mask, int mask_f16, int64_t mask_nb1,
           float * __restrict__ y, int64_t ne00, int64_t nrows, int64_t ne01, float scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t) blockIdx.x * 4 + warp;
    if (row >= nrows) return;
    const float * sp = x + row * ne00;
    float *       dp = y + row * ne00;
    const char *  mp = mask ? mask + (row % ne01) * mask_nb1 : nullptr;

    float mx = -INFINITY;
    for (int64_t i = lane; i < ne00; i += 32) {
        float w = __fmul_rn(sp[i], scale);
        if (mp) w = __fadd_rn(w, mask_f16 ? __half2float(((const __half *) mp)[i]) : ((const float *) mp)[i]);
        dp[i] = w;
        mx = fmaxf(mx, w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __syncwarp();

    // groups of 8 elements: lanes 8g'..8g'+7 handle one group; 4 groups per pass, in order
    const int64_t n8 = ne00 & ~(int64_t) 7;
    const int sub = lane >> 3, l8 = lane & 7;
    double sum = 0.0;    // exact replay needs group order: accumulate in lane 0 of the warp
    for (int64_t base = 0; base < n8; base += 32) {
        const int64_t i = base + sub * 8 + l8;
        float val = 0.0f;
        if (i < n8) { val = v_expf_avx2(__fadd_rn(dp[i], -mx)); dp[i] = val; }
        float t = __fadd_rn(val, __shfl_xor_sync(0xffffffffu, val, 4));
        t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));
        t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 1));
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const float tg = __shfl_sync(0xffffffffu, t, g * 8);
            if (base + g * 8 < n8) sum += (double) tg;
        }
    }
    for (int64_t i = n8; i < ne00; ++i) {       // scalar tail uses libm expf
        float val = 0.0f;
        if (lane == 0) { val = expf_glibc(__fadd_rn(dp[i], -mx), c_exp2f_tab); dp[i] = val; }
        val = __shfl_sync(0xffffffffu, val, 0);
        sum += (double) val;
    }
    __syncwarp();
    const float inv = (float) (1.0 / sum);
    for (int64_t i = lane; i < ne00; i += 32) dp[i] = __fmul_rn(dp[i], inv);
}

extern "C" int b200_soft_max(const float * x, const void * mask, int mask_type, int64_t mask_nb1, int64_t mask_ne1,
                             float * y, int64_t ne00, int64_t nrows, int64_t ne01, float scale, void * stream) {
    (void) mask_ne1;
    if (nrows <= 0 || ne00 <= 0) return 0;
    if (mask && mask_type != B200_TYPE_F16 && mask_type != B200_TYPE_F32) return B200_ERR_ARG;
    ensure_exp_table();
    k_soft_max<<<(unsigned) ((nrows + 3) / 4), 128, 0, as_stream(stream)>>>(x, (const char *) mask, mask_type == B200_TYPE_F16,
                                                                            mask_nb1, y, ne00, nrows, ne01, scale);
    B200_RETURN_LAST();
}
