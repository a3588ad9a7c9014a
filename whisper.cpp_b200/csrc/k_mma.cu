// Q5_0 / Q8_0 x Q8_0 matrix product for many columns (encoder, cross-attention K/V) on the tensor pipe,
// bit-identical to the reference CPU path (ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_q8_0_q8_0, AVX2 variant,
// ggml/src/ggml-cpu/ggml-cpu-quants.c:3076-3100, 3869-3886).
//
// What the reference computes per output and 32-block: eight lane sums q_j (exact integers, elements 4j..4j+3),
// then acc_j = fma(d_w*d_x, float(q_j), acc_j) block after block, hsum_float_8 at the end.  Only the float chain is
// order-bound; the integer lane sums may be formed in any way that keeps them apart.  Here they come from
// mma.m16n8k8 (f16 inputs, f32 accumulate): weights and quantised activations are small integers, exact in f16,
// their products and four-term sums exact in the f32 accumulator, so the MMA returns float(q_j) directly.
// Lanes are kept apart by zero-expanding the weight operand: MMA r of four has lane 2r of eight weight rows in
// A-rows 0..7 (non-zero for k = 0..3) and lane 2r+1 in A-rows 8..15 (k = 4..7); B holds block elements 8r..8r+7 of
// eight columns.  Thread (g, t) then owns, for weight row g, all eight lanes of columns 2t and 2t+1 as register
// pairs: d = d_w * (d_x[2t], d_x[2t+1]) once per block and eight packed fma.f32x2 per four MMAs.
//
// Operand formats (device memory, made by b200_mma_pack_weights / b200_mma_quantize):
//   h[nblocks][16] u32: the block's 32 integers as f16 pairs; pair 4r+t (elements 8r+2t, 8r+2t+1) is stored at
//   position 4t+r, so that one 16-byte shared load gives thread t its pairs of all four MMAs;  d[nblocks] f32 scale.
#include "b200_common.cuh"
#include <string.h>
#include <stdlib.h>

typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void upk2(f32x2 v, float & lo, float & hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }

__device__ __forceinline__ void hmma_lane_sums(f32x2 & q01, f32x2 & q23, uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("{\n\t.reg .f32 d0, d1, d2, d3;\n\t"
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {d0, d1, d2, d3}, {%2, %3}, {%4}, {%5, %5, %5, %5};\n\t"
        "mov.b64 %0, {d0, d1};\n\t"
        "mov.b64 %1, {d2, d3};\n\t}"
        : "=l"(q01), "=l"(q23) : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

__device__ __forceinline__ void cp_async16(unsigned dst, const void * src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(unsigned dst, const void * src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// ---- operand packing ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f16_pair(int lo, int hi) {
    const __half2 h = __halves2half2(__int2half_rn(lo), __int2half_rn(hi));
    return *(const uint32_t *) &h;
}

// one thread per (block, pair): weights of planes -> packed f16 integers + f32 scale
__global__ void k_mma_pack_weights(int type, QPlanes p, int64_t nb, uint32_t * __restrict__ h, float * __restrict__ d) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nb * 16) return;
    const int64_t blk = i >> 4;
    const int pos = (int) (i & 15), t = pos >> 2, r = pos & 3;
    const int e0 = 8 * r + 2 * t;                          // elements e0, e0 + 1
    int v0, v1;
    if (type == B200_TYPE_Q5_0) {
        const uint8_t * qs = p.qs + blk * 16;
        const uint32_t qh = p.qh[blk];
        // element j < 16: low nibble of qs[j] and bit j of qh; element j >= 16: high nibble of qs[j-16], bit j
        const int j0 = e0 & 15, sh = (e0 >> 4) * 4;
        v0 = (int) (((qs[j0]     >> sh) & 0xF) | (((qh >> e0)       & 1u) << 4)) - 16;
        v1 = (int) (((qs[j0 + 1] >> sh) & 0xF) | (((qh >> (e0 + 1)) & 1u) << 4)) - 16;
    } else {
        const int8_t * qs = (const int8_t *) p.qs + blk * 32;
        v0 = qs[e0]; v1 = qs[e0 + 1];
    }
    h[i] = f16_pair(v0, v1);
    if (pos == 0) d[blk] = __half2float(p.d[blk]);
}

extern "C" int b200_mma_pack_weights(int wtype, const void * w_planes, int64_t nb_total, void * h, float * d, void * stream) {
    if (wtype != B200_TYPE_Q5_0 && wtype != B200_TYPE_Q8_0) return B200_ERR_ARG;
    if (nb_total <= 0) return 0;
    if (((uintptr_t) h & 15) != 0 || ((uintptr_t) d & 15) != 0) return B200_ERR_ARG;
    const QPlanes p = q_planes(wtype, w_planes, nb_total);
    const int64_t n = nb_total * 16;
    k_mma_pack_weights<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>(wtype, p, nb_total, (uint32_t *) h, d);
    B200_RETURN_LAST();
}

// quantize_row_q8_0 (AVX2 variant, ggml-cpu-quants.c:808-866) with the integers written as packed f16 pairs:
// a warp per 32-block, lane = element
__global__ void k_mma_quantize(const float * x, int64_t n_rows, int64_t nbk, int64_t row_stride, uint32_t * __restrict__ h, float * __restrict__ d) {
    const int     lane = threadIdx.x & 31;
    const int64_t blk  = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= n_rows * nbk) return;
    const int64_t row = blk / nbk, ib = blk - row * nbk;
    const float v = *(const float *) ((const char *) x + row * row_stride + (ib * 32 + lane) * 4);
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float dd = __fdiv_rn(amax, 127.f);
    const float id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
    const int q  = __float2int_rn(__fmul_rn(v, id));
    const int qn = __shfl_down_sync(0xffffffffu, q, 1);
    if ((lane & 1) == 0) {
        const int pair = lane >> 1, r = pair >> 2, t = pair & 3;       // pair 4r + t -> position 4t + r
        h[blk * 16 + 4 * t + r] = f16_pair(q, qn);
    }
    if (lane == 0) d[blk] = round_f16(dd);
}

extern "C" int b200_mma_quantize(const float * x, int64_t n_rows, int64_t k, int64_t row_stride_bytes, void * h, float * d, void * stream) {
    if (k % 32 != 0) return B200_ERR_ARG;
    const int64_t nblk = n_rows * (k / 32);
    if (nblk <= 0) return 0;
    if (((uintptr_t) h & 15) != 0 || ((uintptr_t) d & 15) != 0) return B200_ERR_ARG;
    k_mma_quantize<<<(unsigned) ((nblk + 7) / 8), 256, 0, as_stream(stream)>>>(x, n_rows, k / 32, row_stride_bytes, (uint32_t *) h, d);
    B200_RETURN_LAST();
}

// ---- the product --------------------------------------------------------------------------------
struct MmaEp {
    int n_steps;
    int kind[4];
    const float * ptr[4];
    int64_t stride_n[4];
    float scalar[4];
    int store_f16;
    const uint16_t * gelu_table;
};

__device__ __forceinline__ float mma_ep_apply(const MmaEp & ep, int64_t n, int64_t m, float v) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        if (s < ep.n_steps) {
            if (ep.kind[s] == B200_EP_ADD)        v = __fadd_rn(v, ep.ptr[s][m + n * ep.stride_n[s]]);
            else if (ep.kind[s] == B200_EP_SCALE) v = __fmul_rn(v, ep.scalar[s]);
            else {
                if (v <= -10.0f)     v = 0.0f;
                else if (v < 10.0f)  v = __half2float(__ushort_as_half(ep.gelu_table[__half_as_ushort(__float2half_rn(v))]));
            }
        }
    }
    return v;
}

// CTA: WM x WN warps, warp tile 8G rows x 8T columns.  Default 4 x 3 warps of 16 x 24: 64 x 72 outputs, so that the
// 1500 columns of a 1280-row weight give 20 x 21 = 420 CTAs, a little under three full waves of one CTA per SM.
// Operands arrive by cp.async (16 bytes, zero fill beyond M / N), three stages of four 32-blocks.
#define MMA_KC 4
#define MMA_STAGES 3
template <int WM, int WN, int G, int T> struct MmaCfg {
    static constexpr int BM = WM * 8 * G, BN = WN * 8 * T, THREADS = WM * WN * 32;
    static constexpr int STAGE_BYTES = MMA_KC * BM * 64 + MMA_KC * BN * 64 + BM * MMA_KC * 4 + MMA_KC * BN * 4;
    static constexpr int SMEM_BYTES = MMA_STAGES * STAGE_BYTES;
};

template <int WM, int WN, int G, int T>
__global__ void __launch_bounds__(WM * WN * 32, 1)
k_mul_mat_mma(const uint32_t * __restrict__ wh, const float * __restrict__ wd, int64_t M, int nbk,
              const uint32_t * __restrict__ xh, const float * __restrict__ xd, int64_t N,
              void * __restrict__ dst, int64_t ldd, MmaEp ep) {
    typedef MmaCfg<WM, WN, G, T> Cfg;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, KC = MMA_KC, MMA_THREADS = Cfg::THREADS, MMA_STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int OFF_X = KC * BM * 64, OFF_DW = OFF_X + KC * BN * 64, OFF_DX = OFF_DW + BM * KC * 4;
    static_assert(BN * (BM + 1) * 4 <= MMA_STAGE_BYTES, "epilogue tile fits one stage");
    static_assert(BN * KC <= MMA_THREADS && BM <= MMA_THREADS, "one scale piece per thread");
    extern __shared__ __align__(16) unsigned char mma_smem[];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp % WM, wn = warp / WM;
    const int64_t m0 = (int64_t) blockIdx.x * BM;
    const int64_t n0 = (int64_t) blockIdx.y * BN;
    const unsigned smem_u = (unsigned) __cvta_generic_to_shared(mma_smem);

    // stage layout: Wh[KC][BM][16] u32 | Xh[KC][BN][16] u32 | dW[BM][KC] f32 | dX[KC][BN] f32
    // Every thread copies the same pieces in every chunk: source offsets (in 4-byte words, advanced by KC blocks per
    // chunk), destination offsets inside a stage and the byte counts (0 = zero fill beyond M / N) are formed once.
    constexpr int NW = (BM * 16 + MMA_THREADS - 1) / MMA_THREADS, NX = (BN * 16 + MMA_THREADS - 1) / MMA_THREADS;
    uint32_t w_src[NW], w_dst[NW], x_src[NX], x_dst[NX], dw_src = 0, dw_dst = 0, dx_src = 0, dx_dst = 0;
    int w_n[NW], x_n[NX], dw_n = -1, dx_n = -1;            // -1: this thread has no such piece
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const int idx = tid + i * MMA_THREADS, row = idx >> 4, piece = idx & 15, kb = piece >> 2, part = piece & 3;
        const bool ok = m0 + row < M;
        w_n[i]   = idx < BM * 16 ? (ok ? 16 : 0) : -1;
        w_src[i] = (uint32_t) ((ok ? m0 + row : 0) * nbk * 16 + piece * 4);
        w_dst[i] = ((kb * BM + row) * 16 + part * 4) * 4;
    }
#pragma unroll
    for (int i = 0; i < NX; ++i) {
        const int idx = tid + i * MMA_THREADS, col = idx >> 4, piece = idx & 15, kb = piece >> 2, part = piece & 3;
        const bool ok = n0 + col < N;
        x_n[i]   = idx < BN * 16 ? (ok ? 16 : 0) : -1;
        x_src[i] = (uint32_t) ((ok ? n0 + col : 0) * nbk * 16 + piece * 4);
        x_dst[i] = OFF_X + ((kb * BN + col) * 16 + part * 4) * 4;
    }
    if (tid < BM) {                                         // four scales of a row: 16 bytes
        const bool ok = m0 + tid < M;
        dw_n = ok ? 16 : 0; dw_src = (uint32_t) ((ok ? m0 + tid : 0) * nbk); dw_dst = OFF_DW + tid * KC * 4;
    }
    if (tid < BN * KC) {
        const int col = tid / KC, kb = tid % KC;
        const bool ok = n0 + col < N;
        dx_n = ok ? 4 : 0; dx_src = (uint32_t) ((ok ? n0 + col : 0) * nbk + kb); dx_dst = OFF_DX + (kb * BN + col) * 4;
    }
    auto issue = [&](int c) {
        const unsigned sb = smem_u + (unsigned) (c % MMA_STAGES) * MMA_STAGE_BYTES;
        const uint32_t adv = (uint32_t) c * KC;             // blocks
#pragma unroll
        for (int i = 0; i < NW; ++i) if (w_n[i] >= 0) cp_async16(sb + w_dst[i], wh + (w_src[i] + adv * 16), w_n[i]);
#pragma unroll
        for (int i = 0; i < NX; ++i) if (x_n[i] >= 0) cp_async16(sb + x_dst[i], xh + (x_src[i] + adv * 16), x_n[i]);
        if (dw_n >= 0) cp_async16(sb + dw_dst, wd + (dw_src + adv), dw_n);
        if (dx_n >= 0) cp_async4(sb + dx_dst, xd + (dx_src + adv), dx_n);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    f32x2 acc[G][T][8];                // [row group][column tile][lane] = (column 2t, column 2t + 1) of row g
#pragma unroll
    for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int ti = 0; ti < T; ++ti)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[gi][ti][j] = 0ull;

    const int n_chunks = nbk / KC;
    issue(0);
    if (n_chunks > 1) issue(1);
    const bool lo_half = t < 2;        // this thread's weight pairs sit in A-rows 0..7 (k = 0..3) or 8..15 (k = 4..7)

    for (int c = 0; c < n_chunks; ++c) {
        if (c + 1 < n_chunks) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else                  asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();               // chunk c visible to all; everybody is done with chunk c-1, whose stage chunk c+2 reuses
        if (c + 2 < n_chunks) issue(c + 2);
        const unsigned char * sb = mma_smem + (size_t) (c % MMA_STAGES) * MMA_STAGE_BYTES;
        const uint32_t * Ws = (const uint32_t *) sb;
        const uint32_t * Xs = (const uint32_t *) (sb + OFF_X);
        const float * dWs = (const float *) (sb + OFF_DW);
        const float * dXs = (const float *) (sb + OFF_DX);

#pragma unroll
        for (int kb = 0; kb < KC; ++kb) {
            uint32_t a0[G][4], a1[G][4];
            f32x2 dwp[G];
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const int row = wm * (8 * G) + gi * 8 + g;
                const uint4 wv = *(const uint4 *) &Ws[(kb * BM + row) * 16 + t * 4];
                const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int r = 0; r < 4; ++r) { a0[gi][r] = lo_half ? wr[r] : 0u; a1[gi][r] = lo_half ? 0u : wr[r]; }
                const float dw = dWs[row * KC + kb];
                dwp[gi] = pk2(dw, dw);
            }
#pragma unroll
            for (int ti = 0; ti < T; ++ti) {
                const int col = wn * (8 * T) + ti * 8;
                const uint4 xv = *(const uint4 *) &Xs[(kb * BN + col + g) * 16 + t * 4];
                const uint32_t xr[4] = {xv.x, xv.y, xv.z, xv.w};
                const f32x2 dxp = *(const f32x2 *) &dXs[kb * BN + col + 2 * t];
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const f32x2 d = mul2(dwp[gi], dxp);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        f32x2 q01, q23;
                        hmma_lane_sums(q01, q23, a0[gi][r], a1[gi][r], xr[r]);
                        acc[gi][ti][2 * r]     = fma2(d, q01, acc[gi][ti][2 * r]);
                        acc[gi][ti][2 * r + 1] = fma2(d, q23, acc[gi][ti][2 * r + 1]);
                    }
                }
            }
        }
    }
    __syncthreads();                   // all warps are done with the last stage before the output tile overwrites stage 0

    // hsum_float_8: (l0+l4, l1+l5, l2+l6, l3+l7) -> (+2) -> (+1), both columns at once
    float (*Cs)[BM + 1] = (float (*)[BM + 1]) mma_smem;
#pragma unroll
    for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int ti = 0; ti < T; ++ti) {
            const f32x2 * a = acc[gi][ti];
            const f32x2 r0 = add2(a[4], a[0]), r1 = add2(a[5], a[1]);
            const f32x2 r2 = add2(a[6], a[2]), r3 = add2(a[7], a[3]);
            const f32x2 s  = add2(add2(r0, r2), add2(r1, r3));
            float lo, hi;
            upk2(s, lo, hi);
            const int row = wm * (8 * G) + gi * 8 + g, col = wn * (8 * T) + ti * 8 + 2 * t;
            Cs[col][row]     = lo;
            Cs[col + 1][row] = hi;
        }
    __syncthreads();
    {   // epilogue with full-row global accesses
        const int ml = tid % BM;
        const int64_t m = m0 + ml;
        if (m < M) {
#pragma unroll 4
            for (int nl = tid / BM; nl < BN; nl += MMA_THREADS / BM) {
                const int64_t n = n0 + nl;
                if (n < N) {
                    const float v = mma_ep_apply(ep, n, m, Cs[nl][ml]);
                    if (ep.store_f16) ((__half *) dst)[n * ldd + m] = __float2half_rn(v);
                    else              ((float *) dst)[n * ldd + m] = v;
                }
            }
        }
    }
}

const uint16_t * b200_gelu_table_device(int * err);

template <int WM, int WN, int G, int T>
static int launch_mma(const void * wh, const float * wd, int64_t M, int64_t K, const void * xh, const float * xd, int64_t N,
                      void * dst, int64_t ldd, const MmaEp & e, cudaStream_t st) {
    typedef MmaCfg<WM, WN, G, T> Cfg;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t ce = cudaFuncSetAttribute(k_mul_mat_mma<WM, WN, G, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (ce != cudaSuccess) return (int) ce;
        attr_done[dev] = true;
    }
    dim3 grid((unsigned) ((M + Cfg::BM - 1) / Cfg::BM), (unsigned) ((N + Cfg::BN - 1) / Cfg::BN));
    k_mul_mat_mma<WM, WN, G, T><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>((const uint32_t *) wh, wd, M, (int) (K / 32),
                                                                              (const uint32_t *) xh, xd, N, dst, ldd, e);
    return 0;
}

extern "C" int b200_mul_mat_mma_ep(const void * wh, const float * wd, int64_t M, int64_t K,
                                   const void * xh, const float * xd, int64_t N,
                                   void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream) {
    if (K % (32 * MMA_KC) != 0 || K <= 0 || M <= 0 || N <= 0) return B200_ERR_ARG;
    if (((uintptr_t) wh & 15) || ((uintptr_t) xh & 15) || ((uintptr_t) wd & 15) || ((uintptr_t) xd & 3)) return B200_ERR_ARG;
    if (M * (K / 2) >= (int64_t) 1 << 32 || N * (K / 2) >= (int64_t) 1 << 32) return B200_ERR_ARG;     // 32-bit word offsets in the kernel
    MmaEp e;
    memset(&e, 0, sizeof(e));
    if (ep) {
        if (ep->n_steps < 0 || ep->n_steps > 4) return B200_ERR_ARG;
        e.n_steps = ep->n_steps; e.store_f16 = ep->store_f16;
        for (int s = 0; s < ep->n_steps; ++s) {
            e.kind[s] = ep->step[s].kind; e.ptr[s] = ep->step[s].ptr; e.stride_n[s] = ep->step[s].stride_n; e.scalar[s] = ep->step[s].scalar;
            if (e.kind[s] == B200_EP_GELU) {
                if (!e.gelu_table) { int err = 0; e.gelu_table = b200_gelu_table_device(&err); if (err) return err; }
            } else if (e.kind[s] == B200_EP_ADD) {
                if (!e.ptr[s]) return B200_ERR_ARG;
            } else if (e.kind[s] != B200_EP_SCALE) return B200_ERR_ARG;
        }
    }
    static const int cfg = getenv("B200_MMA_CFG") ? atoi(getenv("B200_MMA_CFG")) : 0;
    int rc;
    if (cfg == 1)      rc = launch_mma<4, 4, 2, 2>(wh, wd, M, K, xh, xd, N, dst, dst_stride, e, as_stream(stream));
    else if (cfg == 2) rc = launch_mma<2, 7, 2, 2>(wh, wd, M, K, xh, xd, N, dst, dst_stride, e, as_stream(stream));
    else               rc = launch_mma<4, 3, 2, 3>(wh, wd, M, K, xh, xd, N, dst, dst_stride, e, as_stream(stream));
    if (rc) return rc;
    B200_RETURN_LAST();
}
