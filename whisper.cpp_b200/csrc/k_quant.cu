// Block-quantised weights: plane layout, dequantise, Q8_0 activation quantisation and the
// Q5_0/Q8_0 x Q8_0 matrix products.  Every sum is formed in the order of the reference's AVX2
// kernels: eight partial sums ("lanes", four consecutive elements of a 32-block each) that are
// FMA-accumulated block after block and reduced at the end as hsum_float_8 does
// (ggml/src/ggml-cpu/ggml-cpu-quants.c:49-55, 3076-3100, 3869-3886).
#include "b200_common.cuh"
#include <string.h>
#include <stdlib.h>
#include <stdio.h>

std::atomic<int64_t> g_b200_launches{0};

extern "C" int64_t b200_launch_count(void) { return g_b200_launches.load(); }
bool b200_chained_launches(void) {
    static const bool on = getenv("B200_NO_PDL") == nullptr;
    return on;
}
extern "C" const char * b200_version(void) { return "b200-whisper 0.1 (sm_100a)"; }

// ------------------------------------------------------------------------------------------------
// host: ggml blocks <-> planes
// ------------------------------------------------------------------------------------------------
extern "C" int b200_blocks_to_planes(int type, const void * blocks, void * planes, int64_t nb_total,
                                     int64_t nb_first, int64_t nb_count) {
    const uint8_t * src = (const uint8_t *) blocks;   // nb_count blocks, starting at block nb_first
    uint8_t * dst = (uint8_t *) planes;               // the whole tensor's planes
    if (nb_first < 0 || nb_count < 0 || nb_first + nb_count > nb_total) return B200_ERR_ARG;
    if (type == B200_TYPE_Q5_0) {
        uint8_t * qs = dst, * qh = dst + 16 * nb_total, * d = dst + 20 * nb_total;
        for (int64_t i = 0; i < nb_count; ++i) {
            const uint8_t * b = src + 22 * i;
            const int64_t   o = nb_first + i;
            memcpy(d + 2 * o, b, 2);
            memcpy(qh + 4 * o, b + 2, 4);
            memcpy(qs + 16 * o, b + 6, 16);
        }
    } else if (type == B200_TYPE_Q8_0) {
        uint8_t * qs = dst, * d = dst + 32 * nb_total;
        for (int64_t i = 0; i < nb_count; ++i) {
            const uint8_t * b = src + 34 * i;
            const int64_t   o = nb_first + i;
            memcpy(d + 2 * o, b, 2);
            memcpy(qs + 32 * o, b + 2, 32);
        }
    } else {
        return B200_ERR_ARG;
    }
    return 0;
}

extern "C" int b200_planes_to_blocks(int type, const void * planes, void * blocks, int64_t nb_total,
                                     int64_t nb_first, int64_t nb_count) {
    const uint8_t * src = (const uint8_t *) planes;
    uint8_t * dst = (uint8_t *) blocks;
    if (nb_first < 0 || nb_count < 0 || nb_first + nb_count > nb_total) return B200_ERR_ARG;
    if (type == B200_TYPE_Q5_0) {
        const uint8_t * qs = src, * qh = src + 16 * nb_total, * d = src + 20 * nb_total;
        for (int64_t i = 0; i < nb_count; ++i) {
            uint8_t *     b = dst + 22 * i;
            const int64_t o = nb_first + i;
            memcpy(b, d + 2 * o, 2);
            memcpy(b + 2, qh + 4 * o, 4);
            memcpy(b + 6, qs + 16 * o, 16);
        }
    } else if (type == B200_TYPE_Q8_0) {
        const uint8_t * qs = src, * d = src + 32 * nb_total;
        for (int64_t i = 0; i < nb_count; ++i) {
            uint8_t *     b = dst + 34 * i;
            const int64_t o = nb_first + i;
            memcpy(b, d + 2 * o, 2);
            memcpy(b + 2, qs + 32 * o, 32);
        }
    } else {
        return B200_ERR_ARG;
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------
// device: ggml blocks (raw bytes as a model file holds them, 22 / 34 bytes each, unaligned) <-> planes.  One thread
// moves two bytes of a block, so the reads of a warp cover consecutive bytes of the block stream and the writes into
// each plane are contiguous runs; this is how the plugin stores a weight tensor in one upload plus one launch.
// ------------------------------------------------------------------------------------------------
template <bool TO_PLANES>
__global__ void k_blocks_planes(int type, uint8_t * __restrict__ blocks, uint8_t * __restrict__ planes, int64_t nb_total, int64_t nb_first, int64_t nb_count) {
    const int bs2 = type == B200_TYPE_Q5_0 ? 11 : 17;                   // byte pairs per block
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;  // pair index in the block stream
    if (i >= nb_count * bs2) return;
    const int64_t blk = i / bs2;
    const int     off = (int) (i - blk * bs2) * 2;                      // byte offset inside the block (even)
    const int64_t o = nb_first + blk;
    uint8_t * b = blocks + blk * (2 * bs2) + off;
    uint8_t * pl;
    if (type == B200_TYPE_Q5_0) {       // {f16 d; u8 qh[4]; u8 qs[16]}
        if (off < 2)      pl = planes + 20 * nb_total + 2 * o;
        else if (off < 6) pl = planes + 16 * nb_total + 4 * o + (off - 2);
        else              pl = planes + 16 * o + (off - 6);
    } else {                            // {f16 d; i8 qs[32]}
        if (off < 2) pl = planes + 32 * nb_total + 2 * o;
        else         pl = planes + 32 * o + (off - 2);
    }
    if (TO_PLANES) { pl[0] = b[0]; pl[1] = b[1]; }
    else           { b[0] = pl[0]; b[1] = pl[1]; }
}

extern "C" int b200_blocks_to_planes_device(int type, const void * blocks_dev, void * planes_dev, int64_t nb_total, int64_t nb_first,
                                            int64_t nb_count, void * stream) {
    if (type != B200_TYPE_Q5_0 && type != B200_TYPE_Q8_0) return B200_ERR_ARG;
    if (nb_first < 0 || nb_count < 0 || nb_first + nb_count > nb_total || !blocks_dev || !planes_dev) return B200_ERR_ARG;
    if (nb_count == 0) return 0;
    const int64_t n = nb_count * (type == B200_TYPE_Q5_0 ? 11 : 17);
    k_blocks_planes<true><<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>(type, (uint8_t *) blocks_dev, (uint8_t *) planes_dev, nb_total, nb_first, nb_count);
    B200_RETURN_LAST();
}

extern "C" int b200_planes_to_blocks_device(int type, const void * planes_dev, void * blocks_dev, int64_t nb_total, int64_t nb_first,
                                            int64_t nb_count, void * stream) {
    if (type != B200_TYPE_Q5_0 && type != B200_TYPE_Q8_0) return B200_ERR_ARG;
    if (nb_first < 0 || nb_count < 0 || nb_first + nb_count > nb_total || !blocks_dev || !planes_dev) return B200_ERR_ARG;
    if (nb_count == 0) return 0;
    const int64_t n = nb_count * (type == B200_TYPE_Q5_0 ? 11 : 17);
    k_blocks_planes<false><<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>(type, (uint8_t *) blocks_dev, (uint8_t *) planes_dev, nb_total, nb_first, nb_count);
    B200_RETURN_LAST();
}

// ------------------------------------------------------------------------------------------------
// dequantise (one thread per element)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float dequant_elem(int type, const QPlanes & p, int64_t blk, int e) {
    const float d = __half2float(p.d[blk]);
    if (type == B200_TYPE_Q5_0) {
        const uint8_t  b  = p.qs[blk * 16 + (e & 15)];
        const uint32_t qh = p.qh[blk];
        const int nib = (e < 16) ? (b & 0x0F) : (b >> 4);
        const int hi  = (int) ((qh >> e) & 1u) << 4;
        return (float) ((nib | hi) - 16) * d;     // x0*d with x0 converted int -> float
    } else {
        return (float) ((const int8_t *) p.qs)[blk * 32 + e] * d;
    }
}

__global__ void k_dequantize(int type, QPlanes p, int64_t nb_first, int64_t n_elem, float * out) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elem) return;
    out[i] = dequant_elem(type, p, nb_first + (i >> 5), (int) (i & 31));
}

extern "C" int b200_dequantize(int type, const void * planes, int64_t nb_total, int64_t nb_first, int64_t nb_count,
                               float * out, void * stream) {
    if (type != B200_TYPE_Q5_0 && type != B200_TYPE_Q8_0) return B200_ERR_ARG;
    if (nb_count <= 0) return 0;
    const int64_t n = nb_count * 32;
    k_dequantize<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>(type, q_planes(type, planes, nb_total), nb_first, n, out);
    B200_RETURN_LAST();
}

// GET_ROWS from a quantised table: one thread per output element
__global__ void k_get_rows_q(int type, QPlanes p, int64_t ne00, const int32_t * ids, int64_t n_ids, float * dst) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ne00 * n_ids) return;
    const int64_t r = i / ne00, c = i - r * ne00;
    const int64_t blk = (int64_t) ids[r] * (ne00 >> 5) + (c >> 5);
    dst[i] = dequant_elem(type, p, blk, (int) (c & 31));
}

int b200_get_rows_q_launch(int type, const void * table, int64_t nb_total, int64_t ne00, const int32_t * ids,
                           int64_t n_ids, float * dst, cudaStream_t st) {
    const int64_t n = ne00 * n_ids;
    if (n <= 0) return 0;
    k_get_rows_q<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(type, q_planes(type, table, nb_total), ne00, ids, n_ids, dst);
    B200_RETURN_LAST();
}

// ------------------------------------------------------------------------------------------------
// activation quantisation: one warp per 32-block
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void quantize_block_q8_0(float v, int lane, int8_t & q, float & d_out) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d  = __fdiv_rn(amax, 127.f);
    const float id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
    q = (int8_t) __float2int_rn(__fmul_rn(v, id));
    d_out = round_f16(d);
    (void) lane;
}

__global__ void k_quantize_q8_0(const float * x, int64_t n_rows, int64_t nbk, int64_t row_stride, int8_t * qs, float * d) {
    const int     lane = threadIdx.x & 31;
    const int64_t blk  = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= n_rows * nbk) return;
    const int64_t r = blk / nbk, ib = blk - r * nbk;
    const float v = *(const float *) ((const char *) x + r * row_stride + (ib * 32 + lane) * 4);
    int8_t q; float dd;
    quantize_block_q8_0(v, lane, q, dd);
    qs[blk * 32 + lane] = q;
    if (lane == 0) d[blk] = dd;
}

extern "C" int b200_quantize_q8_0(const float * x, int64_t n_rows, int64_t k, int64_t row_stride_bytes,
                                  int8_t * qs, float * d, void * stream) {
    if (k % 32 != 0) return B200_ERR_ARG;
    const int64_t nblk = n_rows * (k / 32);
    if (nblk <= 0) return 0;
    k_quantize_q8_0<<<(unsigned) ((nblk + 7) / 8), 256, 0, as_stream(stream)>>>(x, n_rows, k / 32, row_stride_bytes, qs, d);
    B200_RETURN_LAST();
}

// ------------------------------------------------------------------------------------------------
// GEMM: 64 x 32 output tile per CTA, 256 threads = 32 groups x 8 lanes; a thread owns lane j of an
// 8 x 8 block of outputs.  Per 32-block: q = dp4a(w, x) (exact), acc = fma(dw*dx, q, acc).
// ------------------------------------------------------------------------------------------------
#define MAGIC_I 0x4B400000          // bits of 12582912.0f: integer adds to it stay exact floats
#define MAGIC_F 12582912.0f

struct GemmEp {
    int n_steps;
    int kind[4];
    const float * ptr[4];
    int64_t stride_n[4];
    float scalar[4];
    int store_f16;
    const uint16_t * gelu_table;
};

__device__ __forceinline__ float gemm_ep_apply(const GemmEp & ep, int64_t n, int64_t m, float v) {
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

// packed single-precision pairs (sm_100 fma/add/mul .f32x2): two independent IEEE operations per instruction
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pack2i(int lo, int hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float & lo, float & hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// 32 x 32 output tile per CTA, 256 threads, a thread owns a 2 x 2 block of outputs with all eight lane sums of each
// (32 running sums as 16 register pairs), so the block scale d_w*d_x is formed once per output and the lane updates
// go two at a time through the packed f32x2 pipe.  Per 32-block and output: q_j = dp4a (exact), acc_j = fma(d, q_j, acc_j).
template <int TYPE>
__global__ void __launch_bounds__(256, 2)
k_mul_mat_q(QPlanes w, int64_t M, int64_t nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd,
            int64_t N, void * __restrict__ dst, int64_t ldd, GemmEp ep) {
    constexpr int BM = 32, BN = 32, KC = 4, WSTR = 8, XSTR = 12;       // words per staged row / column (X padded: conflict-free LDS.128)
    __shared__ __align__(16) int   Ws[KC][BM][WSTR];
    __shared__ __align__(16) int   Xs[KC][BN][XSTR];
    __shared__ __align__(16) float dWs[KC][BM];
    __shared__ __align__(16) float dXs[KC][BN];
    __shared__ float Cs[BN][BM + 1];

    const int tid = threadIdx.x;
    const int tx  = tid & 15;          // columns tx and tx + 16
    const int ty  = tid >> 4;          // rows 2*ty, 2*ty + 1
    const int64_t m0 = (int64_t) blockIdx.x * BM;
    const int64_t n0 = (int64_t) blockIdx.y * BN;

    f32x2 acc[2][8];                   // [row][lane] = (column tx, column tx + 16)
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) acc[r][jj] = 0ull;

    // staging roles: threads 0..127 fetch one (row, block) of W, threads 128..255 one (column, block) of X
    const int srow = tid & 31, skb = (tid >> 5) & 3;
    const bool is_w = tid < 128;
    uint4 pa = make_uint4(0, 0, 0, 0), pb = make_uint4(0, 0, 0, 0);
    uint32_t pqh = 0;
    float pd = 0.0f;
    auto fetch = [&](int64_t kb0) {
        pa = make_uint4(0, 0, 0, 0); pb = pa; pqh = 0; pd = 0.0f;
        const int64_t ib = kb0 + skb;
        if (is_w) {
            const int64_t m = m0 + srow;
            if (m < M && ib < nbk) {
                const int64_t blk = m * nbk + ib;
                if (TYPE == B200_TYPE_Q5_0) { pa = ((const uint4 *) w.qs)[blk]; pqh = w.qh[blk]; }
                else { pa = ((const uint4 *) w.qs)[blk * 2]; pb = ((const uint4 *) w.qs)[blk * 2 + 1]; }
                pd = __half2float(w.d[blk]);
            }
        } else {
            const int64_t n = n0 + srow;
            if (n < N && ib < nbk) {
                const uint4 * p = (const uint4 *) (xq + (n * nbk + ib) * 32);
                pa = p[0]; pb = p[1];
                pd = xd[n * nbk + ib];
            }
        }
    };
    fetch(0);

    const f32x2 neg_magic = pack2(-MAGIC_F, -MAGIC_F);
    for (int64_t kb0 = 0; kb0 < nbk; kb0 += KC) {
        if (is_w) {
            int wv[8];
            if (TYPE == B200_TYPE_Q5_0) {
                const uint32_t qw[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
                for (int t = 0; t < 8; ++t) wv[t] = q5_lane_word(qw[t & 3], pqh, t);
            } else {
                wv[0] = pa.x; wv[1] = pa.y; wv[2] = pa.z; wv[3] = pa.w;
                wv[4] = pb.x; wv[5] = pb.y; wv[6] = pb.z; wv[7] = pb.w;
            }
            *(int4 *) &Ws[skb][srow][0] = make_int4(wv[0], wv[1], wv[2], wv[3]);
            *(int4 *) &Ws[skb][srow][4] = make_int4(wv[4], wv[5], wv[6], wv[7]);
            dWs[skb][srow] = pd;
        } else {
            *(uint4 *) &Xs[skb][srow][0] = pa;
            *(uint4 *) &Xs[skb][srow][4] = pb;
            dXs[skb][srow] = pd;
        }
        __syncthreads();
        if (kb0 + KC < nbk) fetch(kb0 + KC);

#pragma unroll 2
        for (int kb = 0; kb < KC; ++kb) {
            int w0[8], w1[8], x0[8], x1[8];
            *(int4 *) &w0[0] = *(const int4 *) &Ws[kb][2 * ty][0];
            *(int4 *) &w0[4] = *(const int4 *) &Ws[kb][2 * ty][4];
            *(int4 *) &w1[0] = *(const int4 *) &Ws[kb][2 * ty + 1][0];
            *(int4 *) &w1[4] = *(const int4 *) &Ws[kb][2 * ty + 1][4];
            *(int4 *) &x0[0] = *(const int4 *) &Xs[kb][tx][0];
            *(int4 *) &x0[4] = *(const int4 *) &Xs[kb][tx][4];
            *(int4 *) &x1[0] = *(const int4 *) &Xs[kb][tx + 16][0];
            *(int4 *) &x1[4] = *(const int4 *) &Xs[kb][tx + 16][4];
            const float dw0 = dWs[kb][2 * ty], dw1 = dWs[kb][2 * ty + 1];
            const f32x2 dx = pack2(dXs[kb][tx], dXs[kb][tx + 16]);
            const f32x2 d0 = mul2(pack2(dw0, dw0), dx);
            const f32x2 d1 = mul2(pack2(dw1, dw1), dx);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const f32x2 q0 = add2(pack2i(__dp4a(w0[jj], x0[jj], MAGIC_I), __dp4a(w0[jj], x1[jj], MAGIC_I)), neg_magic);
                const f32x2 q1 = add2(pack2i(__dp4a(w1[jj], x0[jj], MAGIC_I), __dp4a(w1[jj], x1[jj], MAGIC_I)), neg_magic);
                acc[0][jj] = fma2(d0, q0, acc[0][jj]);
                acc[1][jj] = fma2(d1, q1, acc[1][jj]);
            }
        }
        __syncthreads();
    }

    // hsum_float_8: (l0+l4, l1+l5, l2+l6, l3+l7) -> (+2) -> (+1), both columns at once
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const f32x2 r0 = add2(acc[r][4], acc[r][0]), r1 = add2(acc[r][5], acc[r][1]);
        const f32x2 r2 = add2(acc[r][6], acc[r][2]), r3 = add2(acc[r][7], acc[r][3]);
        const f32x2 s  = add2(add2(r0, r2), add2(r1, r3));
        float lo, hi;
        unpack2(s, lo, hi);
        Cs[tx][2 * ty + r]      = lo;
        Cs[tx + 16][2 * ty + r] = hi;
    }
    __syncthreads();
    {   // epilogue with full-row global accesses
        const int ml = tid & 31;
        const int64_t m = m0 + ml;
        if (m < M) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int nl = (tid >> 5) + 8 * i;
                const int64_t n = n0 + nl;
                if (n < N) {
                    const float v = gemm_ep_apply(ep, n, m, Cs[nl][ml]);
                    if (ep.store_f16) ((__half *) dst)[n * ldd + m] = __float2half_rn(v);
                    else              ((float *) dst)[n * ldd + m] = v;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// GEMM on the tensor pipe, still bit-exact.  The eight lane sums of a (weight row, column, 32-block) are exact
// integers, so ANY summation order gives them; only the float chain acc_j = fma(d, q_j, acc_j) is order-bound.
// An int8 MMA (m16n8k32) is made to deliver separate lane sums by zero-expanding the weight operand: MMA r of four
// carries, for the eight weight rows of a group, lane 2r in A-rows 0..7 and lane 2r+1 in A-rows 8..15, each
// non-zero only in the four K-slots that hold that lane's activations.  K-slots are permuted (low half slot s =
// lane 2s, high half slot s = lane 2s+1), which makes the plain activation fragment one 8-byte shared load and the
// weight fragment of thread (g, t) the quad {word 2t, 0, 0, word 2t+1} of row g in MMA r == t and zero otherwise.
// The quads are laid out ready-made in shared memory (with one zero quad per row record), so a fragment is one
// 16-byte load from an address chosen once per thread.  After the four MMAs thread (g, t) holds all eight lane sums
// of outputs (row g, columns 2t and 2t+1) as register pairs: the block scale d_w*d_x is formed once per output pair
// and the chain runs on packed f32x2 operations.  The accumulator input of the MMA is the magic integer, so its
// result is already the bit pattern of 12582912 + q.
// Warp tile: 8G rows x 8T columns; CTA: 4 x 2 warps.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_lane_sums(f32x2 & q01, f32x2 & q23, const uint4 & a, const uint2 & b, const int4 & c) {
    asm("{\n\t.reg .b32 d0, d1, d2, d3;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {d0, d1, d2, d3}, {%2, %3, %4, %5}, {%6, %7}, {%8, %9, %10, %11};\n\t"
        "mov.b64 %0, {d0, d1};\n\t"
        "mov.b64 %1, {d2, d3};\n\t}"
        : "=l"(q01), "=l"(q23) : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w));
}

template <int TYPE, int G, int T>
__global__ void __launch_bounds__(256, (G * T <= 4) ? 2 : 1)
k_mul_mat_q_mma(QPlanes w, int64_t M, int64_t nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd,
                int64_t N, void * __restrict__ dst, int64_t ldd, GemmEp ep) {
    constexpr int WM = 4, WN = 2, KC = 4;
    constexpr int BM = WM * 8 * G, BN = WN * 8 * T;
    constexpr int WREC = 80;                                        // bytes per (row, block): four fragment quads + a zero quad
    static_assert(BM * KC <= 256 && BN * KC <= 256, "one staged item per thread");
    constexpr int OFF_X = KC * BM * WREC, OFF_DW = OFF_X + KC * BN * 32, OFF_DX = OFF_DW + KC * BM * 8, OFF_MAGIC = OFF_DX + KC * BN * 4;
    constexpr int STAGE_BYTES = OFF_MAGIC + 16;
    constexpr int CS_BYTES = BN * (BM + 1) * 4;
    __shared__ __align__(16) unsigned char smem_raw[STAGE_BYTES > CS_BYTES ? STAGE_BYTES : CS_BYTES];
    unsigned char * Wq = smem_raw;                                  // [KC][BM][WREC]
    int    (*Xs)[BN][8] = (int (*)[BN][8]) (smem_raw + OFF_X);
    float2 (*dWs)[BM]   = (float2 (*)[BM]) (smem_raw + OFF_DW);     // (d, d)
    float  (*dXs)[BN]   = (float (*)[BN]) (smem_raw + OFF_DX);
    float  (*Cs)[BM + 1] = (float (*)[BM + 1]) smem_raw;           // after the main loop

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;
    const int64_t m0 = (int64_t) blockIdx.x * BM;
    const int64_t n0 = (int64_t) blockIdx.y * BN;

    f32x2 acc[G][T][8];                // [row group][column tile][lane] = (column 2t, column 2t + 1) of row g
#pragma unroll
    for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int ti = 0; ti < T; ++ti)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[gi][ti][j] = 0ull;

    // staging: thread i fetches (row i % BM, block i / BM) of W and (column i % BN, block i / BN) of X
    const int wrow = tid % BM, wkb = tid / BM;
    const int xcol = tid % BN, xkb = tid / BN;
    const bool has_w = tid < BM * KC, has_x = tid < BN * KC;
    if (has_w) *(uint4 *) (Wq + (wkb * BM + wrow) * WREC + 64) = make_uint4(0, 0, 0, 0);       // the record's zero quad, written once
    if (tid == 0) *(int4 *) (smem_raw + OFF_MAGIC) = make_int4(MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I);
    uint4 wa = make_uint4(0, 0, 0, 0), wb = wa, xa = wa, xb = wa;
    uint32_t wqh = 0;
    float wd = 0.0f, xdv = 0.0f;
    auto fetch = [&](int64_t kb0) {
        wa = make_uint4(0, 0, 0, 0); wb = wa; xa = wa; xb = wa; wqh = 0; wd = 0.0f; xdv = 0.0f;
        if (has_w) {
            const int64_t m = m0 + wrow, ib = kb0 + wkb;
            if (m < M && ib < nbk) {
                const int64_t blk = m * nbk + ib;
                if (TYPE == B200_TYPE_Q5_0) { wa = ((const uint4 *) w.qs)[blk]; wqh = w.qh[blk]; }
                else { wa = ((const uint4 *) w.qs)[blk * 2]; wb = ((const uint4 *) w.qs)[blk * 2 + 1]; }
                wd = __half2float(w.d[blk]);
            }
        }
        if (has_x) {
            const int64_t n = n0 + xcol, ib = kb0 + xkb;
            if (n < N && ib < nbk) {
                const uint4 * p = (const uint4 *) (xq + (n * nbk + ib) * 32);
                xa = p[0]; xb = p[1];
                xdv = xd[n * nbk + ib];
            }
        }
    };
    fetch(0);

    // per-thread byte offsets inside a row record: the thread's own quad for MMA r == t, the zero quad otherwise
    int aoff[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) aoff[r] = (t == r) ? t * 16 : 64;
    const unsigned char * wq_thr = Wq + (wm * (8 * G) + g) * WREC;
    const f32x2 neg_magic = pack2(-MAGIC_F, -MAGIC_F);
    int4 magic = make_int4(0, 0, 0, 0);

    for (int64_t kb0 = 0; kb0 < nbk; kb0 += KC) {
        if (has_w) {
            int wv[8];
            if (TYPE == B200_TYPE_Q5_0) {
                const uint32_t qw[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
                for (int u = 0; u < 8; ++u) wv[u] = q5_lane_word(qw[u & 3], wqh, u);
            } else {
                wv[0] = wa.x; wv[1] = wa.y; wv[2] = wa.z; wv[3] = wa.w;
                wv[4] = wb.x; wv[5] = wb.y; wv[6] = wb.z; wv[7] = wb.w;
            }
            unsigned char * rec = Wq + (wkb * BM + wrow) * WREC;
#pragma unroll
            for (int u = 0; u < 4; ++u) *(int4 *) (rec + u * 16) = make_int4(wv[2 * u], 0, 0, wv[2 * u + 1]);
            dWs[wkb][wrow] = make_float2(wd, wd);
        }
        if (has_x) {
            *(uint4 *) &Xs[xkb][xcol][0] = xa;
            *(uint4 *) &Xs[xkb][xcol][4] = xb;
            dXs[xkb][xcol] = xdv;
        }
        __syncthreads();
        if (kb0 == 0)       // the four accumulator inputs come from memory so that they stay in four registers
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(magic.x), "=r"(magic.y), "=r"(magic.z), "=r"(magic.w)
                         : "r"((unsigned) __cvta_generic_to_shared(smem_raw + OFF_MAGIC)));
        if (kb0 + KC < nbk) fetch(kb0 + KC);

#pragma unroll 1
        for (int kb = 0; kb < KC; ++kb) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const int row = wm * (8 * G) + gi * 8 + g;
                const unsigned char * rec = wq_thr + (kb * BM + gi * 8) * WREC;
                uint4 a[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) a[r] = *(const uint4 *) (rec + aoff[r]);
                const f32x2 dwp = *(const f32x2 *) &dWs[kb][row];
#pragma unroll
                for (int ti = 0; ti < T; ++ti) {
                    const int col = wn * (8 * T) + ti * 8;
                    const uint2 xv = *(const uint2 *) &Xs[kb][col + g][2 * t];
                    const f32x2 dxp = *(const f32x2 *) &dXs[kb][col + 2 * t];
                    const f32x2 d = mul2(dwp, dxp);
                    f32x2 q[8];
#pragma unroll
                    for (int r = 0; r < 4; ++r) mma_lane_sums(q[2 * r], q[2 * r + 1], a[r], xv, magic);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[gi][ti][j] = fma2(d, add2(q[j], neg_magic), acc[gi][ti][j]);
                }
            }
        }
        __syncthreads();
    }

    // hsum_float_8: (l0+l4, l1+l5, l2+l6, l3+l7) -> (+2) -> (+1), both columns at once
#pragma unroll
    for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int ti = 0; ti < T; ++ti) {
            const f32x2 * a = acc[gi][ti];
            const f32x2 r0 = add2(a[4], a[0]), r1 = add2(a[5], a[1]);
            const f32x2 r2 = add2(a[6], a[2]), r3 = add2(a[7], a[3]);
            const f32x2 s  = add2(add2(r0, r2), add2(r1, r3));
            float lo, hi;
            unpack2(s, lo, hi);
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
            for (int nl = tid / BM; nl < BN; nl += 256 / BM) {
                const int64_t n = n0 + nl;
                if (n < N) {
                    const float v = gemm_ep_apply(ep, n, m, Cs[nl][ml]);
                    if (ep.store_f16) ((__half *) dst)[n * ldd + m] = __float2half_rn(v);
                    else              ((float *) dst)[n * ldd + m] = v;
                }
            }
        }
    }
}

// 0: dp4a kernel, 1: MMA 64 x 64 tile, 2: MMA 32 x 64 tile (B200_GEMM_VARIANT, read once)
static int gemm_variant() {
    static const int v = getenv("B200_GEMM_VARIANT") ? atoi(getenv("B200_GEMM_VARIANT")) : 1;
    return v;
}

template <int TYPE>
static void launch_gemm(const QPlanes & w, int64_t M, int64_t nbk, const int8_t * xq, const float * xd, int64_t N,
                        void * dst, int64_t ldd, const GemmEp & e, cudaStream_t st) {
    const int v = gemm_variant();
    if (v == 1) {
        dim3 grid((unsigned) ((M + 63) / 64), (unsigned) ((N + 63) / 64));
        k_mul_mat_q_mma<TYPE, 2, 4><<<grid, 256, 0, st>>>(w, M, nbk, xq, xd, N, dst, ldd, e);
    } else if (v == 2) {
        dim3 grid((unsigned) ((M + 31) / 32), (unsigned) ((N + 63) / 64));
        k_mul_mat_q_mma<TYPE, 1, 4><<<grid, 256, 0, st>>>(w, M, nbk, xq, xd, N, dst, ldd, e);
    } else {
        dim3 grid((unsigned) ((M + 31) / 32), (unsigned) ((N + 31) / 32));
        k_mul_mat_q<TYPE><<<grid, 256, 0, st>>>(w, M, nbk, xq, xd, N, dst, ldd, e);
    }
}

const uint16_t * b200_gelu_table_device(int * err);

extern "C" int b200_mul_mat_q_ep(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                 const int8_t * xq, const float * xd, int64_t N,
                                 void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream) {
    if (K % 32 != 0 || M <= 0 || N <= 0) return B200_ERR_ARG;
    if (((uintptr_t) xq & 15) != 0 || ((uintptr_t) w_planes & 15) != 0) return B200_ERR_ARG;
    const int64_t nbk = K / 32;
    if (M * nbk > nb_total) return B200_ERR_ARG;
    GemmEp e;
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
    const QPlanes w = q_planes(wtype, w_planes, nb_total);
    if (wtype == B200_TYPE_Q5_0)      launch_gemm<B200_TYPE_Q5_0>(w, M, nbk, xq, xd, N, dst, dst_stride, e, as_stream(stream));
    else if (wtype == B200_TYPE_Q8_0) launch_gemm<B200_TYPE_Q8_0>(w, M, nbk, xq, xd, N, dst, dst_stride, e, as_stream(stream));
    else return B200_ERR_ARG;
    B200_RETURN_LAST();
}

extern "C" int b200_mul_mat_q(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                              const int8_t * xq, const float * xd, int64_t N,
                              float * dst, int64_t dst_stride, void * stream) {
    return b200_mul_mat_q_ep(wtype, w_planes, nb_total, M, K, xq, xd, N, dst, dst_stride, nullptr, stream);
}

// ------------------------------------------------------------------------------------------------
// GEMV for 1..8 columns: a warp streams one weight row (coalesced plane loads), forms the exact
// integer lane sums for 32 blocks in parallel, then eight threads per column replay the FMA chain in
// block order.  Activations are quantised by the CTA itself.
// ------------------------------------------------------------------------------------------------
// Per-column operands: every activation column may live anywhere (columns of one tensor, or single columns of
// several decoder states that step together), and so may its result and the tensors its epilogue adds.
struct GemvCols {
    const float * x[8];
    void *        dst[8];
    const float * add[4][8];      // add[s][n]: operand of epilogue step s for column n (ADD steps only)
};
struct GemvEp {
    int n_steps;
    int kind[4];
    float scalar[4];
    int store_f16;
    const uint16_t * gelu_table;
};

__device__ __forceinline__ void ep_store(const GemvEp & ep, const GemvCols & c, int n, int64_t m, float v) {
    for (int s = 0; s < ep.n_steps; ++s) {
        if (ep.kind[s] == B200_EP_ADD)        v = __fadd_rn(v, c.add[s][n][m]);
        else if (ep.kind[s] == B200_EP_SCALE) v = __fmul_rn(v, ep.scalar[s]);
        else {
            if (v <= -10.0f)     v = 0.0f;
            else if (v < 10.0f)  v = __half2float(__ushort_as_half(ep.gelu_table[__half_as_ushort(__float2half_rn(v))]));
        }
    }
    if (ep.store_f16) ((__half *) c.dst[n])[m] = __float2half_rn(v);
    else              ((float *) c.dst[n])[m] = v;
}

template <int TYPE, int N>
__global__ void __launch_bounds__(128)
k_mul_mat_vec_q(QPlanes w, int64_t M, int64_t nbk, GemvCols cols, int rows_per_warp, GemvEp ep) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int PSTR = 32 * 8 + 8;                 // padded per-column stride of P
    const int K = (int) nbk * 32;
    int *   Xq = (int *) smem_raw;                                   // [N][K/4]
    float * Xd = (float *) (Xq + (size_t) N * (K / 4));              // [N][nbk]
    unsigned char * wbase = smem_raw + (((size_t) N * K + (size_t) N * nbk * 4 + 15) & ~(size_t) 15);   // 16-byte aligned
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int WARP_BYTES = (32 * 12 + 32 + N * PSTR + N * 32) * 4;
    int *   sW  = (int *) (wbase + (size_t) warp * WARP_BYTES);      // [32][12] (8 used)
    float * sDw = (float *) (sW + 32 * 12);                          // [32]
    float * P   = sDw + 32;                                          // [N][PSTR]
    float * D   = P + N * PSTR;                                      // [N][32]

    const int j = lane & 7, bsub = lane >> 3, cn = lane >> 3;
    const int64_t row0 = ((int64_t) blockIdx.x * 4 + warp) * rows_per_warp;
    const int n_chunks = ((int) nbk + 31) / 32;
    const int64_t rows_here = min((int64_t) rows_per_warp, M - row0);

    // weight blocks are fetched one (row, chunk) ahead of the arithmetic; the first fetch overlaps the
    // activation quantisation below
    uint4 pa = make_uint4(0, 0, 0, 0), pb = make_uint4(0, 0, 0, 0);
    uint32_t pqh = 0;
    float pdw = 0.0f;
    auto prefetch = [&](int64_t m, int c0) {
        const int ib = c0 + lane;
        pa = make_uint4(0, 0, 0, 0); pb = pa; pqh = 0; pdw = 0.0f;
        if (ib < (int) nbk) {
            const int64_t blk = m * nbk + ib;
            if (TYPE == B200_TYPE_Q5_0) { pa = __ldg(((const uint4 *) w.qs) + blk); pqh = __ldg(w.qh + blk); }
            else { pa = __ldg(((const uint4 *) w.qs) + blk * 2); pb = __ldg(((const uint4 *) w.qs) + blk * 2 + 1); }
            pdw = __half2float(w.d[blk]);
        }
    };
    chain_release();
    if (rows_here > 0) prefetch(row0, 0);
    chain_wait();                                    // the activations come from the kernel before this one

    // quantise the activation columns (whole CTA): every thread fetches float4 pieces up front (four loads in
    // flight per column), eight consecutive lanes hold one 32-block and share its maximum by shuffles.
    const int n_it = (K + 511) / 512;
#pragma unroll
    for (int n = 0; n < N; ++n) {
        const float * xr = cols.x[n];
        for (int u0 = 0; u0 < n_it; u0 += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = ((u0 + u) * 128 + threadIdx.x) * 4;
                v[u] = e < K ? *(const float4 *) (xr + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = ((u0 + u) * 128 + threadIdx.x) * 4;
                if (u0 + u < n_it) {            // uniform over the CTA
                    float amax = fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                    if (e < K) {
                        const float id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
                        const int q0 = __float2int_rn(__fmul_rn(v[u].x, id)), q1 = __float2int_rn(__fmul_rn(v[u].y, id));
                        const int q2 = __float2int_rn(__fmul_rn(v[u].z, id)), q3 = __float2int_rn(__fmul_rn(v[u].w, id));
                        Xq[(size_t) n * (K / 4) + (e >> 2)] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
                        if ((threadIdx.x & 7) == 0) Xd[n * nbk + (e >> 5)] = round_f16(__fdiv_rn(amax, 127.f));
                    }
                }
            }
        }
    }
    __syncthreads();

    for (int r = 0; r < rows_here; ++r) {
        const int64_t m = row0 + r;
        float acc0 = 0.0f, acc1 = 0.0f;
        for (int c = 0; c < n_chunks; ++c) {
            const int c0 = c * 32;
            {   // publish the prefetched block of this lane, then start the next fetch
                int wv[8];
                if (TYPE == B200_TYPE_Q5_0) {
                    const uint32_t qw[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
                    for (int t = 0; t < 8; ++t) wv[t] = q5_lane_word(qw[t & 3], pqh, t);
                } else {
                    wv[0] = pa.x; wv[1] = pa.y; wv[2] = pa.z; wv[3] = pa.w;
                    wv[4] = pb.x; wv[5] = pb.y; wv[6] = pb.z; wv[7] = pb.w;
                }
                *(int4 *) &sW[lane * 12]     = make_int4(wv[0], wv[1], wv[2], wv[3]);
                *(int4 *) &sW[lane * 12 + 4] = make_int4(wv[4], wv[5], wv[6], wv[7]);
                sDw[lane] = pdw;
            }
            __syncwarp();
            if (c + 1 < n_chunks)       prefetch(m, c0 + 32);
            else if (r + 1 < rows_here) prefetch(m + 1, 0);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int ibl = i * 4 + bsub;
                const int ib  = c0 + ibl;
                if (ib < (int) nbk) {
                    const int wv = sW[ibl * 12 + j];
#pragma unroll
                    for (int n = 0; n < N; ++n) {
                        const int xv = Xq[(size_t) n * (K / 4) + ib * 8 + j];
                        P[n * PSTR + ibl * 8 + j] = __fadd_rn(__int_as_float(__dp4a(wv, xv, MAGIC_I)), -MAGIC_F);
                    }
                    if (j == 0) {
                        const float dw = sDw[ibl];
#pragma unroll
                        for (int n = 0; n < N; ++n) D[n * 32 + ibl] = __fmul_rn(dw, Xd[n * nbk + ib]);
                    }
                }
            }
            __syncwarp();
            const int nblk = min(32, (int) nbk - c0);
            if (cn < N) {
#pragma unroll 8
                for (int ibl = 0; ibl < nblk; ++ibl) acc0 = __fmaf_rn(D[cn * 32 + ibl], P[cn * PSTR + ibl * 8 + j], acc0);
            }
            if (N > 4 && cn + 4 < N) {
#pragma unroll 8
                for (int ibl = 0; ibl < nblk; ++ibl) acc1 = __fmaf_rn(D[(cn + 4) * 32 + ibl], P[(cn + 4) * PSTR + ibl * 8 + j], acc1);
            }
            __syncwarp();
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            acc0 = __fadd_rn(acc0, __shfl_xor_sync(0xffffffffu, acc0, o));
            acc1 = __fadd_rn(acc1, __shfl_xor_sync(0xffffffffu, acc1, o));
        }
        if (j == 0) {
            if (cn < N) ep_store(ep, cols, cn, m, acc0);
            if (N > 4 && cn + 4 < N) ep_store(ep, cols, cn + 4, m, acc1);
        }
    }
}

template <int TYPE, int N>
static int launch_vec(const QPlanes & w, int64_t M, int64_t nbk, const GemvCols & cols, const GemvEp & ep, cudaStream_t st) {
    constexpr int PSTR = 32 * 8 + 8;
    const size_t smem = (((size_t) N * nbk * 32 + (size_t) N * nbk * 4 + 15) & ~(size_t) 15) + 4 * (size_t) ((32 * 12 + 32 + N * PSTR + N * 32) * 4);
    static bool attr_done[64] = {false};   // per instantiation and device; benign race (idempotent call)
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(k_mul_mat_vec_q<TYPE, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_done[dev] = true;
    }
    if (smem > 200 * 1024) return B200_ERR_ARG;
    // rows per warp: one wave of CTAs when M allows it (148 SMs x several CTAs), more rows per warp for tall matrices
    int rpw = 1;
    while (rpw < 8 && (M + 4 * (rpw * 2) - 1) / (4 * (rpw * 2)) >= 148 * 4) rpw *= 2;
    const int64_t rows_per_cta = 4 * rpw;
    launch_chained(k_mul_mat_vec_q<TYPE, N>, dim3((unsigned) ((M + rows_per_cta - 1) / rows_per_cta)), dim3(128), smem, st, w, M, nbk, cols, rpw, ep);
    B200_RETURN_LAST();
}

template <int TYPE>
static int launch_vec_n(int N, const QPlanes & w, int64_t M, int64_t nbk, const GemvCols & cols, const GemvEp & ep, cudaStream_t st) {
    switch (N) {
        case 1: return launch_vec<TYPE, 1>(w, M, nbk, cols, ep, st);
        case 2: return launch_vec<TYPE, 2>(w, M, nbk, cols, ep, st);
        case 3: return launch_vec<TYPE, 3>(w, M, nbk, cols, ep, st);
        case 4: return launch_vec<TYPE, 4>(w, M, nbk, cols, ep, st);
        case 5: return launch_vec<TYPE, 5>(w, M, nbk, cols, ep, st);
        case 6: return launch_vec<TYPE, 6>(w, M, nbk, cols, ep, st);
        case 7: return launch_vec<TYPE, 7>(w, M, nbk, cols, ep, st);
        case 8: return launch_vec<TYPE, 8>(w, M, nbk, cols, ep, st);
    }
    return B200_ERR_ARG;
}

const uint16_t * b200_gelu_table_device(int * err);

static int fill_ep(GemvEp & e, int n_steps, const int * kind, const float * scalar, int store_f16) {
    memset(&e, 0, sizeof(e));
    if (n_steps < 0 || n_steps > 4) return B200_ERR_ARG;
    e.n_steps = n_steps;
    e.store_f16 = store_f16;
    for (int s = 0; s < n_steps; ++s) {
        e.kind[s] = kind[s]; e.scalar[s] = scalar[s];
        if (e.kind[s] == B200_EP_GELU) {
            if (!e.gelu_table) {
                int err = 0;
                e.gelu_table = b200_gelu_table_device(&err);
                if (err) return err;
            }
        } else if (e.kind[s] != B200_EP_ADD && e.kind[s] != B200_EP_SCALE) return B200_ERR_ARG;
    }
    return 0;
}

extern "C" int b200_mul_mat_vec_q_cols(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                       const b200_gemv_col * cols, int n_cols, const b200_gemv_ep * ep, void * stream) {
    if (K % 32 != 0 || M <= 0 || n_cols < 1 || n_cols > 8 || !cols) return B200_ERR_ARG;
    if (((uintptr_t) w_planes & 15) != 0) return B200_ERR_ARG;
    const int64_t nbk = K / 32;
    if (M * nbk > nb_total) return B200_ERR_ARG;
    GemvEp e;
    static const int   no_kind[4]   = {0, 0, 0, 0};
    static const float no_scalar[4] = {0, 0, 0, 0};
    int rc = ep ? fill_ep(e, ep->n_steps, ep->kind, ep->scalar, ep->store_f16) : fill_ep(e, 0, no_kind, no_scalar, 0);
    if (rc) return rc;
    GemvCols c;
    memset(&c, 0, sizeof(c));
    for (int n = 0; n < n_cols; ++n) {
        if (((uintptr_t) cols[n].x & 15) != 0 || !cols[n].dst) return B200_ERR_ARG;
        c.x[n] = cols[n].x; c.dst[n] = cols[n].dst;
        for (int s = 0; s < e.n_steps; ++s) {
            c.add[s][n] = cols[n].add[s];
            if (e.kind[s] == B200_EP_ADD && !c.add[s][n]) return B200_ERR_ARG;
        }
    }
    const QPlanes w = q_planes(wtype, w_planes, nb_total);
    if (wtype == B200_TYPE_Q5_0) return launch_vec_n<B200_TYPE_Q5_0>(n_cols, w, M, nbk, c, e, as_stream(stream));
    if (wtype == B200_TYPE_Q8_0) return launch_vec_n<B200_TYPE_Q8_0>(n_cols, w, M, nbk, c, e, as_stream(stream));
    return B200_ERR_ARG;
}

extern "C" int b200_mul_mat_vec_q_ep(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                     const float * x, int64_t x_stride_bytes, int64_t N,
                                     void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream) {
    if (N < 1 || N > 8 || (x_stride_bytes & 15) != 0) return B200_ERR_ARG;
    b200_gemv_col cols[8];
    b200_gemv_ep  e;
    memset(&e, 0, sizeof(e));
    memset(cols, 0, sizeof(cols));
    if (ep) {
        if (ep->n_steps < 0 || ep->n_steps > 4) return B200_ERR_ARG;
        e.n_steps = ep->n_steps; e.store_f16 = ep->store_f16;
        for (int s = 0; s < ep->n_steps; ++s) { e.kind[s] = ep->step[s].kind; e.scalar[s] = ep->step[s].scalar; }
    }
    const int64_t esz = (ep && ep->store_f16) ? 2 : 4;
    for (int n = 0; n < (int) N; ++n) {
        cols[n].x   = (const float *) ((const char *) x + n * x_stride_bytes);
        cols[n].dst = (char *) dst + n * dst_stride * esz;
        for (int s = 0; ep && s < ep->n_steps; ++s)
            cols[n].add[s] = ep->step[s].ptr ? ep->step[s].ptr + n * ep->step[s].stride_n : nullptr;
    }
    return b200_mul_mat_vec_q_cols(wtype, w_planes, nb_total, M, K, cols, (int) N, &e, stream);
}

extern "C" int b200_mul_mat_vec_q(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                  const float * x, int64_t x_stride_bytes, int64_t N,
                                  float * dst, int64_t dst_stride, void * stream) {
    return b200_mul_mat_vec_q_ep(wtype, w_planes, nb_total, M, K, x, x_stride_bytes, N, dst, dst_stride, nullptr, stream);
}

// ------------------------------------------------------------------------------------------------
// Skinny product for up to 32 activation columns that were quantised beforehand (columns of one tensor or single
// columns of many decoder states).  A CTA owns R weight rows for the whole K: the rows are dequantised to int8 lane
// words in shared memory once, the quantised columns are copied next to them, and then every thread replays the
// FMA chain of lane j for one row and CT columns, block after block.  Same sums, same order as the kernels above.
// ------------------------------------------------------------------------------------------------
struct GemvCols32 {
    void *        dst[32];
    const float * add[4][32];
};

__device__ __forceinline__ void ep_store32(const GemvEp & ep, const GemvCols32 & c, int n, int64_t m, float v) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        if (s < ep.n_steps) {
            if (ep.kind[s] == B200_EP_ADD)        v = __fadd_rn(v, c.add[s][n][m]);
            else if (ep.kind[s] == B200_EP_SCALE) v = __fmul_rn(v, ep.scalar[s]);
            else {
                if (v <= -10.0f)     v = 0.0f;
                else if (v < 10.0f)  v = __half2float(__ushort_as_half(ep.gelu_table[__half_as_ushort(__float2half_rn(v))]));
            }
        }
    }
    if (ep.store_f16) ((__half *) c.dst[n])[m] = __float2half_rn(v);
    else              ((float *) c.dst[n])[m] = v;
}

template <int TYPE, int R, int CT, int U>
__device__ __forceinline__ void gemv_skinny_body(const QPlanes & w, int64_t M, int nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd,
                                                 int n_cols, const GemvCols32 & cols, const GemvEp & ep, int64_t row0) {
    extern __shared__ __align__(16) unsigned char sk_smem[];
    constexpr int CG = 32 / R;
    const int RS   = nbk * 8 + ((8 - (nbk * 8) % 32 + 32) % 32);      // row stride in words, == 8 mod 32
    const int XS   = nbk * 8;                                         // words per column
    int *   Wsm = (int *) sk_smem;                                    // [R][RS]
    int *   Xsm = Wsm + R * RS;                                       // [n_cols][XS]
    float * dW  = (float *) (Xsm + n_cols * XS);                      // [R][nbk]
    float * dX  = dW + R * nbk;                                       // [n_cols][nbk]
    const int tid = threadIdx.x;
    chain_release();

    // weight rows: one (row, block) per thread and pass, the loads of U passes in flight at once (a pass is one round trip
    // to HBM; the long rows of the second MLP product would otherwise pay five of them in sequence)
    for (int it0 = tid; it0 < R * nbk; it0 += U * 256) {
        uint4 qa[U], qb[U]; uint32_t qh[U]; __half dh[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int it = it0 + u * 256;
            const int r = it / nbk, ib = it - r * nbk;
            const int64_t m = row0 + r;
            qa[u] = make_uint4(0, 0, 0, 0); qb[u] = make_uint4(0, 0, 0, 0); qh[u] = 0; dh[u] = __ushort_as_half((unsigned short) 0);
            if (it < R * nbk && m < M) {
                const int64_t blk = m * nbk + ib;
                if (TYPE == B200_TYPE_Q5_0) { qa[u] = __ldg(((const uint4 *) w.qs) + blk); qh[u] = __ldg(w.qh + blk); }
                else { qa[u] = __ldg(((const uint4 *) w.qs) + blk * 2); qb[u] = __ldg(((const uint4 *) w.qs) + blk * 2 + 1); }
                dh[u] = w.d[blk];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int it = it0 + u * 256;
            if (it >= R * nbk) break;
            const int r = it / nbk, ib = it - r * nbk;
            const int64_t m = row0 + r;
            int wv[8];
            float dw = 0.0f;
#pragma unroll
            for (int t = 0; t < 8; ++t) wv[t] = 0;
            if (m < M) {
                if (TYPE == B200_TYPE_Q5_0) {
                    const uint32_t qw[4] = {qa[u].x, qa[u].y, qa[u].z, qa[u].w};
#pragma unroll
                    for (int t = 0; t < 8; ++t) wv[t] = q5_lane_word(qw[t & 3], qh[u], t);
                } else {
                    wv[0] = qa[u].x; wv[1] = qa[u].y; wv[2] = qa[u].z; wv[3] = qa[u].w;
                    wv[4] = qb[u].x; wv[5] = qb[u].y; wv[6] = qb[u].z; wv[7] = qb[u].w;
                }
                dw = __half2float(dh[u]);
            }
            *(int4 *) &Wsm[r * RS + ib * 8]     = make_int4(wv[0], wv[1], wv[2], wv[3]);
            *(int4 *) &Wsm[r * RS + ib * 8 + 4] = make_int4(wv[4], wv[5], wv[6], wv[7]);
            dW[r * nbk + ib] = dw;
        }
    }
    chain_wait();                                                     // the columns come from the kernel before this one
    {
        const uint4 * src = (const uint4 *) xq;
        uint4 * dstv = (uint4 *) Xsm;
        const int n16 = n_cols * XS / 4;
        for (int it = tid; it < n16; it += 256) dstv[it] = src[it];
        for (int it = tid; it < n_cols * nbk; it += 256) dX[it] = xd[it];
    }
    __syncthreads();

    const int j = tid & 7, grp = tid >> 3;
    const int r = grp % R, cg = grp / R;
    const int c0 = cg * CT;
    float acc[CT];
#pragma unroll
    for (int c = 0; c < CT; ++c) acc[c] = 0.0f;
    const int *   wrow = Wsm + r * RS + j;
    const float * dwr  = dW + r * nbk;
#pragma unroll 4
    for (int ib = 0; ib < nbk; ++ib) {
        const int   wv = wrow[ib * 8];
        const float dw = dwr[ib];
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const int col = min(c0 + c, n_cols - 1);
            const int   xv = Xsm[col * XS + ib * 8 + j];
            const float q  = __fadd_rn(__int_as_float(__dp4a(wv, xv, MAGIC_I)), -MAGIC_F);
            acc[c] = __fmaf_rn(__fmul_rn(dw, dX[col * nbk + ib]), q, acc[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < CT; ++c) {
        float v = acc[c];
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
        acc[c] = v;
    }
    const int64_t m = row0 + r;
    if (j == 0 && m < M) {
#pragma unroll
        for (int c = 0; c < CT; ++c) if (c0 + c < n_cols) ep_store32(ep, cols, c0 + c, m, acc[c]);
    }
}

template <int TYPE, int R, int CT, int U>
__global__ void __launch_bounds__(256)
k_gemv_skinny(QPlanes w, int64_t M, int nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd, int n_cols,
              GemvCols32 cols, GemvEp ep) {
    gemv_skinny_body<TYPE, R, CT, U>(w, M, nbk, xq, xd, n_cols, cols, ep, (int64_t) blockIdx.x * R);
}

// Up to three products that share their activation columns (the Q, K and V projections of a layer) in one launch:
// blockIdx.y selects the weight matrix with its own outputs and epilogue.
struct SkinnyJob { QPlanes w; int64_t M; GemvCols32 cols; GemvEp ep; };
struct SkinnyJobs { SkinnyJob j[3]; };
template <int TYPE, int R, int CT>
__global__ void __launch_bounds__(256)
k_gemv_skinny_multi(const __grid_constant__ SkinnyJobs jobs, int nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd, int n_cols) {
    const SkinnyJob & J = jobs.j[blockIdx.y];
    const int64_t row0 = (int64_t) blockIdx.x * R;
    if (row0 >= J.M) return;
    gemv_skinny_body<TYPE, R, CT, 2>(J.w, J.M, nbk, xq, xd, n_cols, J.cols, J.ep, row0);
}

template <int TYPE, int R, int CT>
static int launch_skinny_multi(const SkinnyJobs & jobs, int n_jobs, int nbk, const int8_t * xq, const float * xd, int n_cols, cudaStream_t st) {
    const int RS = nbk * 8 + ((8 - (nbk * 8) % 32 + 32) % 32);
    const size_t smem = ((size_t) R * RS + (size_t) n_cols * nbk * 8 + (size_t) R * nbk + (size_t) n_cols * nbk) * 4;
    if (smem > 220 * 1024) return B200_ERR_ARG;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(k_gemv_skinny_multi<TYPE, R, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        attr_done[dev] = true;
    }
    int64_t max_m = 0;
    for (int i = 0; i < n_jobs; ++i) max_m = jobs.j[i].M > max_m ? jobs.j[i].M : max_m;
    launch_chained(k_gemv_skinny_multi<TYPE, R, CT>, dim3((unsigned) ((max_m + R - 1) / R), (unsigned) n_jobs), dim3(256), smem, st, jobs, nbk, xq, xd, n_cols);
    B200_RETURN_LAST();
}

template <int TYPE, int R, int CT>
static int launch_skinny(const QPlanes & w, int64_t M, int nbk, const int8_t * xq, const float * xd, int n_cols, const GemvCols32 & cols,
                         const GemvEp & ep, cudaStream_t st) {
    const int RS = nbk * 8 + ((8 - (nbk * 8) % 32 + 32) % 32);
    const size_t smem = ((size_t) R * RS + (size_t) n_cols * nbk * 8 + (size_t) R * nbk + (size_t) n_cols * nbk) * 4;
    if (smem > 220 * 1024) return B200_ERR_ARG;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(k_gemv_skinny<TYPE, R, CT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(k_gemv_skinny<TYPE, R, CT, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        attr_done[dev] = true;
    }
    // Loads in flight per thread while the weight rows are staged.  Measured on B200 (12 columns): the deeper form (more
    // registers) is faster when the grid is about one CTA per SM (1280 x 1280: 8.6 against 10.6 us) and for long rows,
    // the shallow form when several CTAs share an SM (5120 x 1280: 13.7 against 14.6 us).
    if (R * nbk <= 512 && (M + R - 1) / R > 300) launch_chained(k_gemv_skinny<TYPE, R, CT, 2>, dim3((unsigned) ((M + R - 1) / R)), dim3(256), smem, st, w, M, nbk, xq, xd, n_cols, cols, ep);
    else                launch_chained(k_gemv_skinny<TYPE, R, CT, 4>, dim3((unsigned) ((M + R - 1) / R)), dim3(256), smem, st, w, M, nbk, xq, xd, n_cols, cols, ep);
    B200_RETURN_LAST();
}

// Second form of the skinny product: a thread owns one weight row and a PAIR of columns with all eight lane sums of
// both (eight packed f32x2 accumulators), so the block scale is formed once per output and every lane update is one
// packed FMA.  R rows per CTA, blockDim = R * ceil(n_cols / 2).
template <int TYPE, int R>
__global__ void __launch_bounds__(256)
k_gemv_skinny2(QPlanes w, int64_t M, int nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd, int n_cols,
               GemvCols32 cols, GemvEp ep) {
    extern __shared__ __align__(16) unsigned char sk_smem[];
    const int CP  = (n_cols + 1) >> 1;
    const int WS  = nbk * 8;                                          // words per weight row
    const int XS  = nbk * 8 + 4;                                      // words per column, == 4 mod 32: conflict-free LDS.128 across columns
    int *   Wsm = (int *) sk_smem;                                    // [R][WS]
    int *   Xsm = Wsm + R * WS;                                       // [n_cols][XS]
    float * dW  = (float *) (Xsm + n_cols * XS);                      // [R][nbk]
    float * dX  = dW + R * nbk;                                       // [n_cols][nbk]
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int64_t row0 = (int64_t) blockIdx.x * R;
    chain_release();

    for (int it = tid; it < R * nbk; it += nthr) {
        const int r = it / nbk, ib = it - r * nbk;
        const int64_t m = row0 + r;
        int wv[8];
        float dw = 0.0f;
#pragma unroll
        for (int t = 0; t < 8; ++t) wv[t] = 0;
        if (m < M) {
            const int64_t blk = m * nbk + ib;
            if (TYPE == B200_TYPE_Q5_0) {
                const uint4    q  = __ldg(((const uint4 *) w.qs) + blk);
                const uint32_t qh = __ldg(w.qh + blk);
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int t = 0; t < 8; ++t) wv[t] = q5_lane_word(qw[t & 3], qh, t);
            } else {
                const uint4 a = __ldg(((const uint4 *) w.qs) + blk * 2), b = __ldg(((const uint4 *) w.qs) + blk * 2 + 1);
                wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w;
                wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
            }
            dw = __half2float(w.d[blk]);
        }
        *(int4 *) &Wsm[r * WS + ib * 8]     = make_int4(wv[0], wv[1], wv[2], wv[3]);
        *(int4 *) &Wsm[r * WS + ib * 8 + 4] = make_int4(wv[4], wv[5], wv[6], wv[7]);
        dW[r * nbk + ib] = dw;
    }
    chain_wait();                                                     // the columns come from the kernel before this one
    {
        const uint4 * src = (const uint4 *) xq;
        const int per_col = nbk * 2;                                  // 16-byte pieces per column
        for (int it = tid; it < n_cols * per_col; it += nthr) {
            const int c = it / per_col, pz = it - c * per_col;
            *(uint4 *) &Xsm[c * XS + pz * 4] = src[it];
        }
        for (int it = tid; it < n_cols * nbk; it += nthr) dX[it] = xd[it];
    }
    __syncthreads();

    const int r = tid / CP, cp = tid - r * CP;
    const int cA = cp, cB = min(cp + CP, n_cols - 1);
    f32x2 acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0ull;
    const int *   wrow = Wsm + r * WS;
    const int *   xa   = Xsm + cA * XS;
    const int *   xb   = Xsm + cB * XS;
    const float * dwr  = dW + r * nbk;
    const float * dxa  = dX + cA * nbk;
    const float * dxb  = dX + cB * nbk;
    const f32x2 neg_magic = pack2(-MAGIC_F, -MAGIC_F);
#pragma unroll 2
    for (int ib = 0; ib < nbk; ++ib) {
        int wv[8], x0[8], x1[8];
        *(int4 *) &wv[0] = *(const int4 *) &wrow[ib * 8];
        *(int4 *) &wv[4] = *(const int4 *) &wrow[ib * 8 + 4];
        *(int4 *) &x0[0] = *(const int4 *) &xa[ib * 8];
        *(int4 *) &x0[4] = *(const int4 *) &xa[ib * 8 + 4];
        *(int4 *) &x1[0] = *(const int4 *) &xb[ib * 8];
        *(int4 *) &x1[4] = *(const int4 *) &xb[ib * 8 + 4];
        const float dw = dwr[ib];
        const f32x2 d = mul2(pack2(dw, dw), pack2(dxa[ib], dxb[ib]));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const f32x2 q = add2(pack2i(__dp4a(wv[j], x0[j], MAGIC_I), __dp4a(wv[j], x1[j], MAGIC_I)), neg_magic);
            acc[j] = fma2(d, q, acc[j]);
        }
    }
    const f32x2 r0 = add2(acc[4], acc[0]), r1 = add2(acc[5], acc[1]);
    const f32x2 r2 = add2(acc[6], acc[2]), r3 = add2(acc[7], acc[3]);
    const f32x2 sres = add2(add2(r0, r2), add2(r1, r3));
    float lo, hi;
    unpack2(sres, lo, hi);
    const int64_t m = row0 + r;
    if (m < M) {
        ep_store32(ep, cols, cA, m, lo);
        if (cp + CP < n_cols) ep_store32(ep, cols, cp + CP, m, hi);
    }
}

template <int TYPE, int R>
static int launch_skinny2(const QPlanes & w, int64_t M, int nbk, const int8_t * xq, const float * xd, int n_cols, const GemvCols32 & cols,
                          const GemvEp & ep, cudaStream_t st) {
    const int CP = (n_cols + 1) / 2;
    const size_t smem = ((size_t) R * nbk * 8 + (size_t) n_cols * (nbk * 8 + 4) + (size_t) R * nbk + (size_t) n_cols * nbk) * 4;
    if (smem > 220 * 1024 || R * CP > 256) return B200_ERR_ARG;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(k_gemv_skinny2<TYPE, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        attr_done[dev] = true;
    }
    launch_chained(k_gemv_skinny2<TYPE, R>, dim3((unsigned) ((M + R - 1) / R)), dim3(R * CP), smem, st, w, M, nbk, xq, xd, n_cols, cols, ep);
    B200_RETURN_LAST();
}

template <int TYPE>
static int launch_skinny_n(const QPlanes & w, int64_t M, int nbk, const int8_t * xq, const float * xd, int n_cols, const GemvCols32 & cols,
                           const GemvEp & ep, cudaStream_t st) {
    // measured on B200: the column-pair form wins for many columns on short rows and for the tall logits matrix; for 9..16
    // columns it neither helps nor hurts the throughput of 64 concurrent states (19.5 against 19.2-20.1 ms per round of
    // decode steps) and its single launch is slower, so the lane-per-thread form keeps those
    if (n_cols >= 9 && M >= 16384) return launch_skinny2<TYPE, 16>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    if (n_cols >= 17 && nbk <= 80) return launch_skinny2<TYPE, 8>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    if (M >= 16384 && n_cols > 4) {      // tall matrices (logits): more rows per CTA so that the columns are staged fewer times
        if (n_cols <= 8)  return launch_skinny<TYPE, 32, 8>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
        if (n_cols <= 16) return launch_skinny<TYPE, 32, 16>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
        return launch_skinny<TYPE, 32, 32>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    }
    if (n_cols == 1)  return launch_skinny<TYPE, 32, 1>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    if (n_cols == 2)  return launch_skinny<TYPE, 16, 1>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    if (n_cols <= 4)  return launch_skinny<TYPE, 8, 1>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    if (n_cols <= 8)  return launch_skinny<TYPE, 8, 2>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    if (n_cols <= 16) return launch_skinny<TYPE, 8, 4>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
    return launch_skinny<TYPE, 8, 8>(w, M, nbk, xq, xd, n_cols, cols, ep, st);
}

struct ColPtrs32 { const float * x[32]; };
__global__ void k_quantize_cols(ColPtrs32 cols, int n_cols, int nbk, int8_t * __restrict__ qs, float * __restrict__ d) {
    const int lane = threadIdx.x & 31;
    const int blk  = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    chain_release();
    chain_wait();
    if (blk >= n_cols * nbk) return;
    const int c = blk / nbk, ib = blk - c * nbk;
    const float v = cols.x[c][ib * 32 + lane];
    int8_t q; float dd;
    quantize_block_q8_0(v, lane, q, dd);
    qs[(size_t) blk * 32 + lane] = q;
    if (lane == 0) d[blk] = dd;
}

extern "C" int b200_quantize_cols(const float * const * x_cols, int n_cols, int64_t K, int8_t * xq, float * xd, void * stream) {
    if (n_cols < 1 || n_cols > 32 || K % 32 != 0 || K <= 0) return B200_ERR_ARG;
    ColPtrs32 c;
    memset(&c, 0, sizeof(c));
    for (int i = 0; i < n_cols; ++i) { if (!x_cols[i]) return B200_ERR_ARG; c.x[i] = x_cols[i]; }
    const int nbk = (int) (K / 32);
    const int nblk = n_cols * nbk;
    launch_chained(k_quantize_cols, dim3((unsigned) ((nblk + 7) / 8)), dim3(256), 0, as_stream(stream), c, n_cols, nbk, xq, xd);
    B200_RETURN_LAST();
}

extern "C" int b200_mul_mat_cols_q(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                   const int8_t * xq, const float * xd, const b200_gemv_col * cols, int n_cols,
                                   const b200_gemv_ep * ep, void * stream) {
    if (K % 32 != 0 || M <= 0 || n_cols < 1 || n_cols > 32 || !cols) return B200_ERR_ARG;
    if (((uintptr_t) w_planes & 15) != 0 || ((uintptr_t) xq & 15) != 0) return B200_ERR_ARG;
    const int64_t nbk = K / 32;
    if (M * nbk > nb_total) return B200_ERR_ARG;
    GemvEp e;
    static const int   no_kind[4]   = {0, 0, 0, 0};
    static const float no_scalar[4] = {0, 0, 0, 0};
    int rc = ep ? fill_ep(e, ep->n_steps, ep->kind, ep->scalar, ep->store_f16) : fill_ep(e, 0, no_kind, no_scalar, 0);
    if (rc) return rc;
    GemvCols32 c;
    memset(&c, 0, sizeof(c));
    for (int n = 0; n < n_cols; ++n) {
        if (!cols[n].dst) return B200_ERR_ARG;
        c.dst[n] = cols[n].dst;
        for (int s = 0; s < e.n_steps; ++s) {
            c.add[s][n] = cols[n].add[s];
            if (e.kind[s] == B200_EP_ADD && !c.add[s][n]) return B200_ERR_ARG;
        }
    }
    const QPlanes w = q_planes(wtype, w_planes, nb_total);
    if (wtype == B200_TYPE_Q5_0) return launch_skinny_n<B200_TYPE_Q5_0>(w, M, (int) nbk, xq, xd, n_cols, c, e, as_stream(stream));
    if (wtype == B200_TYPE_Q8_0) return launch_skinny_n<B200_TYPE_Q8_0>(w, M, (int) nbk, xq, xd, n_cols, c, e, as_stream(stream));
    return B200_ERR_ARG;
}

extern "C" int b200_mul_mat_cols_q_multi(int wtype, int n_jobs, const void * const * w_planes, const int64_t * nb_total, const int64_t * M,
                                         int64_t K, const int8_t * xq, const float * xd, const b200_gemv_col * const * cols, int n_cols,
                                         const b200_gemv_ep * const * ep, void * stream) {
    if (n_jobs < 1 || n_jobs > 3 || K % 32 != 0 || n_cols < 1 || n_cols > 32 || !cols || !w_planes || !nb_total || !M) return B200_ERR_ARG;
    if (((uintptr_t) xq & 15) != 0) return B200_ERR_ARG;
    const int64_t nbk = K / 32;
    static const int   no_kind[4]   = {0, 0, 0, 0};
    static const float no_scalar[4] = {0, 0, 0, 0};
    SkinnyJobs jobs;
    memset(&jobs, 0, sizeof(jobs));
    for (int i = 0; i < n_jobs; ++i) {
        if (!w_planes[i] || ((uintptr_t) w_planes[i] & 15) != 0 || M[i] <= 0 || M[i] * nbk > nb_total[i] || !cols[i]) return B200_ERR_ARG;
        SkinnyJob & J = jobs.j[i];
        const b200_gemv_ep * e = ep ? ep[i] : nullptr;
        const int rc = e ? fill_ep(J.ep, e->n_steps, e->kind, e->scalar, e->store_f16) : fill_ep(J.ep, 0, no_kind, no_scalar, 0);
        if (rc) return rc;
        for (int n = 0; n < n_cols; ++n) {
            if (!cols[i][n].dst) return B200_ERR_ARG;
            J.cols.dst[n] = cols[i][n].dst;
            for (int st = 0; st < J.ep.n_steps; ++st) {
                J.cols.add[st][n] = cols[i][n].add[st];
                if (J.ep.kind[st] == B200_EP_ADD && !J.cols.add[st][n]) return B200_ERR_ARG;
            }
        }
        J.w = q_planes(wtype, w_planes[i], nb_total[i]);
        J.M = M[i];
    }
    cudaStream_t st = as_stream(stream);
#define B200_MULTI(T) \
    (n_cols <= 8 ? launch_skinny_multi<T, 8, 2>(jobs, n_jobs, (int) nbk, xq, xd, n_cols, st) : \
     n_cols <= 16 ? launch_skinny_multi<T, 8, 4>(jobs, n_jobs, (int) nbk, xq, xd, n_cols, st) : \
                    launch_skinny_multi<T, 8, 8>(jobs, n_jobs, (int) nbk, xq, xd, n_cols, st))
    if (wtype == B200_TYPE_Q5_0) return B200_MULTI(B200_TYPE_Q5_0);
    if (wtype == B200_TYPE_Q8_0) return B200_MULTI(B200_TYPE_Q8_0);
#undef B200_MULTI
    return B200_ERR_ARG;
}


// ------------------------------------------------------------------------------------------------
// Product with the activation scratch in a fixed device array (for callers that cannot allocate).
// ------------------------------------------------------------------------------------------------
#define B200_STATIC_SCRATCH_BYTES (9 * 1024 * 1024)
static __device__ __align__(256) unsigned char g_static_scratch[B200_STATIC_SCRATCH_BYTES];

extern "C" int64_t b200_static_scratch_bytes(void) { return B200_STATIC_SCRATCH_BYTES; }

// In host code the array's name is only a handle for the runtime, not a device address: the address each
// device gave its copy is asked for once per device, with that device current.
static int static_scratch_address(unsigned char ** out) {
    static std::atomic<unsigned char *> addr[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int) e;
    if (dev < 0 || dev >= 64) return B200_ERR_ARG;
    unsigned char * p = addr[dev].load(std::memory_order_acquire);
    if (!p) {
        void * sym = nullptr;
        e = cudaGetSymbolAddress(&sym, g_static_scratch);
        if (e != cudaSuccess) return (int) e;
        p = (unsigned char *) sym;
        addr[dev].store(p, std::memory_order_release);      // same value from every thread that races here
    }
    *out = p;
    return 0;
}

extern "C" int b200_mul_mat_q_static(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                     const float * x, int64_t x_stride_bytes, int64_t N,
                                     float * dst, int64_t dst_stride, void * stream) {
    if (K % 32 != 0 || M <= 0 || N <= 0 || K <= 0) return B200_ERR_ARG;
    if (wtype != B200_TYPE_Q5_0 && wtype != B200_TYPE_Q8_0) return B200_ERR_ARG;
    if (N > B200_STATIC_SCRATCH_BYTES / K) {             // also keeps N * K from overflowing
        fprintf(stderr, "b200_mul_mat_q_static: %lld activation rows of %lld values do not fit the fixed array of %d bytes\n",
                (long long) N, (long long) K, B200_STATIC_SCRATCH_BYTES);
        return B200_ERR_TOO_LARGE;
    }
    const int64_t q_bytes = N * K, d_bytes = N * (K / 32) * 4;
    const int64_t q_pad = (q_bytes + 255) & ~(int64_t) 255;
    if (q_pad + d_bytes > B200_STATIC_SCRATCH_BYTES) {
        fprintf(stderr, "b200_mul_mat_q_static: %lld activation rows of %lld values need %lld bytes of scratch, the fixed array holds %d\n",
                (long long) N, (long long) K, (long long) (q_pad + d_bytes), B200_STATIC_SCRATCH_BYTES);
        return B200_ERR_TOO_LARGE;
    }
    // everything else is checked before the first launch: a bad argument never costs a kernel on the device
    if (!x || !dst || !w_planes) return B200_ERR_ARG;
    if (((uintptr_t) w_planes & 15) != 0 || ((uintptr_t) x & 3) != 0) return B200_ERR_ARG;
    if (x_stride_bytes < 4 * K || (x_stride_bytes & 3) != 0 || dst_stride < M) return B200_ERR_ARG;
    if (M > nb_total / (K / 32)) return B200_ERR_ARG;
    unsigned char * scratch = nullptr;
    int e = static_scratch_address(&scratch);
    if (e) return e;
    int8_t * xq = (int8_t *) scratch;
    float *  xd = (float *) (scratch + q_pad);
    e = b200_quantize_q8_0(x, N, K, x_stride_bytes, xq, xd, stream);
    if (e) return e;
    return b200_mul_mat_q(wtype, w_planes, nb_total, M, K, xq, xd, N, dst, dst_stride, stream);
}
