// F16 matrix products in the summation order of ggml_vec_dot_f16 on AVX2/F16C
// (ggml/src/ggml-cpu/vec.cpp:128-167, simd-mappings.h:236-332): 32 running sums (4 vectors of 8
// lanes), element k goes to sum k%32 by FMA, then sum0+=sum2, sum1+=sum3, sum0+=sum1, fold the two
// 128-bit halves and two horizontal adds; the tail (K % 32) is added in double.
// Also the 1-D im2col that feeds the conv stem.
#include "b200_common.cuh"

// d = a * b + c with two f16 factors (bit patterns), f32 addend and result: the mixed-precision FMA of sm_100.  The
// product of two f16 numbers is exact in f32, so this is fmaf(float(a), float(b), c) without the two conversions.
__device__ __forceinline__ float fma_f16_f32(unsigned short a, unsigned short b, float c) {
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(c) : "h"(a), "h"(b));
    return c;
}

// A warp owns TM x TN outputs (lane = running sum k % 32): 4 x 4 for small products, 8 x 8 where both extents are large
// (the conv stem: 3000 x 1280 and 1500 x 1280 outputs), which halves the loads per FMA.
template <bool X_F16, int TM, int TN>
__global__ void __launch_bounds__(128)
k_mul_mat_f16(const char * __restrict__ a, Dims4 da, const char * __restrict__ b, Dims4 db,
              char * __restrict__ dst, int64_t nbd1, int64_t nbd2, int64_t nbd3) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t M = da.ne[1], N = db.ne[1], K = da.ne[0];
    const int64_t m0 = ((int64_t) blockIdx.x * 2 + (warp & 1)) * TM;
    const int64_t n0 = ((int64_t) blockIdx.y * 2 + (warp >> 1)) * TN;
    if (m0 >= M || n0 >= N) return;
    const int64_t i12 = blockIdx.z % db.ne[2], i13 = blockIdx.z / db.ne[2];
    const int64_t i02 = i12 / (db.ne[2] / da.ne[2]), i03 = i13 / (db.ne[3] / da.ne[3]);
    const char * ap = a + i02 * da.nb[2] + i03 * da.nb[3];
    const char * bp = b + i12 * db.nb[2] + i13 * db.nb[3];

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    const int64_t np = K & ~(int64_t) 31;
    for (int64_t k0 = 0; k0 < np; k0 += 32) {
        unsigned short av[TM], bv[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int64_t m = m0 + i;
            av[i] = (m < M) ? *(const unsigned short *) (ap + m * da.nb[1] + (k0 + lane) * 2) : (unsigned short) 0;
        }
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int64_t n = n0 + j;
            if (n < N) {
                if (X_F16) bv[j] = *(const unsigned short *) (bp + n * db.nb[1] + (k0 + lane) * 2);
                else       bv[j] = __half_as_ushort(__float2half_rn(*(const float *) (bp + n * db.nb[1] + (k0 + lane) * 4)));
            } else {
                bv[j] = 0;
            }
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = fma_f16_f32(av[i], bv[j], acc[i][j]);
    }

#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            float v = acc[i][j];
            v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 16));   // sum0 += sum2 ; sum1 += sum3
            v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 8));    // sum0 += sum1
            v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 4));    // low half + high half
            v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 1));    // hadd
            v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 2));    // hadd
            acc[i][j] = v;
        }

    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int64_t m = m0 + i, n = n0 + j;
                if (m < M && n < N) {
                    double sumf = (double) acc[i][j];
                    for (int64_t k = np; k < K; ++k) {
                        const float x = __half2float(*(const __half *) (ap + m * da.nb[1] + k * 2));
                        const float y = X_F16 ? __half2float(*(const __half *) (bp + n * db.nb[1] + k * 2))
                                              : round_f16(*(const float *) (bp + n * db.nb[1] + k * 4));
                        sumf += (double) __fmul_rn(x, y);
                    }
                    *(float *) (dst + m * 4 + n * nbd1 + i12 * nbd2 + i13 * nbd3) = (float) sumf;
                }
            }
    }
}

extern "C" int b200_mul_mat_f16(const void * src0, const int64_t * ne0, const int64_t * nb0,
                                const void * src1, int src1_type, const int64_t * ne1, const int64_t * nb1,
                                float * dst, const int64_t * nbd, void * stream) {
    const Dims4 da = make_dims(ne0, nb0), db = make_dims(ne1, nb1);
    if (da.ne[0] != db.ne[0] || da.nb[0] != 2) return B200_ERR_ARG;
    if (src1_type == B200_TYPE_F32 ? db.nb[0] != 4 : db.nb[0] != 2) return B200_ERR_ARG;
    if (src1_type != B200_TYPE_F32 && src1_type != B200_TYPE_F16) return B200_ERR_ARG;
    if (da.ne[2] <= 0 || da.ne[3] <= 0 || db.ne[2] % da.ne[2] != 0 || db.ne[3] % da.ne[3] != 0) return B200_ERR_ARG;
    const int64_t M = da.ne[1], N = db.ne[1], batch = db.ne[2] * db.ne[3];
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (batch > 65535 || (N + 7) / 8 > 65535) return B200_ERR_ARG;
    const bool big = M >= 256 && N >= 256;
    const int t = big ? 8 : 4;
    dim3 grid((unsigned) ((M + 2 * t - 1) / (2 * t)), (unsigned) ((N + 2 * t - 1) / (2 * t)), (unsigned) batch);
#define B200_F16_GO(XF, T) k_mul_mat_f16<XF, T, T><<<grid, 128, 0, as_stream(stream)>>>((const char *) src0, da, (const char *) src1, db, (char *) dst, nbd[1], nbd[2], nbd[3])
    if (src1_type == B200_TYPE_F16) { if (big) B200_F16_GO(true, 8); else B200_F16_GO(true, 4); }
    else                            { if (big) B200_F16_GO(false, 8); else B200_F16_GO(false, 4); }
#undef B200_F16_GO
    B200_RETURN_LAST();
}

// dst f16 [IC*KW, OW]: element (iow, iic, ikw) = x[iic][iow*s0 + ikw*d0 - p0] rounded to f16, 0 outside
__global__ void k_im2col_1d_f16(const char * __restrict__ x, int64_t x_stride, int64_t IW, int64_t IC, int64_t KW,
                                int64_t OW, int s0, int p0, int d0, __half * __restrict__ dst) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t row = IC * KW;
    if (i >= row * OW) return;
    const int64_t iow = i / row, rem = i - iow * row;
    const int64_t iic = rem / KW, ikw = rem - iic * KW;
    const int64_t iiw = iow * s0 + ikw * d0 - p0;
    float v = 0.0f;
    if (iiw >= 0 && iiw < IW) v = *(const float *) (x + iic * x_stride + iiw * 4);
    dst[i] = __float2half_rn(v);
}

extern "C" int b200_im2col_1d_f16(const float * x, int64_t x_stride_bytes, int64_t IW, int64_t IC, int64_t KW,
                                  int64_t OW, int s0, int p0, int d0, void * dst, void * stream) {
    const int64_t n = IC * KW * OW;
    if (n <= 0) return 0;
    k_im2col_1d_f16<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>((const char *) x, x_stride_bytes, IW, IC, KW, OW, s0, p0, d0, (__half *) dst);
    B200_RETURN_LAST();
}
