// Row-wise and element-wise operators: norm, add/mul with broadcast, scale, GELU (F16 table),
// cpy/dup/cont, get_rows (f16/f32 tables), concat.
#include "b200_common.cuh"
#include <mutex>

// ---- norm: one warp per row (ggml/src/ggml-cpu/ops.cpp:3109-3158) -----------------------------
// Sums are formed in double as in the reference; only their association differs, which moves the
// double result by ~1e-16 relative, far below the f32 rounding of mean and variance.
__global__ void __launch_bounds__(128)
k_norm(const char * __restrict__ x, char * __restrict__ y, int64_t ne00, int64_t ne01, int64_t ne02, int64_t nrows,
       int64_t nbx1, int64_t nbx2, int64_t nbx3, int64_t nby1, int64_t nby2, int64_t nby3, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t) blockIdx.x * 4 + warp;
    if (row >= nrows) return;
    const int64_t i3 = row / (ne01 * ne02), i2 = (row / ne01) % ne02, i1 = row % ne01;
    const float * xp = (const float *) (x + i1 * nbx1 + i2 * nbx2 + i3 * nbx3);
    float *       yp = (float *)       (y + i1 * nby1 + i2 * nby2 + i3 * nby3);

    double sum = 0.0;
    for (int64_t i = lane; i < ne00; i += 32) sum += (double) xp[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = (float) (sum / (double) ne00);

    double sum2 = 0.0;
    for (int64_t i = lane; i < ne00; i += 32) {
        const float v = __fadd_rn(xp[i], -mean);
        sum2 += (double) __fmul_rn(v, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
    const float variance = (float) (sum2 / (double) ne00);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
    for (int64_t i = lane; i < ne00; i += 32) yp[i] = __fmul_rn(__fadd_rn(xp[i], -mean), scale);
}

extern "C" int b200_norm(const float * x, float * y, int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                         const int64_t * nbx, const int64_t * nby, float eps, void * stream) {
    const int64_t nrows = ne01 * ne02 * ne03;
    if (nrows <= 0 || ne00 <= 0) return 0;
    k_norm<<<(unsigned) ((nrows + 3) / 4), 128, 0, as_stream(stream)>>>((const char *) x, (char *) y, ne00, ne01, ne02, nrows,
        nbx[1], nbx[2], nbx[3], nby[1], nby[2], nby[3], eps);
    B200_RETURN_LAST();
}

__global__ void __launch_bounds__(128)
k_layer_norm(const char * __restrict__ x, const float * __restrict__ gamma, const float * __restrict__ beta, char * __restrict__ y,
             int64_t ne00, int64_t nrows, int64_t xs, int64_t ys, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t) blockIdx.x * 4 + warp;
    if (row >= nrows) return;
    const float * xp = (const float *) (x + row * xs);
    float *       yp = (float *)       (y + row * ys);
    double sum = 0.0;
    for (int64_t i = lane; i < ne00; i += 32) sum += (double) xp[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = (float) (sum / (double) ne00);
    double sum2 = 0.0;
    for (int64_t i = lane; i < ne00; i += 32) {
        const float v = __fadd_rn(xp[i], -mean);
        sum2 += (double) __fmul_rn(v, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
    const float variance = (float) (sum2 / (double) ne00);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
    for (int64_t i = lane; i < ne00; i += 32) {
        const float t = __fmul_rn(__fadd_rn(xp[i], -mean), scale);
        yp[i] = __fadd_rn(__fmul_rn(t, gamma[i]), beta[i]);
    }
}

// few rows (decode): one CTA of 256 threads per row, row held in registers
struct LnRows { const float * x[64]; float * y[64]; };
__global__ void __launch_bounds__(256)
k_layer_norm_row(LnRows rows, const float * __restrict__ gamma, const float * __restrict__ beta, int ne00, float eps,
                 int8_t * __restrict__ xq, float * __restrict__ xd) {
    __shared__ double red[8];
    __shared__ float s_mean, s_scale;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    chain_release();
    chain_wait();
    const float * xp = rows.x[blockIdx.x];
    float *       yp = rows.y[blockIdx.x];
    float v[8];
    double sum = 0.0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        v[u] = i < ne00 ? xp[i] : 0.0f;
        if (i < ne00) sum += (double) v[u];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += red[w];
        s_mean = (float) (t / (double) ne00);
    }
    __syncthreads();
    const float mean = s_mean;
    double sum2 = 0.0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        v[u] = __fadd_rn(v[u], -mean);
        if (i < ne00) sum2 += (double) __fmul_rn(v[u], v[u]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
    if (lane == 0) red[warp] = sum2;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += red[w];
        const float variance = (float) (t / (double) ne00);
        s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
    }
    __syncthreads();
    const float scale = s_scale;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        float y = 0.0f;
        if (i < ne00) { y = __fadd_rn(__fmul_rn(__fmul_rn(v[u], scale), gamma[i]), beta[i]); yp[i] = y; }
        // optional second output: the row quantised as quantize_row_q8_0 does it (ne00 a multiple of 32: a warp holds one
        // 32-block per pass), in the layout of b200_quantize_cols, for the product that consumes this row next
        if (xq != nullptr && u * 256 + warp * 32 < ne00) {
            float amax = fabsf(y);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
            xq[(size_t) blockIdx.x * ne00 + i] = (int8_t) __float2int_rn(__fmul_rn(y, id));
            if (lane == 0) xd[(size_t) blockIdx.x * (ne00 >> 5) + (i >> 5)] = round_f16(__fdiv_rn(amax, 127.f));
        }
    }
}

extern "C" int b200_layer_norm(const float * x, const float * gamma, const float * beta, float * y, int64_t ne00, int64_t nrows,
                               int64_t x_row_stride_bytes, int64_t y_row_stride_bytes, float eps, void * stream) {
    if (nrows <= 0 || ne00 <= 0) return 0;
    if (nrows <= 64 && ne00 <= 2048) {
        LnRows r;
        for (int i = 0; i < (int) nrows; ++i) {
            r.x[i] = (const float *) ((const char *) x + i * x_row_stride_bytes);
            r.y[i] = (float *) ((char *) y + i * y_row_stride_bytes);
        }
        k_layer_norm_row<<<(unsigned) nrows, 256, 0, as_stream(stream)>>>(r, gamma, beta, (int) ne00, eps, nullptr, nullptr);
        B200_RETURN_LAST();
    }
    k_layer_norm<<<(unsigned) ((nrows + 3) / 4), 128, 0, as_stream(stream)>>>((const char *) x, gamma, beta, (char *) y, ne00, nrows,
        x_row_stride_bytes, y_row_stride_bytes, eps);
    B200_RETURN_LAST();
}

extern "C" int b200_layer_norm_rows(const b200_ln_row * rows, int n_rows, const float * gamma, const float * beta, int64_t ne00, float eps, void * stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > 64 || ne00 <= 0 || ne00 > 2048) return B200_ERR_ARG;
    LnRows r;
    for (int i = 0; i < n_rows; ++i) { r.x[i] = rows[i].x; r.y[i] = rows[i].y; }
    launch_chained(k_layer_norm_row, dim3((unsigned) n_rows), dim3(256), 0, as_stream(stream), r, gamma, beta, (int) ne00, eps, (int8_t *) nullptr, (float *) nullptr);
    B200_RETURN_LAST();
}

extern "C" int b200_layer_norm_rows_q(const b200_ln_row * rows, int n_rows, const float * gamma, const float * beta, int64_t ne00, float eps,
                                      int8_t * xq, float * xd, void * stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > 64 || ne00 <= 0 || ne00 > 2048 || ne00 % 32 != 0 || !xq || !xd) return B200_ERR_ARG;
    LnRows r;
    for (int i = 0; i < n_rows; ++i) { r.x[i] = rows[i].x; r.y[i] = rows[i].y; }
    launch_chained(k_layer_norm_row, dim3((unsigned) n_rows), dim3(256), 0, as_stream(stream), r, gamma, beta, (int) ne00, eps, xq, xd);
    B200_RETURN_LAST();
}

// ---- add / mul with broadcast ----------------------------------------------------------------
template <int OP>
__global__ void k_binary(const char * __restrict__ a, Dims4 da, const char * __restrict__ b, Dims4 db,
                         char * __restrict__ d, int64_t nbd0, int64_t nbd1, int64_t nbd2, int64_t nbd3, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t i0 = i % da.ne[0], t1 = i / da.ne[0];
    const int64_t i1 = t1 % da.ne[1], t2 = t1 / da.ne[1];
    const int64_t i2 = t2 % da.ne[2], i3 = t2 / da.ne[2];
    const float x = *(const float *) (a + i0 * da.nb[0] + i1 * da.nb[1] + i2 * da.nb[2] + i3 * da.nb[3]);
    const float y = *(const float *) (b + (i0 % db.ne[0]) * db.nb[0] + (i1 % db.ne[1]) * db.nb[1] +
                                          (i2 % db.ne[2]) * db.nb[2] + (i3 % db.ne[3]) * db.nb[3]);
    *(float *) (d + i0 * nbd0 + i1 * nbd1 + i2 * nbd2 + i3 * nbd3) = OP == 0 ? __fadd_rn(x, y) : __fmul_rn(x, y);
}

extern "C" int b200_binary(int op, const float * a, const int64_t * nea, const int64_t * nba,
                           const float * b, const int64_t * neb, const int64_t * nbb,
                           float * dst, const int64_t * nbd, void * stream) {
    const Dims4 da = make_dims(nea, nba), db = make_dims(neb, nbb);
    const int64_t n = da.ne[0] * da.ne[1] * da.ne[2] * da.ne[3];
    if (n <= 0) return 0;
    for (int i = 0; i < 4; ++i) if (db.ne[i] <= 0 || da.ne[i] % db.ne[i] != 0) return B200_ERR_ARG;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    if (op == 0)      k_binary<0><<<grid, 256, 0, as_stream(stream)>>>((const char *) a, da, (const char *) b, db, (char *) dst, nbd[0], nbd[1], nbd[2], nbd[3], n);
    else if (op == 1) k_binary<1><<<grid, 256, 0, as_stream(stream)>>>((const char *) a, da, (const char *) b, db, (char *) dst, nbd[0], nbd[1], nbd[2], nbd[3], n);
    else return B200_ERR_ARG;
    B200_RETURN_LAST();
}

// ---- scale -----------------------------------------------------------------------------------
__global__ void k_scale(const float * __restrict__ x, float * __restrict__ y, int64_t n, float s) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fmul_rn(x[i], s);
}
extern "C" int b200_scale(const float * x, float * y, int64_t n, float s, void * stream) {
    if (n <= 0) return 0;
    k_scale<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, y, n, s);
    B200_RETURN_LAST();
}

// ---- GELU through the F16 table ----------------------------------------------------------------
__device__ uint16_t g_gelu_table[1 << 16];
extern "C" void b200_build_gelu_table(uint16_t * table);

static int ensure_gelu_table() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int) e;
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64) return B200_ERR_ARG;
    if (done[dev]) return 0;
    static uint16_t host_table[1 << 16];
    static bool built = false;
    if (!built) { b200_build_gelu_table(host_table); built = true; }
    e = cudaMemcpyToSymbol(g_gelu_table, host_table, sizeof(host_table));
    if (e != cudaSuccess) return (int) e;
    done[dev] = true;
    return 0;
}

// device address of the table on the current device (for kernels of other translation units)
const uint16_t * b200_gelu_table_device(int * err) {
    *err = ensure_gelu_table();
    if (*err) return nullptr;
    void * p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_gelu_table);
    if (e != cudaSuccess) { *err = (int) e; return nullptr; }
    return (const uint16_t *) p;
}

__global__ void k_gelu(const float * __restrict__ x, float * __restrict__ y, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    float r;
    if (v <= -10.0f)      r = 0.0f;
    else if (v >= 10.0f)  r = v;
    else                  r = __half2float(__ushort_as_half(g_gelu_table[__half_as_ushort(__float2half_rn(v))]));
    y[i] = r;
}
extern "C" int b200_gelu(const float * x, float * y, int64_t n, void * stream) {
    if (n <= 0) return 0;
    const int e = ensure_gelu_table();
    if (e) return e;
    k_gelu<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, y, n);
    B200_RETURN_LAST();
}

// ---- cpy / dup / cont --------------------------------------------------------------------------
template <typename TS, typename TD> __device__ __forceinline__ TD cvt(TS v);
template <> __device__ __forceinline__ float  cvt<float, float>(float v)   { return v; }
template <> __device__ __forceinline__ __half cvt<float, __half>(float v)  { return __float2half_rn(v); }
template <> __device__ __forceinline__ __half cvt<__half, __half>(__half v){ return v; }
template <> __device__ __forceinline__ float  cvt<__half, float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ int    cvt<int, int>(int v)         { return v; }

template <typename TS, typename TD>
__global__ void k_cpy(const char * __restrict__ s, Dims4 ds, char * __restrict__ d, Dims4 dd, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t r = i;
    const int64_t s0 = r % ds.ne[0]; r /= ds.ne[0];
    const int64_t s1 = r % ds.ne[1]; r /= ds.ne[1];
    const int64_t s2 = r % ds.ne[2]; const int64_t s3 = r / ds.ne[2];
    r = i;
    const int64_t d0 = r % dd.ne[0]; r /= dd.ne[0];
    const int64_t d1 = r % dd.ne[1]; r /= dd.ne[1];
    const int64_t d2 = r % dd.ne[2]; const int64_t d3 = r / dd.ne[2];
    const TS v = *(const TS *) (s + s0 * ds.nb[0] + s1 * ds.nb[1] + s2 * ds.nb[2] + s3 * ds.nb[3]);
    *(TD *) (d + d0 * dd.nb[0] + d1 * dd.nb[1] + d2 * dd.nb[2] + d3 * dd.nb[3]) = cvt<TS, TD>(v);
}

extern "C" int b200_cpy(const void * src, int src_type, const int64_t * nes, const int64_t * nbs,
                        void * dst, int dst_type, const int64_t * ned, const int64_t * nbd, void * stream) {
    const Dims4 ds = make_dims(nes, nbs), dd = make_dims(ned, nbd);
    const int64_t n = ds.ne[0] * ds.ne[1] * ds.ne[2] * ds.ne[3];
    if (n != dd.ne[0] * dd.ne[1] * dd.ne[2] * dd.ne[3]) return B200_ERR_ARG;
    if (n <= 0) return 0;
    const unsigned grid = (unsigned) ((n + 255) / 256);
    cudaStream_t st = as_stream(stream);
    if      (src_type == B200_TYPE_F32 && dst_type == B200_TYPE_F32) k_cpy<float, float><<<grid, 256, 0, st>>>((const char *) src, ds, (char *) dst, dd, n);
    else if (src_type == B200_TYPE_F32 && dst_type == B200_TYPE_F16) k_cpy<float, __half><<<grid, 256, 0, st>>>((const char *) src, ds, (char *) dst, dd, n);
    else if (src_type == B200_TYPE_F16 && dst_type == B200_TYPE_F16) k_cpy<__half, __half><<<grid, 256, 0, st>>>((const char *) src, ds, (char *) dst, dd, n);
    else if (src_type == B200_TYPE_F16 && dst_type == B200_TYPE_F32) k_cpy<__half, float><<<grid, 256, 0, st>>>((const char *) src, ds, (char *) dst, dd, n);
    else if (src_type == B200_TYPE_I32 && dst_type == B200_TYPE_I32) k_cpy<int, int><<<grid, 256, 0, st>>>((const char *) src, ds, (char *) dst, dd, n);
    else return B200_ERR_ARG;
    B200_RETURN_LAST();
}

// ---- get_rows ------------------------------------------------------------------------------------
template <typename T>
__global__ void k_get_rows(const char * __restrict__ table, int64_t row_stride, int64_t ne00, const int32_t * __restrict__ ids,
                           int64_t n_ids, float * __restrict__ dst) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ne00 * n_ids) return;
    const int64_t r = i / ne00, c = i - r * ne00;
    dst[i] = cvt<T, float>(*(const T *) (table + (int64_t) ids[r] * row_stride + c * (int64_t) sizeof(T)));
}

int b200_get_rows_q_launch(int type, const void * table, int64_t nb_total, int64_t ne00, const int32_t * ids,
                           int64_t n_ids, float * dst, cudaStream_t st);

extern "C" int b200_get_rows(int type, const void * table, int64_t nb_total_or_row_stride, int64_t ne00,
                             const int32_t * ids, int64_t n_ids, float * dst, void * stream) {
    const int64_t n = ne00 * n_ids;
    if (n <= 0) return 0;
    cudaStream_t st = as_stream(stream);
    const unsigned grid = (unsigned) ((n + 255) / 256);
    if (type == B200_TYPE_Q5_0 || type == B200_TYPE_Q8_0) {
        if (ne00 % 32 != 0) return B200_ERR_ARG;
        return b200_get_rows_q_launch(type, table, nb_total_or_row_stride, ne00, ids, n_ids, dst, st);
    }
    if (type == B200_TYPE_F16)      k_get_rows<__half><<<grid, 256, 0, st>>>((const char *) table, nb_total_or_row_stride, ne00, ids, n_ids, dst);
    else if (type == B200_TYPE_F32) k_get_rows<float><<<grid, 256, 0, st>>>((const char *) table, nb_total_or_row_stride, ne00, ids, n_ids, dst);
    else return B200_ERR_ARG;
    B200_RETURN_LAST();
}

// ---- concat --------------------------------------------------------------------------------------
__global__ void k_concat(const char * __restrict__ a, Dims4 da, const char * __restrict__ b, Dims4 db,
                         char * __restrict__ d, Dims4 dd, int dim, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t idx[4];
    int64_t r = i;
    idx[0] = r % dd.ne[0]; r /= dd.ne[0];
    idx[1] = r % dd.ne[1]; r /= dd.ne[1];
    idx[2] = r % dd.ne[2]; idx[3] = r / dd.ne[2];
    float v;
    if (idx[dim] < da.ne[dim]) {
        v = *(const float *) (a + idx[0] * da.nb[0] + idx[1] * da.nb[1] + idx[2] * da.nb[2] + idx[3] * da.nb[3]);
    } else {
        int64_t jb[4] = {idx[0], idx[1], idx[2], idx[3]};
        jb[dim] -= da.ne[dim];
        v = *(const float *) (b + jb[0] * db.nb[0] + jb[1] * db.nb[1] + jb[2] * db.nb[2] + jb[3] * db.nb[3]);
    }
    *(float *) (d + idx[0] * dd.nb[0] + idx[1] * dd.nb[1] + idx[2] * dd.nb[2] + idx[3] * dd.nb[3]) = v;
}

extern "C" int b200_concat(const float * a, const int64_t * nea, const int64_t * nba,
                           const float * b, const int64_t * neb, const int64_t * nbb,
                           float * dst, const int64_t * ned, const int64_t * nbd, int dim, void * stream) {
    if (dim < 0 || dim > 3) return B200_ERR_ARG;
    const Dims4 da = make_dims(nea, nba), db = make_dims(neb, nbb), dd = make_dims(ned, nbd);
    const int64_t n = dd.ne[0] * dd.ne[1] * dd.ne[2] * dd.ne[3];
    if (n <= 0) return 0;
    k_concat<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(stream)>>>((const char *) a, da, (const char *) b, db, (char *) dst, dd, dim, n);
    B200_RETURN_LAST();
}

// ---- top-k of logits rows ------------------------------------------------------------------------
// The host sampler of whisper.cpp reads every row of logits back and scans it (whisper_process_logits /
// whisper_sample_token, src/whisper.cpp:5015-5430; greedy = first index of the maximum).  This kernel leaves, per
// row, the k largest values with their indices (ties: lower index first, as a forward scan with `>` finds them), the
// maximum and log(sum(exp(x - max))) + max, so that a caller that only needs those can skip the 200 KB row.
#define TOPK_THREADS 512
struct TopkRows { const float * row[64]; b200_topk_result * out[64]; };

__device__ __forceinline__ bool topk_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// One CTA per row, ONE pass over the row: every thread keeps the k best of its own elements (sorted, ties towards the
// lower index - a thread meets its indices in ascending order) and a running (max, sum of exp) pair; then k rounds of a
// block-wide arg-max over the threads' current heads pick the global winners, and the (max, sum) pairs are merged.
__global__ void __launch_bounds__(TOPK_THREADS)
k_topk_rows(TopkRows rows, int n, int k) {
    chain_release();
    chain_wait();
    __shared__ float  s_v[TOPK_THREADS / 32];
    __shared__ int    s_i[TOPK_THREADS / 32];
    __shared__ int    s_t[TOPK_THREADS / 32];
    __shared__ double s_d[TOPK_THREADS / 32];
    __shared__ float  s_m[TOPK_THREADS / 32];
    __shared__ int    win_t;
    __shared__ float  row_max;
    const float * x = rows.row[blockIdx.x];
    b200_topk_result * out = rows.out[blockIdx.x];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float bv[B200_TOPK_MAX];
    int   bi[B200_TOPK_MAX];
#pragma unroll
    for (int j = 0; j < B200_TOPK_MAX; ++j) { bv[j] = -INFINITY; bi[j] = 0x7fffffff; }
    float  m = -INFINITY;      // running maximum of this thread's elements
    float  se = 0.0f;          // sum of exp(x - m) over them (about a hundred terms per thread; the threads' sums are merged in double)
    float thr = -INFINITY;     // value of the k-th entry of the list once the list is full
    bool  thr_set = false;
    // eight loads in flight per thread (the pass is bound by load latency, not by bandwidth); the running sum takes every
    // element, the sorted list only the few that beat its last entry, in ascending index order
    for (int i = tid; i < n; i += 8 * TOPK_THREADS) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = (i + u * TOPK_THREADS < n) ? x[i + u * TOPK_THREADS] : 0.0f;
        unsigned cand = 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (i + u * TOPK_THREADS < n) {
                if (v[u] > m) { se = se * __expf(m - v[u]) + 1.0f; m = v[u]; }
                else if (v[u] == v[u]) se += __expf(v[u] - m);
                if (!thr_set || v[u] > thr) cand |= 1u << u;
            }
        }
        while (cand) {
            const int u = __ffs(cand) - 1;
            cand &= cand - 1;
            float cv = v[0];
#pragma unroll
            for (int t = 1; t < 8; ++t) if (u == t) cv = v[t];
            int ci = i + u * TOPK_THREADS;
            if (thr_set && !(cv > thr)) continue;              // an earlier candidate of these eight raised the bar
            // insertion into the sorted list (strictly greater moves ahead; an equal value with a higher index stays behind)
#pragma unroll
            for (int j = 0; j < B200_TOPK_MAX; ++j) {
                if (j < k && (bi[j] == 0x7fffffff || cv > bv[j])) {
                    const float tv = bv[j]; const int ti = bi[j];
                    bv[j] = cv; bi[j] = ci; cv = tv; ci = ti;
                }
                if (j == k - 1) { thr = bv[j]; thr_set = bi[j] != 0x7fffffff; }      // the list's last entry, without a dynamic index
            }
        }
    }
    // k rounds: the best head of all threads wins, its owner moves on to its next candidate
    int head = 0;
    for (int r = 0; r < k; ++r) {
        float cv = -INFINITY; int ci = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < B200_TOPK_MAX; ++j) if (j == head) { cv = bv[j]; ci = bi[j]; }
        if (head >= k) ci = 0x7fffffff;
        int ct = tid;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, cv, o);
            const int   oi = __shfl_xor_sync(0xffffffffu, ci, o);
            const int   ot = __shfl_xor_sync(0xffffffffu, ct, o);
            if (oi != 0x7fffffff && (ci == 0x7fffffff || topk_better(ov, oi, cv, ci))) { cv = ov; ci = oi; ct = ot; }
        }
        if (lane == 0) { s_v[warp] = cv; s_i[warp] = ci; s_t[warp] = ct; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < TOPK_THREADS / 32; ++w)
                if (s_i[w] != 0x7fffffff && (ci == 0x7fffffff || topk_better(s_v[w], s_i[w], cv, ci))) { cv = s_v[w]; ci = s_i[w]; ct = s_t[w]; }
            out->ids[r] = ci == 0x7fffffff ? -1 : ci;
            out->vals[r] = cv;
            if (r == 0) { row_max = cv; out->max = cv; }
            win_t = ci == 0x7fffffff ? -1 : ct;
        }
        __syncthreads();
        if (tid == win_t) ++head;
    }
    // log-sum-exp: merge the (max, sum) pairs around the row maximum
    const float mx = row_max;
    double s = (double) se * (double) __expf(m - mx);
    if (m == -INFINITY) s = 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) s_d[warp] = s;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < TOPK_THREADS / 32; ++w) s += s_d[w];
        out->logsumexp = (float) (log(s) + (double) mx);
        out->n = n; out->k = k;
    }
    (void) s_m;
}

extern "C" int b200_topk_rows(const float * const * rows, b200_topk_result * const * out, int n_rows, int64_t n, int k, void * stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > 64 || n <= 0 || n > 0x7ffffff0 || k < 1 || k > B200_TOPK_MAX || !rows || !out) return B200_ERR_ARG;
    TopkRows r;
    for (int i = 0; i < n_rows; ++i) {
        if (!rows[i] || !out[i]) return B200_ERR_ARG;
        r.row[i] = rows[i]; r.out[i] = out[i];
    }
    const cudaError_t e = launch_chained(k_topk_rows, dim3((unsigned) n_rows), dim3(TOPK_THREADS), 0, as_stream(stream), r, (int) n, k);
    if (e != cudaSuccess) return (int) e;
    B200_RETURN_LAST();
}
