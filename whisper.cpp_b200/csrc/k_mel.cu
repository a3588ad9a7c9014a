// Log-mel front-end (src/whisper.cpp:3008-3271 of the reference) on the device.
//
// One CTA per 400-sample frame.  The reference's recursive radix-2 FFT bottoms out in sixteen
// 25-point table DFTs (400 -> 200 -> 100 -> 50 -> 25); here the same sums are formed in the same
// order - each DFT output is a sequential 25-term sum, each butterfly uses the reference's
// left-to-right float expression, no fused multiply-add (the reference file is compiled for baseline
// x86-64) - but all 400 DFT outputs / 200 butterflies of a level run in parallel.  The mel projection
// keeps the float groups of four and the double accumulator.  Window and twiddle tables are built on
// the host with libm, as the reference does.
#include "b200_common.cuh"
#include <math.h>
#include <mutex>
#include <vector>

#define MEL_N_FFT      400
#define MEL_HOP        160
#define MEL_N_BINS     201
#define MEL_CHUNK_PAD  (16000 * 30)

struct mel_tables { float sin_vals[MEL_N_FFT]; float cos_vals[MEL_N_FFT]; float hann[MEL_N_FFT]; };
__constant__ mel_tables c_mel;

static int ensure_mel_tables() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int) e;
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64) return B200_ERR_ARG;
    if (done[dev]) return 0;
    mel_tables t;
    for (int i = 0; i < MEL_N_FFT; i++) {
        double theta = (2 * M_PI * i) / MEL_N_FFT;
        t.sin_vals[i] = sinf(theta);
        t.cos_vals[i] = cosf(theta);
        t.hann[i] = 0.5 * (1.0 - cosf((2.0 * M_PI * i) / (MEL_N_FFT)));
    }
    e = cudaMemcpyToSymbol(c_mel, &t, sizeof(t));
    if (e != cudaSuccess) return (int) e;
    done[dev] = true;
    return 0;
}

// samples: padded signal (200 reflected + n + zeros); n_valid = n_samples + 200 (first index not backed by audio/reflection)
__global__ void __launch_bounds__(256)
k_mel_frames(const float * __restrict__ samples, int64_t n_valid, const float * __restrict__ filters, int n_mel,
             int n_len, float * __restrict__ mel) {
    __shared__ float x[MEL_N_FFT];
    __shared__ float2 A[MEL_N_FFT];
    __shared__ float2 B[MEL_N_FFT];
    __shared__ float pw[MEL_N_BINS + 3];
    const int i = blockIdx.x;                 // frame
    const int tid = threadIdx.x;
    const int64_t offset = (int64_t) i * MEL_HOP;

    for (int j = tid; j < MEL_N_FFT; j += blockDim.x)
        x[j] = (offset + j < n_valid) ? __fmul_rn(c_mel.hann[j], samples[offset + j]) : 0.0f;
    __syncthreads();

    // 16 leaf DFTs of 25 points: leaf o holds x[o + 16 m]; output (o, k) -> A[o*25 + k]
    for (int t = tid; t < MEL_N_FFT; t += blockDim.x) {
        const int o = t / 25, k = t - o * 25;
        float re = 0.0f, im = 0.0f;
        for (int m = 0; m < 25; ++m) {
            const int idx = (k * m * 16) % MEL_N_FFT;
            const float v = x[o + 16 * m];
            re = __fadd_rn(re, __fmul_rn(v, c_mel.cos_vals[idx]));
            im = __fadd_rn(im, -__fmul_rn(v, c_mel.sin_vals[idx]));     // im -= v*sin
        }
        A[t] = make_float2(re, im);
    }
    __syncthreads();

    // four combine levels; at level with half size h the even/odd leaves are o and o + leaves/2
    float2 * src = A;
    float2 * dst = B;
    int leaves = 16, h = 25;
    for (int level = 0; level < 4; ++level) {
        const int out_leaves = leaves / 2, N = 2 * h, step = MEL_N_FFT / N;
        for (int t = tid; t < out_leaves * h; t += blockDim.x) {
            const int o = t / h, k = t - o * h;
            const float2 ev = src[o * h + k];
            const float2 od = src[(o + out_leaves) * h + k];
            const float re = c_mel.cos_vals[k * step];
            const float im = -c_mel.sin_vals[k * step];
            float2 lo, hi;
            lo.x = __fadd_rn(__fadd_rn(ev.x, __fmul_rn(re, od.x)), -__fmul_rn(im, od.y));
            lo.y = __fadd_rn(__fadd_rn(ev.y, __fmul_rn(re, od.y)),  __fmul_rn(im, od.x));
            hi.x = __fadd_rn(__fadd_rn(ev.x, -__fmul_rn(re, od.x)),  __fmul_rn(im, od.y));
            hi.y = __fadd_rn(__fadd_rn(ev.y, -__fmul_rn(re, od.y)), -__fmul_rn(im, od.x));
            dst[o * N + k]     = lo;
            dst[o * N + k + h] = hi;
        }
        __syncthreads();
        float2 * tmp = src; src = dst; dst = tmp;
        leaves = out_leaves; h = N;
    }
    // src now holds the 400-point spectrum
    for (int j = tid; j < MEL_N_BINS; j += blockDim.x) {
        const float2 c = src[j];
        pw[j] = __fadd_rn(__fmul_rn(c.x, c.x), __fmul_rn(c.y, c.y));
    }
    __syncthreads();

    for (int j = tid; j < n_mel; j += blockDim.x) {
        const float * f = filters + (size_t) j * MEL_N_BINS;
        double sum = 0.0;
        int k = 0;
        for (k = 0; k < MEL_N_BINS - 3; k += 4) {
            float g = __fmul_rn(pw[k], f[k]);
            g = __fadd_rn(g, __fmul_rn(pw[k + 1], f[k + 1]));
            g = __fadd_rn(g, __fmul_rn(pw[k + 2], f[k + 2]));
            g = __fadd_rn(g, __fmul_rn(pw[k + 3], f[k + 3]));
            sum += (double) g;
        }
        for (; k < MEL_N_BINS; k++) sum += (double) __fmul_rn(pw[k], f[k]);
        sum = log10(fmax(sum, 1e-10));
        mel[(size_t) j * n_len + i] = (float) sum;
    }
}

__global__ void k_mel_fill(float * __restrict__ mel, int n_mel, int n_len, int first, float v) {
    const int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int w = n_len - first;
    if (w <= 0 || t >= (int64_t) n_mel * w) return;
    const int j = (int) (t / w), i = first + (int) (t - (int64_t) j * w);
    mel[(size_t) j * n_len + i] = v;
}

// monotone float <-> uint mapping so that atomicMax on the integer orders the floats
__device__ __forceinline__ unsigned f2ord(float f) { const unsigned u = __float_as_uint(f); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }
__device__ __forceinline__ float ord2f(unsigned u) { return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u); }

__global__ void k_mel_max(const float * __restrict__ mel, int64_t n, unsigned * __restrict__ out) {
    unsigned best = 0;
    for (int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (int64_t) gridDim.x * blockDim.x)
        best = max(best, f2ord(mel[t]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out, best);
}

__global__ void k_mel_normalize(float * __restrict__ mel, int64_t n, const unsigned * __restrict__ mx) {
    const int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const double mmax = (double) ord2f(*mx) - 8.0;
    float v = mel[t];
    if ((double) v < mmax) v = (float) mmax;
    mel[t] = (float) (((double) v + 4.0) / 4.0);
}

struct b200_mel_plan {
    int          device;
    int          n_mel;
    cudaStream_t stream;
    float *      d_filters;
    float *      d_samples;   int64_t cap_samples;
    float *      d_mel;       int64_t cap_mel;
    unsigned *   d_max;
    float *      h_pinned;    int64_t cap_pinned;    // staging for the padded signal and the result
};

extern "C" void * b200_mel_create(int device, const float * filters_host, int n_mel) {
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (ensure_mel_tables() != 0) return nullptr;
    b200_mel_plan * p = new b200_mel_plan();
    p->device = device; p->n_mel = n_mel;
    p->d_samples = nullptr; p->cap_samples = 0; p->d_mel = nullptr; p->cap_mel = 0; p->h_pinned = nullptr; p->cap_pinned = 0;
    bool ok = cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMalloc(&p->d_filters, sizeof(float) * n_mel * MEL_N_BINS) == cudaSuccess;
    ok = ok && cudaMalloc(&p->d_max, sizeof(unsigned)) == cudaSuccess;
    ok = ok && cudaMemcpy(p->d_filters, filters_host, sizeof(float) * n_mel * MEL_N_BINS, cudaMemcpyHostToDevice) == cudaSuccess;
    if (!ok) { cudaGetLastError(); delete p; return nullptr; }
    return p;
}

extern "C" void b200_mel_destroy(void * plan) {
    b200_mel_plan * p = (b200_mel_plan *) plan;
    if (!p) return;
    cudaSetDevice(p->device);
    cudaStreamSynchronize(p->stream);
    cudaFree(p->d_filters); cudaFree(p->d_samples); cudaFree(p->d_mel); cudaFree(p->d_max);
    if (p->h_pinned) cudaFreeHost(p->h_pinned);
    cudaStreamDestroy(p->stream);
    delete p;
}

// pcm_host -> out_host [n_mel][n_len]; returns 0 or an error code.  Synchronous.
extern "C" int b200_mel_compute(void * plan, const float * pcm_host, int64_t n_samples, float * out_host, int64_t out_capacity,
                                int * n_len_out, int * n_len_org_out) {
    b200_mel_plan * p = (b200_mel_plan *) plan;
    if (!p || n_samples < 201) return B200_ERR_ARG;
    cudaError_t e = cudaSetDevice(p->device);
    if (e != cudaSuccess) return (int) e;
    const int64_t pad2 = MEL_N_FFT / 2;
    const int64_t n_padded = n_samples + MEL_CHUNK_PAD + 2 * pad2;
    const int n_len = (int) ((n_padded - MEL_N_FFT) / MEL_HOP);
    const int n_len_org = 1 + (int) ((n_samples + pad2 - MEL_N_FFT) / MEL_HOP);
    const int64_t n_out = (int64_t) p->n_mel * n_len;
    if (n_len_out) *n_len_out = n_len;
    if (n_len_org_out) *n_len_org_out = n_len_org;
    if (out_capacity < n_out) return B200_ERR_ARG;
    const int64_t n_valid = n_samples + pad2;                    // frames beyond it see zeros
    const int64_t n_dev_samples = n_valid + MEL_N_FFT;           // what the kernels may touch
    if (p->cap_samples < n_dev_samples) {
        cudaFree(p->d_samples);
        if ((e = cudaMalloc(&p->d_samples, sizeof(float) * n_dev_samples)) != cudaSuccess) { p->cap_samples = 0; return (int) e; }
        p->cap_samples = n_dev_samples;
    }
    if (p->cap_mel < n_out) {
        cudaFree(p->d_mel);
        if ((e = cudaMalloc(&p->d_mel, sizeof(float) * n_out)) != cudaSuccess) { p->cap_mel = 0; return (int) e; }
        p->cap_mel = n_out;
    }
    const int64_t need_pinned = n_out > n_dev_samples ? n_out : n_dev_samples;
    if (p->cap_pinned < need_pinned) {
        if (p->h_pinned) cudaFreeHost(p->h_pinned);
        if ((e = cudaMallocHost(&p->h_pinned, sizeof(float) * need_pinned)) != cudaSuccess) { p->cap_pinned = 0; p->h_pinned = nullptr; return (int) e; }
        p->cap_pinned = need_pinned;
    }
    // padded signal: 200 reflected samples, the audio, zeros (whisper.cpp:3200-3212)
    for (int64_t i = 0; i < pad2; ++i) p->h_pinned[i] = pcm_host[pad2 - i];
    memcpy(p->h_pinned + pad2, pcm_host, sizeof(float) * n_samples);
    memset(p->h_pinned + pad2 + n_samples, 0, sizeof(float) * (n_dev_samples - pad2 - n_samples));
    cudaStream_t st = p->stream;
    cudaMemcpyAsync(p->d_samples, p->h_pinned, sizeof(float) * n_dev_samples, cudaMemcpyHostToDevice, st);
    cudaMemsetAsync(p->d_max, 0, sizeof(unsigned), st);
    int n_frames = (int) (n_valid / MEL_HOP) + 1;
    if (n_frames > n_len) n_frames = n_len;
    k_mel_frames<<<n_frames, 256, 0, st>>>(p->d_samples, n_valid, p->d_filters, p->n_mel, n_len, p->d_mel);
    B200_LAUNCHED();
    if (n_frames < n_len) {
        const int64_t n_fill = (int64_t) p->n_mel * (n_len - n_frames);
        k_mel_fill<<<(unsigned) ((n_fill + 255) / 256), 256, 0, st>>>(p->d_mel, p->n_mel, n_len, n_frames, (float) log10(1e-10));
        B200_LAUNCHED();
    }
    k_mel_max<<<148 * 4, 256, 0, st>>>(p->d_mel, n_out, p->d_max);
    B200_LAUNCHED();
    k_mel_normalize<<<(unsigned) ((n_out + 255) / 256), 256, 0, st>>>(p->d_mel, n_out, p->d_max);
    B200_LAUNCHED();
    cudaMemcpyAsync(p->h_pinned, p->d_mel, sizeof(float) * n_out, cudaMemcpyDeviceToHost, st);
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int) e;
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int) e;
    memcpy(out_host, p->h_pinned, sizeof(float) * n_out);
    return 0;
}

extern "C" int b200_log_mel(int device, const float * pcm_host, int64_t n_samples, const float * filters_host,
                            int n_mel, float * out_host, int64_t out_capacity, int * n_len, int * n_len_org) {
    void * plan = b200_mel_create(device, filters_host, n_mel);
    if (!plan) return B200_ERR_NO_DEVICE;
    const int e = b200_mel_compute(plan, pcm_host, n_samples, out_host, out_capacity, n_len, n_len_org);
    b200_mel_destroy(plan);
    return e;
}
