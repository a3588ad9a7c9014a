// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <atomic>
#include <utility>
#include "b200_whisper.h"

extern std::atomic<int64_t> g_b200_launches;

#define B200_LAUNCHED() (g_b200_launches.fetch_add(1, std::memory_order_relaxed))
#define B200_RETURN_LAST() do { B200_LAUNCHED(); return (int) cudaGetLastError(); } while (0)

static inline cudaStream_t as_stream(void * s) { return (cudaStream_t) s; }

// Programmatic dependent launch for the chain of small kernels of a decode step.  A kernel launched through
// launch_chained may start (block scheduling, its own prologue, loads of weights) while its predecessor in the
// stream is still running; it calls chain_wait() before it touches anything the predecessor writes or reads, and
// every such kernel calls chain_release() first thing so that its own successor may be scheduled early.  Both are
// no-ops for a kernel launched the ordinary way.  B200_NO_PDL=1 turns the launch attribute off.
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait()    { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool b200_chained_launches(void);

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = b200_chained_launches() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// f32 -> f16 round-to-nearest-even -> f32, the F16C round trip of GGML_FP32_TO_FP16 / GGML_FP16_TO_FP32.
// The packed conversion (cvt.rn.f16x2.f32) is used on purpose: the scalar f32->f16 conversion issues to the
// quarter-rate conversion unit, which throttles the sequential F16 accumulation of the attention kernels.
__device__ __forceinline__ float round_f16(float x) { return __low2float(__floats2half2_rn(x, 0.0f)); }

struct Dims4 { int64_t ne[4]; int64_t nb[4]; };

static inline Dims4 make_dims(const int64_t * ne, const int64_t * nb) {
    Dims4 d;
    for (int i = 0; i < 4; ++i) { d.ne[i] = ne ? ne[i] : 1; d.nb[i] = nb ? nb[i] : 0; }
    return d;
}

// planes of a block-quantised tensor (see b200_whisper.h)
struct QPlanes {
    const uint8_t *  qs;   // 16 (Q5_0) or 32 (Q8_0) bytes per block
    const uint32_t * qh;   // Q5_0 only
    const __half *   d;
};

__host__ __device__ __forceinline__ QPlanes q_planes(int type, const void * base, int64_t nb_total) {
    QPlanes p;
    const uint8_t * b = (const uint8_t *) base;
    if (type == B200_TYPE_Q5_0) {
        p.qs = b;
        p.qh = (const uint32_t *) (b + 16 * nb_total);
        p.d  = (const __half *)   (b + 20 * nb_total);
    } else {
        p.qs = b;
        p.qh = nullptr;
        p.d  = (const __half *)   (b + 32 * nb_total);
    }
    return p;
}

// Q5_0: the four signed weights (q - 16) of AVX lane j (elements 4j..4j+3) packed as int8x4.
// qs_word = 32-bit word (j & 3) of the block's 16 nibble bytes.
__device__ __forceinline__ int q5_lane_word(uint32_t qs_word, uint32_t qh, int j) {
    const uint32_t nib  = (j < 4) ? (qs_word & 0x0F0F0F0Fu) : ((qs_word >> 4) & 0x0F0F0F0Fu);
    const uint32_t bits = (qh >> (4 * j)) & 0xFu;
    const uint32_t hi   = ((bits & 1u) << 4) | ((bits & 2u) << 11) | ((bits & 4u) << 18) | ((bits & 8u) << 25);
    return (int) __vsub4(nib | hi, 0x10101010u);
}
