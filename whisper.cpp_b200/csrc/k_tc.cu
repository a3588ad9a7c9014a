// Q5_0 / Q8_0 x Q8_0 matrix product for 9 or more columns on the fifth-generation tensor cores (tcgen05.mma with
// the accumulator in tensor memory), bit-identical to the reference CPU path (ggml_compute_forward_mul_mat,
// ggml/src/ggml-cpu/ggml-cpu.c:1266-1458, with ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_q8_0_q8_0, AVX2 variant,
// ggml/src/ggml-cpu/ggml-cpu-quants.c:3076-3100, 3869-3886).
//
// What the reference computes per output and 32-block b: eight lane sums S_j (exact integers, lane j = elements
// 4j..4j+3), then acc_j = fma(d_w * d_x, float(S_j), acc_j) block after block and hsum_float_8 at the end.  Only
// the float chain is order-bound.  The integer part is one tensor-core product per block with a FRESH accumulator:
//
//     D[m][(n, j)] = sum_k A[m][k] * B[(n, j)][k]          M = 128 weight rows, N = 32 columns x 8 lanes = 256
//
// A holds the block's 32 weights of 128 rows as f16 (integers -16..15 / -127..127, exact), B holds the block's
// quantised activations of 32 columns, each column as eight rows of which row j is non-zero only at k = 4j..4j+3.
// Products and 4-term sums of such integers are exact in the f32 accumulator, so D is float(S_j) itself.
// Tensor memory is used as a double-buffered mailbox (2 x 256 columns): while the tensor core forms block b + 1,
// eight epilogue warps read block b with tcgen05.ld and run the fma chain in registers (a thread owns one weight
// row, 16 columns, all eight lanes: 128 accumulators).
//
// Roles (512 threads, one CTA per SM, persistent over output tiles of 128 rows x 32 columns):
//   warps 0-3   converters: read the weight planes (16/32 bytes + scale per row and block, Q5_0 unpacked in
//               registers) and the int8 activations straight from global memory / L2 and write the two operand
//               tiles of a stage in the canonical no-swizzle K-major layout (8-row x 16-byte core matrices), plus
//               the block's scales; the zero part of B is written once at start and never touched again;
//   warps 4-11  epilogue (see above), final hsum_float_8 order, fused ADD / SCALE / GELU / F16-store steps;
//   warp  12    one thread issues the two K = 16 MMAs of a block; one tcgen05.commit per block publishes the
//               tensor-memory buffer, and the epilogue, having seen it, hands the operand stage back to the
//               converters (warps 13-15 only give their registers away).
// Registers: the kernel starts with 128 per thread (the whole register file); setmaxnreg moves them between the
// warpgroups - converters keep 80, the MMA warpgroup 40, the epilogue warps grow to 192.  A warpgroup can only grow
// by what the others of the same CTA have released: 128*80 + 256*192 + 128*40 = 64512 <= 512*128.
// All hand-offs are mbarriers; every wait is bounded (about one second; the clock is read only after thousands of failed
// polls), records a code in the status word and makes all roles leave through the common exit that frees tensor memory.
//
// Measured (1280 x 1280 x 1500): 134 us, against 87 us for the mma.sync form (k_mma.cu) and 139 us for dp4a.  A
// block-step costs about 1600 cycles here although its two MMAs take 256: every 32-block needs its own accumulator
// hand-off (commit -> mbarrier -> tcgen05.ld -> mbarrier), a chain of about a thousand cycles, and tensor memory holds
// only two blocks of a 128 x 32 tile.  Smaller tiles with four buffers were measured too (slower: the cost is per
// hand-off, not per column).  The plugin therefore uses this kernel only on request (GGML_B200_TC=1).
#include "b200_common.cuh"
#include <string.h>
#include <stdlib.h>
#include <stdio.h>

#define TC_BM      128
#define TC_BN      32
#define TC_NST     6
#define TC_SLOTS   (TC_NST + 4)           // scale slots: a slot lives from conversion until the epilogue has used it
#define TC_A_BYTES (128 * 32 * 2)
#define TC_B_BYTES (256 * 32 * 2)
#define TC_STAGE_BYTES (TC_A_BYTES + TC_B_BYTES)
#define TC_THREADS 512
#define TC_OFF_DW   (TC_NST * TC_STAGE_BYTES)
#define TC_OFF_DX   (TC_OFF_DW + TC_SLOTS * 128 * 4)
#define TC_OFF_BAR  (TC_OFF_DX + TC_SLOTS * 32 * 4)
#define TC_OFF_MISC (TC_OFF_BAR + (2 * TC_NST + 4) * 8)
#define TC_SMEM_BYTES (TC_OFF_MISC + 16)

struct TcEp {
    int n_steps;
    int kind[4];
    const float * ptr[4];
    int64_t stride_n[4];
    float scalar[4];
    int store_f16;
    const uint16_t * gelu_table;
};

// Per-column operands (decode steps of several whisper_states that share one pass over the weights): column n writes M
// values to dst[n] (f32, or f16 with store_f16) and epilogue step s adds add[s][n][m].
#define TC_MAX_COLS 64
struct TcCols { void * dst[TC_MAX_COLS]; const float * add[4][TC_MAX_COLS]; };

typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 tc_pk2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void tc_upk2(f32x2 v, float & lo, float & hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 tc_fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }

__device__ __forceinline__ unsigned long long tc_now_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }


__device__ long long g_tc_prof[6][128];      // timing experiment: per-step clock stamps of CTA 0 (first 128 steps)
extern "C" int b200_tc_prof_read(long long * out) { return (int) cudaMemcpyFromSymbol(out, g_tc_prof, sizeof(g_tc_prof)); }

__device__ __forceinline__ bool tc_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded mbarrier wait: false after about one second or when another role has already given up.  The clock is only
// looked at after many failed polls: reading it costs a few hundred cycles, which the ordinary hand-off (a barrier that
// is ready or becomes ready within microseconds) must not pay.
__device__ __forceinline__ bool tc_wait_slow(uint32_t bar, uint32_t parity, volatile int * abort_flag, int * status, int code) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (tc_try(bar, parity)) return true;
        if ((i & 255) == 255) {
            if (*abort_flag) return false;
            const unsigned long long t = tc_now_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull || i > (1u << 28)) { *abort_flag = 1; atomicCAS(status, 0, code); return false; }
        }
    }
}
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int * abort_flag, int * status, int code) {
#pragma unroll 1
    for (int i = 0; i < 2048; ++i) if (tc_try(bar, parity)) return true;
    return tc_wait_slow(bar, parity, abort_flag, status, code);
}
// The same for a whole warp: one lane polls (32 lanes polling the same barrier word only slow its arrivals down), the
// warp-level sync publishes what that lane acquired to the others.
__device__ __forceinline__ bool tc_wait_warp(uint32_t bar, uint32_t parity, volatile int * abort_flag, int * status, int code) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = tc_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void tc_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ float tc_ep_apply(const TcEp & ep, int64_t n, int64_t m, float v) {
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

// four bytes holding small unsigned integers u (< 256) -> two f16x2 registers holding u - bias, exactly:
// 0x6400 | u is the f16 number 1024 + u
__device__ __forceinline__ void tc_bytes_to_f16(uint32_t v, uint32_t bias_h2, uint32_t & lo, uint32_t & hi) {
    const uint32_t a = __byte_perm(v, 0x64646464u, 0x4140), b = __byte_perm(v, 0x64646464u, 0x4342);
    const __half2 ha = __hsub2(*(const __half2 *) &a, *(const __half2 *) &bias_h2);
    const __half2 hb = __hsub2(*(const __half2 *) &b, *(const __half2 *) &bias_h2);
    lo = *(const uint32_t *) &ha; hi = *(const uint32_t *) &hb;
}

// shared-memory matrix descriptor, no swizzle, K-major: core matrices of 8 rows x 16 bytes stored as 128 contiguous
// bytes; 128 bytes between core matrices along K, 512 bytes between 8-row groups
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t) ((smem_addr >> 4) & 0x3FFF) | ((uint64_t) (lbo >> 4) << 16) | ((uint64_t) (sbo >> 4) << 32) | ((uint64_t) 1 << 46);
}

template <int TYPE, bool COLS>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_mul_mat_tc(QPlanes w, int64_t M, int nbk, const int8_t * __restrict__ xq, const float * __restrict__ xd, int64_t N,
             void * __restrict__ dst, int64_t ldd, TcEp ep, const __grid_constant__ TcCols cols, int * status, int relaxed, uint32_t lbo, uint32_t sbo, int dbg) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_u = (uint32_t) __cvta_generic_to_shared(tc_smem);
    const uint32_t bar_full = smem_u + TC_OFF_BAR, bar_empty = bar_full + TC_NST * 8, bar_tfull = bar_empty + TC_NST * 8, bar_tempty = bar_tfull + 16;
    volatile int * abort_flag = (volatile int *) (tc_smem + TC_OFF_MISC + 4);
    uint32_t * tmem_slot = (uint32_t *) (tc_smem + TC_OFF_MISC);

    // ---- set-up ----
    for (int i = tid; i < TC_NST * TC_STAGE_BYTES / 16; i += TC_THREADS) ((uint4 *) tc_smem)[i] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        for (int s = 0; s < TC_NST; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_full + s * 8), "r"(4));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_empty + s * 8), "r"(1));
        }
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_tfull + b * 8), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_tempty + b * 8), "r"(8));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 12) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(smem_u + TC_OFF_MISC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the zeros are read by the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (int) ((M + TC_BM - 1) / TC_BM), tiles_n = (int) ((N + TC_BN - 1) / TC_BN);
    const int n_tiles = tiles_m * tiles_n;
    if ((dbg & 64) && blockIdx.x == 0 && tid == 128) g_tc_prof[0][0] = clock64();       // timing experiment: cycles of CTA 0

    if (warp < 4) {
        // ================= converters =================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
        const int row = tid;                        // A row of the tile
        const int bn = tid >> 2, bq = tid & 3;      // B: column of the tile, quarter of the block (lanes 2bq, 2bq + 1)
        const uint32_t a_off = (uint32_t) ((row >> 3) * 512 + (row & 7) * 16);
        const uint32_t b_off0 = (uint32_t) (TC_A_BYTES + bn * 512 + bq * 128 + (2 * bq) * 16);
        const uint32_t b_off1 = b_off0 + 16 + 8;
        uint32_t step = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            int64_t m = (int64_t) tm * TC_BM + row;      if (m > M - 1) m = M - 1;
            int64_t n = (int64_t) tn * TC_BN + bn;       if (n > N - 1) n = N - 1;
            const int64_t wblk = m * nbk;
            const uint8_t *  qs_p = w.qs + wblk * (TYPE == B200_TYPE_Q5_0 ? 16 : 32);
            const uint32_t * qh_p = TYPE == B200_TYPE_Q5_0 ? w.qh + wblk : nullptr;
            const __half *   dw_p = w.d + wblk;
            const int8_t *   x_p  = xq + n * (int64_t) nbk * 32 + bq * 8;
            const float *    dx_p = xd + n * nbk;
            // raw operands of the next block are fetched before the current one is converted
            uint4 r_qs0, r_qs1 = make_uint4(0, 0, 0, 0); uint32_t r_qh = 0; __half r_dw; uint2 r_x; float r_dx;
            auto fetch = [&](int b) {
                if (TYPE == B200_TYPE_Q5_0) { r_qs0 = __ldg((const uint4 *) (qs_p + (size_t) b * 16)); r_qh = __ldg(qh_p + b); }
                else { r_qs0 = __ldg((const uint4 *) (qs_p + (size_t) b * 32)); r_qs1 = __ldg((const uint4 *) (qs_p + (size_t) b * 32 + 16)); }
                r_dw = __ldg(dw_p + b);
                r_x  = __ldg((const uint2 *) (x_p + (size_t) b * 32));
                r_dx = __ldg(dx_p + b);
            };
            fetch(0);
            for (int b = 0; b < nbk; ++b, ++step) {
                const uint4 qs0 = r_qs0, qs1 = r_qs1; const uint32_t qh = r_qh; const __half dw = r_dw; const uint2 xv = r_x; const float dxv = r_dx;
                if (b + 1 < nbk) fetch(b + 1);
                const int st = step % TC_NST;
                const uint32_t it = step / TC_NST;
                if (!tc_wait_warp(bar_empty + st * 8, (it & 1) ^ 1, abort_flag, status, 1)) goto done;
                unsigned char * sA = tc_smem + (size_t) st * TC_STAGE_BYTES;
                uint32_t h[16];                                  // h[2e/2]: elements 2i, 2i+1 as f16x2
                if (TYPE == B200_TYPE_Q5_0) {
                    const uint32_t W[4] = {qs0.x, qs0.y, qs0.z, qs0.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t hl = (((qh >> (4 * i)) & 0xFu) * 0x02040810u) & 0x10101010u;
                        const uint32_t hh = (((qh >> (16 + 4 * i)) & 0xFu) * 0x02040810u) & 0x10101010u;
                        const uint32_t vlo = (W[i] & 0x0F0F0F0Fu) | hl, vhi = ((W[i] >> 4) & 0x0F0F0F0Fu) | hh;
                        tc_bytes_to_f16(vlo, 0x64106410u, h[2 * i], h[2 * i + 1]);              // elements 4i .. 4i+3 (minus 16)
                        tc_bytes_to_f16(vhi, 0x64106410u, h[8 + 2 * i], h[8 + 2 * i + 1]);      // elements 16+4i ..
                    }
                } else {
                    const uint32_t W[8] = {qs0.x, qs0.y, qs0.z, qs0.w, qs1.x, qs1.y, qs1.z, qs1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) tc_bytes_to_f16(W[i] ^ 0x80808080u, 0x64806480u, h[2 * i], h[2 * i + 1]);
                }
#pragma unroll
                for (int ki = 0; ki < 4; ++ki)
                    *(uint4 *) (sA + a_off + ki * 128) = make_uint4(h[4 * ki], h[4 * ki + 1], h[4 * ki + 2], h[4 * ki + 3]);
                {
                    uint32_t x0, x1, y0, y1;
                    tc_bytes_to_f16(xv.x ^ 0x80808080u, 0x64806480u, x0, x1);
                    tc_bytes_to_f16(xv.y ^ 0x80808080u, 0x64806480u, y0, y1);
                    *(uint2 *) (sA + b_off0) = make_uint2(x0, x1);
                    *(uint2 *) (sA + b_off1) = make_uint2(y0, y1);
                }
                const int slot = step % TC_SLOTS;
                ((float *) (tc_smem + TC_OFF_DW))[slot * 128 + row] = __half2float(dw);
                if (bq == 0) ((float *) (tc_smem + TC_OFF_DX))[slot * 32 + bn] = dxv;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) tc_arrive(bar_full + st * 8);
            }
        }
    } else if (warp >= 12) {
        // ================= MMA issue =================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 12 && lane == 0) {
            // instruction descriptor: f32 accumulate, f16 x f16, both K-major, N = 256, M = 128
            const uint32_t idesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
            uint32_t step = 0;
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                for (int b = 0; b < nbk; ++b, ++step) {
                    const int st = step % TC_NST;
                    const uint32_t it = step / TC_NST;
                    const int buf = step & 1;
                    if (!tc_wait(bar_full + st * 8, it & 1, abort_flag, status, 2)) goto done;
                    if (!tc_wait(bar_tempty + buf * 8, ((step >> 1) & 1) ^ 1, abort_flag, status, 3)) goto done;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u + (uint32_t) st * TC_STAGE_BYTES, b_addr = a_addr + TC_A_BYTES;
                    const uint64_t da = tc_desc(a_addr, lbo, sbo), db = tc_desc(b_addr, lbo, sbo);
                    const uint32_t d_tmem = tmem_base + (uint32_t) buf * 256;
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                 :: "r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(0) : "memory");
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                 :: "r"(d_tmem), "l"(da + (256 >> 4)), "l"(db + (256 >> 4)), "r"(idesc), "r"(1) : "memory");
                    // one commit per block: its arrival tells the epilogue that the lane sums are in tensor memory AND that the
                    // operand stage has been read; the epilogue passes the second fact on to the converters
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar_tfull + buf * 8) : "memory");
                }
            }
        }
    } else {
        // ================= epilogue =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
        const int g = (warp - 4) >> 2, quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t t_lane = (uint32_t) (quarter * 32) << 16;
        const float * dWs = (const float *) (tc_smem + TC_OFF_DW);
        const float * dXs = (const float *) (tc_smem + TC_OFF_DX);
        uint32_t step = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            f32x2 acc[16][4];              // [column][lane pair]
#pragma unroll
            for (int c = 0; c < 16; ++c)
#pragma unroll
                for (int p = 0; p < 4; ++p) acc[c][p] = 0ull;
            for (int b = 0; b < nbk; ++b, ++step) {
                const int buf = step & 1;
                if (!tc_wait_warp(bar_tfull + buf * 8, (step >> 1) & 1, abort_flag, status, 4)) goto done;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (warp == 4 && lane == 0) tc_arrive(bar_empty + (step % TC_NST) * 8);      // the MMAs of this block have read their stage
                const int slot = step % TC_SLOTS;
                const float dw = dWs[slot * 128 + row];
                const float * dxs = dXs + slot * 32 + g * 16;
                const uint32_t taddr = tmem_base + t_lane + (uint32_t) buf * 256 + (uint32_t) g * 128;
                uint32_t v0[16], v1[16];
#define TC_LD16(v, col) asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];" \
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), \
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]) : "r"(taddr + (col)) : "memory")
                // the loaded registers are valid only after the wait: they pass through it as in/out operands so that no use can
                // be scheduled ahead of it
#define TC_WAIT16(v) asm volatile("tcgen05.wait::ld.sync.aligned;" \
                    : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), \
                      "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]) :: "memory")
#define TC_FMA16(v, c0) do { \
                    const float2 dxp = *(const float2 *) &dxs[(c0)]; \
                    const float dd0 = __fmul_rn(dw, dxp.x), dd1 = __fmul_rn(dw, dxp.y); \
                    if (relaxed) {      /* measurement switch: one fma per block on the whole block sum, as a K = 32 MMA would give it */ \
                        float s0 = 0.0f, s1 = 0.0f; \
                        _Pragma("unroll") for (int j = 0; j < 8; ++j) { s0 += __uint_as_float(v[j]); s1 += __uint_as_float(v[8 + j]); } \
                        float lo, hi; \
                        tc_upk2(acc[(c0)][0], lo, hi);     acc[(c0)][0]     = tc_pk2(__fmaf_rn(dd0, s0, lo), hi); \
                        tc_upk2(acc[(c0) + 1][0], lo, hi); acc[(c0) + 1][0] = tc_pk2(__fmaf_rn(dd1, s1, lo), hi); \
                        break; \
                    } \
                    const f32x2 d0 = tc_pk2(dd0, dd0), d1 = tc_pk2(dd1, dd1); \
                    _Pragma("unroll") for (int p = 0; p < 4; ++p) { \
                        acc[(c0)][p]     = tc_fma2(d0, tc_pk2(__uint_as_float(v[2 * p]),     __uint_as_float(v[2 * p + 1])), acc[(c0)][p]); \
                        acc[(c0) + 1][p] = tc_fma2(d1, tc_pk2(__uint_as_float(v[8 + 2 * p]), __uint_as_float(v[8 + 2 * p + 1])), acc[(c0) + 1][p]); \
                    } } while (0)
                TC_LD16(v0, 0);
#pragma unroll
                for (int c = 0; c < 8; c += 2) {
                    TC_WAIT16(v0);
                    TC_LD16(v1, (c + 1) * 16);
                    TC_FMA16(v0, 2 * c);
                    TC_WAIT16(v1);
                    if (c + 2 < 8) TC_LD16(v0, (c + 2) * 16);
                    else {
                        // every tcgen05.ld of this buffer has completed: hand it back to the MMA warp
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) tc_arrive(bar_tempty + buf * 8);
                    }
                    TC_FMA16(v1, 2 * c + 2);
                }
            }
            // hsum_float_8: ((l0 + l4) + (l2 + l6)) + ((l1 + l5) + (l3 + l7)), then the fused steps and the store
            const int64_t m = (int64_t) tm * TC_BM + row;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                float l[8];
#pragma unroll
                for (int p = 0; p < 4; ++p) tc_upk2(acc[c][p], l[2 * p], l[2 * p + 1]);
                const float r0 = __fadd_rn(l[4], l[0]), r1 = __fadd_rn(l[5], l[1]), r2 = __fadd_rn(l[6], l[2]), r3 = __fadd_rn(l[7], l[3]);
                float v = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
                const int64_t n = (int64_t) tn * TC_BN + g * 16 + c;
                if (m < M && n < N) {
                    if (COLS) {
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            if (s < ep.n_steps) {
                                if (ep.kind[s] == B200_EP_ADD)        v = __fadd_rn(v, cols.add[s][n][m]);
                                else if (ep.kind[s] == B200_EP_SCALE) v = __fmul_rn(v, ep.scalar[s]);
                                else {
                                    if (v <= -10.0f)     v = 0.0f;
                                    else if (v < 10.0f)  v = __half2float(__ushort_as_half(ep.gelu_table[__half_as_ushort(__float2half_rn(v))]));
                                }
                            }
                        }
                        if (ep.store_f16) ((__half *) cols.dst[n])[m] = __float2half_rn(v);
                        else              ((float *) cols.dst[n])[m] = v;
                    } else {
                        v = tc_ep_apply(ep, n, m, v);
                        if (ep.store_f16) ((__half *) dst)[n * ldd + m] = __float2half_rn(v);
                        else              ((float *) dst)[n * ldd + m] = v;
                    }
                }
            }
        }
    }
done:
    if ((dbg & 64) && blockIdx.x == 0 && tid == 128) g_tc_prof[0][1] = clock64();
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 12) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem_base) : "memory");
    }
}

const uint16_t * b200_gelu_table_device(int * err);

// status word (device) that the kernels write when a wait runs out; one per device, allocated on first use
static int * tc_status_word(int * err) {
    static int * words[64] = {nullptr};
    static std::atomic<int> lock{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *err = B200_ERR_ARG; return nullptr; }
    if (words[dev]) return words[dev];
    while (lock.exchange(1)) {}
    if (!words[dev]) {
        int * p = nullptr;
        cudaError_t e = cudaMalloc(&p, sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(int));
        if (e != cudaSuccess) { *err = (int) e; lock = 0; return nullptr; }
        words[dev] = p;
    }
    lock = 0;
    return words[dev];
}

extern "C" int b200_mul_mat_tc_status(void) {
    int err = 0, v = 0;
    int * p = tc_status_word(&err);
    if (!p) return err;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return (int) cudaGetLastError();
    return v;
}

static int tc_launch(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K, const int8_t * xq, const float * xd, int64_t N,
                     void * dst, int64_t dst_stride, const TcEp & e, const TcCols * cols, void * stream) {
    int err = 0;
    int * status = tc_status_word(&err);
    if (!status) return err;
    static int n_sm[64] = {0};
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return B200_ERR_ARG;
    if (!attr_done[dev]) {
        cudaError_t ce = cudaFuncSetAttribute(k_mul_mat_tc<B200_TYPE_Q5_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (ce == cudaSuccess) ce = cudaFuncSetAttribute(k_mul_mat_tc<B200_TYPE_Q8_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (ce == cudaSuccess) ce = cudaFuncSetAttribute(k_mul_mat_tc<B200_TYPE_Q5_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (ce == cudaSuccess) ce = cudaFuncSetAttribute(k_mul_mat_tc<B200_TYPE_Q8_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
        if (ce != cudaSuccess) return (int) ce;
        attr_done[dev] = true;
    }
    const int64_t n_tiles = ((M + TC_BM - 1) / TC_BM) * ((N + TC_BN - 1) / TC_BN);
    const unsigned grid = (unsigned) (n_tiles < n_sm[dev] ? n_tiles : n_sm[dev]);
    const QPlanes w = q_planes(wtype, w_planes, nb_total);
    static const int relaxed = getenv("GGML_B200_RELAXED") != nullptr && atoi(getenv("GGML_B200_RELAXED")) != 0;
    // byte distance between core matrices along K (leading) and between 8-row groups (stride) in the operand tiles
    static const uint32_t lbo = getenv("B200_TC_LBO") ? (uint32_t) atoi(getenv("B200_TC_LBO")) : 128u;
    static const uint32_t sbo = getenv("B200_TC_SBO") ? (uint32_t) atoi(getenv("B200_TC_SBO")) : 512u;
    const int nbk = (int) (K / 32);
    static const int dbg = getenv("B200_TC_DBG") ? atoi(getenv("B200_TC_DBG")) : 0;      // timing experiments: 1 = no conversion, 2 = no epilogue
    cudaStream_t st = as_stream(stream);
    static const TcCols no_cols = {};
    const TcCols & ct = cols ? *cols : no_cols;
#define TC_GO(T, C) k_mul_mat_tc<T, C><<<grid, TC_THREADS, TC_SMEM_BYTES, st>>>(w, M, nbk, xq, xd, N, dst, dst_stride, e, ct, status, relaxed, lbo, sbo, dbg)
    if (wtype == B200_TYPE_Q5_0) { if (cols) TC_GO(B200_TYPE_Q5_0, true); else TC_GO(B200_TYPE_Q5_0, false); }
    else                         { if (cols) TC_GO(B200_TYPE_Q8_0, true); else TC_GO(B200_TYPE_Q8_0, false); }
#undef TC_GO
    B200_RETURN_LAST();
}

static int tc_check(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K, const int8_t * xq, const float * xd, int64_t N) {
    if (K % 32 != 0 || K <= 0 || M <= 0 || N <= 0) return B200_ERR_ARG;
    if (wtype != B200_TYPE_Q5_0 && wtype != B200_TYPE_Q8_0) return B200_ERR_ARG;
    if (!w_planes || !xq || !xd) return B200_ERR_ARG;
    if (((uintptr_t) xq & 15) != 0 || ((uintptr_t) w_planes & 15) != 0 || ((uintptr_t) xd & 3) != 0) return B200_ERR_ARG;
    const int64_t nbk = K / 32;
    if (M * nbk > nb_total || nbk > (1 << 20)) return B200_ERR_ARG;
    return 0;
}

extern "C" int b200_mul_mat_tc_ep(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                  const int8_t * xq, const float * xd, int64_t N,
                                  void * dst, int64_t dst_stride, const b200_epilogue * ep, void * stream) {
    int rc = tc_check(wtype, w_planes, nb_total, M, K, xq, xd, N);
    if (rc) return rc;
    if (!dst) return B200_ERR_ARG;
    TcEp e;
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
    return tc_launch(wtype, w_planes, nb_total, M, K, xq, xd, N, dst, dst_stride, e, nullptr, stream);
}

// Per-column form (the decode step of up to 64 whisper_states in one pass over the weights): cols[n].dst / cols[n].add as in
// b200_mul_mat_cols_q; the column table travels as a kernel parameter.
extern "C" int b200_mul_mat_tc_cols(int wtype, const void * w_planes, int64_t nb_total, int64_t M, int64_t K,
                                    const int8_t * xq, const float * xd, const b200_gemv_col * cols, int n_cols,
                                    const b200_gemv_ep * ep, void * stream) {
    int rc = tc_check(wtype, w_planes, nb_total, M, K, xq, xd, n_cols);
    if (rc) return rc;
    if (!cols || n_cols > TC_MAX_COLS) return B200_ERR_ARG;
    TcEp e;
    memset(&e, 0, sizeof(e));
    TcCols tc;
    memset(&tc, 0, sizeof(tc));
    if (ep) {
        if (ep->n_steps < 0 || ep->n_steps > 4) return B200_ERR_ARG;
        e.n_steps = ep->n_steps; e.store_f16 = ep->store_f16;
        for (int s = 0; s < ep->n_steps; ++s) {
            e.kind[s] = ep->kind[s]; e.scalar[s] = ep->scalar[s];
            if (e.kind[s] == B200_EP_GELU) {
                if (!e.gelu_table) { int err = 0; e.gelu_table = b200_gelu_table_device(&err); if (err) return err; }
            } else if (e.kind[s] != B200_EP_ADD && e.kind[s] != B200_EP_SCALE) return B200_ERR_ARG;
        }
    }
    for (int n = 0; n < n_cols; ++n) {
        if (!cols[n].dst) return B200_ERR_ARG;
        tc.dst[n] = cols[n].dst;
        for (int s = 0; s < e.n_steps; ++s) {
            if (e.kind[s] == B200_EP_ADD && !cols[n].add[s]) return B200_ERR_ARG;
            tc.add[s][n] = cols[n].add[s];
        }
    }
    return tc_launch(wtype, w_planes, nb_total, M, K, xq, xd, n_cols, nullptr, 0, e, &tc, stream);
}
