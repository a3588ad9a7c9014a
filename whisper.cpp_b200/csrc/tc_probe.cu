// Timing probes for the building blocks of the tcgen05 / tensor-memory product (k_tc.cu): how long do the primitives the
// pipeline is made of take on this GPU?  Stand-alone program, cycle counts by clock64 inside single CTAs.
//
//   tc_probe tmem      tcgen05.ld + wait::ld latency and tensor-memory read bandwidth for 1..16 warps
//   tc_probe barrier   mbarrier hand-off between two warps, tcgen05.commit latency, MMA + commit latency and issue rate
//   tc_probe barops    throughput of mbarrier arrive / test_wait operations issued by 1..16 warps
//   tc_probe skeleton  the pipeline skeleton (producer warps -> MMA thread -> consumer warps, two tensor-memory buffers)
//                      with three hand-off schemes, with and without consumer work
//
// Every wait in these probes is bounded by an iteration count.
#include <cstdio>
#include <cstdint>
#include <cstring>
#include <cuda_runtime.h>

namespace probe_tmem {
template <int X> __device__ __forceinline__ void ld_wait(uint32_t taddr, uint32_t & sink);
template <> __device__ __forceinline__ void ld_wait<16>(uint32_t taddr, uint32_t & sink) {
    uint32_t v[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v[0]), "+r"(v[15]) :: "memory");
    sink += v[0] + v[15];
}
template <> __device__ __forceinline__ void ld_wait<32>(uint32_t taddr, uint32_t & sink) {
    uint32_t v[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]),
          "=r"(v[16]),"=r"(v[17]),"=r"(v[18]),"=r"(v[19]),"=r"(v[20]),"=r"(v[21]),"=r"(v[22]),"=r"(v[23]),"=r"(v[24]),"=r"(v[25]),"=r"(v[26]),"=r"(v[27]),"=r"(v[28]),"=r"(v[29]),"=r"(v[30]),"=r"(v[31]) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v[0]), "+r"(v[31]) :: "memory");
    sink += v[0] + v[31];
}
template <> __device__ __forceinline__ void ld_wait<64>(uint32_t taddr, uint32_t & sink) {
    uint32_t v[64];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]),
          "=r"(v[16]),"=r"(v[17]),"=r"(v[18]),"=r"(v[19]),"=r"(v[20]),"=r"(v[21]),"=r"(v[22]),"=r"(v[23]),"=r"(v[24]),"=r"(v[25]),"=r"(v[26]),"=r"(v[27]),"=r"(v[28]),"=r"(v[29]),"=r"(v[30]),"=r"(v[31]),
          "=r"(v[32]),"=r"(v[33]),"=r"(v[34]),"=r"(v[35]),"=r"(v[36]),"=r"(v[37]),"=r"(v[38]),"=r"(v[39]),"=r"(v[40]),"=r"(v[41]),"=r"(v[42]),"=r"(v[43]),"=r"(v[44]),"=r"(v[45]),"=r"(v[46]),"=r"(v[47]),
          "=r"(v[48]),"=r"(v[49]),"=r"(v[50]),"=r"(v[51]),"=r"(v[52]),"=r"(v[53]),"=r"(v[54]),"=r"(v[55]),"=r"(v[56]),"=r"(v[57]),"=r"(v[58]),"=r"(v[59]),"=r"(v[60]),"=r"(v[61]),"=r"(v[62]),"=r"(v[63]) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v[0]), "+r"(v[63]) :: "memory");
    sink += v[0] + v[63];
}
template <int X>
__global__ void probe(long long * out, int iters, int n_warps_active) {
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"((uint32_t) __cvta_generic_to_shared(&slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t base = slot;
    uint32_t sink = 0;
    long long t0 = 0, t1 = 0;
    if (warp < n_warps_active) {
        const uint32_t taddr = base + ((uint32_t) ((warp & 3) * 32) << 16) + (uint32_t) ((warp >> 2) * X) % (512 - X);
        ld_wait<X>(taddr, sink);
        t0 = clock64();
        for (int i = 0; i < iters; ++i) ld_wait<X>(taddr, sink);
        t1 = clock64();
    }
    __syncthreads();
    if (threadIdx.x % 32 == 0 && warp < n_warps_active) out[blockIdx.x * 32 + warp] = (t1 - t0) + (sink == 0x12345 ? 1 : 0);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(base) : "memory");
}
template <int X> void run(int n_warps) {
    long long * d; cudaMalloc(&d, 32 * 8); cudaMemset(d, 0, 32 * 8);
    const int iters = 200;
    probe<X><<<1, 512>>>(d, iters, n_warps);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[32]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    long long mx = 0; for (int i = 0; i < n_warps; ++i) mx = h[i] > mx ? h[i] : mx;
    printf("x%-3d warps %2d: %6.1f clk per dependent ld+wait  (%s)  => %.0f B/clk/SM\n", X, n_warps, (double) mx / iters, cudaGetErrorString(e),
           (double) n_warps * 32 * X * 4 * iters / (double) mx);
    cudaFree(d);
}
static int run_all() {
    for (int w : {1, 4, 8, 12, 16}) { run<16>(w); run<32>(w); run<64>(w); }
    return 0;
}

}  // namespace probe_tmem

namespace probe_barrier {
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ bool test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
template <bool TEST> __device__ __forceinline__ bool waitb(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < (1 << 22); ++i) if (TEST ? test_wait(bar, parity) : try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }

// mode 0/1: ping-pong between warp 0 and warp 1 (lane 0 each) with try_wait / test_wait
// mode 2: commit with nothing outstanding, then wait;  mode 3: 2 MMAs (M128 N256 K16 f16) + commit, then wait; mode 4: 8 MMAs + commit
template <bool TEST>
__global__ void probe(long long * out, int iters, int mode) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b0 = (uint32_t) __cvta_generic_to_shared(&bars[0]), b1 = b0 + 8;
    for (int i = threadIdx.x; i < 49152 / 16; i += blockDim.x) ((uint4 *) smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(b0));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(b1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"((uint32_t) __cvta_generic_to_shared(&slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = slot;
    long long t0 = 0, t1 = 0;
    bool ok = true;
    if (mode <= 1) {
        if (warp == 0 && lane == 0) {
            t0 = clock64();
            for (int i = 0; i < iters && ok; ++i) { arrive(b0); ok = waitb<TEST>(b1, i & 1); }
            t1 = clock64();
        } else if (warp == 1 && lane == 0) {
            for (int i = 0; i < iters && ok; ++i) { ok = waitb<TEST>(b0, i & 1); arrive(b1); }
        }
    } else if (warp == 0 && lane == 0) {
        const uint32_t sa = (uint32_t) __cvta_generic_to_shared(smem);
        const uint64_t da = (uint64_t) ((sa >> 4) & 0x3FFF) | ((uint64_t) 8 << 16) | ((uint64_t) 32 << 32) | ((uint64_t) 1 << 46);
        const uint64_t db = (uint64_t) (((sa + 8192) >> 4) & 0x3FFF) | ((uint64_t) 8 << 16) | ((uint64_t) 32 << 32) | ((uint64_t) 1 << 46);
        const uint32_t idesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
        const int n_mma = mode == 2 ? 0 : (mode == 3 ? 2 : 8);
        if (mode >= 5) {   // mode 5: back-to-back commits (no MMA), mode 6: 2 MMA + commit back-to-back, mode 7: 2 MMA + 2 commits back-to-back; one wait at the end
            t0 = clock64();
            for (int i = 0; i < iters; ++i) {
                if (mode >= 6) for (int m = 0; m < 2; ++m)
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                 :: "r"(tmem + (uint32_t) (i & 1) * 256), "l"(da + (uint64_t) (m * 16)), "l"(db + (uint64_t) (m * 16)), "r"(idesc), "r"(m) : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(b1) : "memory");
                if (mode == 7) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(b1) : "memory");
            }
            long long tm = clock64();
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(b0) : "memory");
            ok = waitb<TEST>(b0, 0);
            t1 = clock64();
            out[1] = tm - t0;
        } else {
        t0 = clock64();
        for (int i = 0; i < iters && ok; ++i) {
            for (int m = 0; m < n_mma; ++m)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                             :: "r"(tmem + (uint32_t) (m & 1) * 256), "l"(da + (uint64_t) ((m & 1) * 16)), "l"(db + (uint64_t) ((m & 1) * 16)), "r"(idesc), "r"(m & 1) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(b0) : "memory");
            ok = waitb<TEST>(b0, i & 1);
        }
        t1 = clock64();
        }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) out[0] = ok ? (t1 - t0) : -1;
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
}
static int run_all() {
    long long * d; cudaMalloc(&d, 16);
    const int iters = 500;
    const char * names[] = {"ping-pong (2 hand-offs)", "ping-pong (2 hand-offs)", "commit (nothing outstanding) + wait", "2 MMA M128 N256 K16 + commit + wait", "8 MMA + commit + wait",
                            "commit back-to-back", "2 MMA + commit back-to-back", "2 MMA + 2 commits back-to-back"};
    for (int test = 0; test < 1; ++test)
        for (int mode = 0; mode < 8; ++mode) {
            if (mode == 1) continue;
            cudaFuncSetAttribute(probe<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152);
            cudaFuncSetAttribute(probe<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152);
            if (test) probe<true><<<1, 64, 49152>>>(d, iters, mode); else probe<false><<<1, 64, 49152>>>(d, iters, mode);
            cudaError_t e = cudaDeviceSynchronize();
            long long h[2] = {0, 0}; cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
            printf("%-9s %-40s: %8.1f clk per iteration, issue side %8.1f (%s)\n", test ? "test_wait" : "try_wait", names[mode], (double) h[0] / iters, mode >= 5 ? (double) h[1] / iters : 0.0, cudaGetErrorString(e));
        }
    return 0;
}

}  // namespace probe_barrier

namespace probe_barops {
__global__ void ops(long long * out, int iters, int n_warps, int mode) {
    __shared__ __align__(8) unsigned long long bars[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b0 = (uint32_t) __cvta_generic_to_shared(&bars[0]);
    if (threadIdx.x == 0) for (int i = 0; i < 32; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(b0 + i * 8));
    __syncthreads();
    long long t0 = clock64();
    uint32_t acc = 0;
    if (warp < n_warps && lane == 0) {
        const uint32_t bar = b0 + (mode & 1 ? 0 : warp * 8);       // mode bit 0: all warps on one barrier, else one barrier per warp
        for (int i = 0; i < iters; ++i) {
            if (mode & 2) {      // failing polls (phase never completes with parity we ask for... ask for the current, incomplete phase)
                uint32_t ok;
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(0) : "memory");
                acc += ok;
            } else {             // arrive (completes a phase each time: count 1) 
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
            }
        }
    }
    long long t1 = clock64();
    __syncthreads();
    if (threadIdx.x == 0) { out[0] = t1 - t0; out[1] = acc; }
}
static int run_all() {
    long long * d; cudaMalloc(&d, 16);
    const int iters = 2000;
    for (int mode : {0, 1, 2, 3})
        for (int nw : {1, 4, 8, 16}) {
            ops<<<1, 512>>>(d, iters, nw, mode);
            cudaDeviceSynchronize();
            long long h = 0; cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
            printf("%s, %s, %2d warps: %6.1f cycles per op per warp, %6.1f cycles per op overall\n", mode & 2 ? "test_wait (fails)" : "arrive", mode & 1 ? "one barrier" : "own barriers", nw,
                   (double) h / iters, (double) h / iters / nw);
        }
    return 0;
}

}  // namespace probe_barops

namespace probe_skeleton {
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ void waitb(uint32_t bar, uint32_t parity, int backoff) {
    for (int i = 0; i < (1 << 22); ++i) { if (try_wait(bar, parity)) return; if (backoff) __nanosleep(backoff); }
}
__device__ __forceinline__ void arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
#define NST 6
// scheme 0: every consumer warp polls tfull itself (lane 0), arrives tempty itself (count 8)
// scheme 1: one poller + bar.sync over all 256 consumer threads; every warp arrives tempty itself (count 8)
// scheme 2: one poller per consumer warpgroup (128 threads) + bar.sync inside the warpgroup; every warp arrives itself
// backoff: nanosleep between failed polls of consumers and producers (ns)
__global__ void __launch_bounds__(512, 1) skel(long long * out, int steps, int scheme, int backoff, int fma_iters) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bars[2 * NST + 4];
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b_full = (uint32_t) __cvta_generic_to_shared(&bars[0]), b_empty = b_full + NST * 8, b_tfull = b_empty + NST * 8, b_tempty = b_tfull + 16;
    for (int i = threadIdx.x; i < 6 * 24576 / 16; i += blockDim.x) ((uint4 *) smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" :: "r"(b_full + s * 8)); asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(b_empty + s * 8)); }
        for (int b = 0; b < 2; ++b) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(b_tfull + b * 8)); asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" :: "r"(b_tempty + b * 8)); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 12) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"((uint32_t) __cvta_generic_to_shared(&slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = slot;
    long long t0 = clock64();
    if (warp < 4) {
        for (int s = 0; s < steps; ++s) {
            const int st = s % NST; const uint32_t it = s / NST;
            if (lane == 0) waitb(b_empty + st * 8, (it & 1) ^ 1, backoff ? 200 : 0);
            __syncwarp();
            if (lane == 0) arrive(b_full + st * 8);
        }
    } else if (warp == 12) {
        if (lane == 0) {
            const uint32_t sa = (uint32_t) __cvta_generic_to_shared(smem);
            const uint32_t idesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
            for (int s = 0; s < steps; ++s) {
                const int st = s % NST; const uint32_t it = s / NST; const int buf = s & 1;
                waitb(b_full + st * 8, it & 1, 0);
                waitb(b_tempty + buf * 8, ((s >> 1) & 1) ^ 1, 0);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a = sa + st * 24576, b = a + 8192;
                const uint64_t da = (uint64_t) ((a >> 4) & 0x3FFF) | ((uint64_t) 8 << 16) | ((uint64_t) 32 << 32) | ((uint64_t) 1 << 46);
                const uint64_t db = (uint64_t) ((b >> 4) & 0x3FFF) | ((uint64_t) 8 << 16) | ((uint64_t) 32 << 32) | ((uint64_t) 1 << 46);
                for (int m = 0; m < 2; ++m)
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                 :: "r"(tmem + (uint32_t) buf * 256), "l"(da + (uint64_t) (m * 16)), "l"(db + (uint64_t) (m * 16)), "r"(idesc), "r"(m) : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(b_tfull + buf * 8) : "memory");
            }
        }
    } else if (warp >= 4 && warp < 12) {
        float acc[64];
        for (int i = 0; i < 64; ++i) acc[i] = (float) i;
        const int g = (warp - 4) >> 2;
        for (int s = 0; s < steps; ++s) {
            const int buf = s & 1;
            if (scheme == 0) {
                if (lane == 0) waitb(b_tfull + buf * 8, (s >> 1) & 1, backoff);
                __syncwarp();
            } else if (scheme == 1) {
                if (warp == 4 && lane == 0) waitb(b_tfull + buf * 8, (s >> 1) & 1, backoff);
                asm volatile("bar.sync 1, 256;" ::: "memory");
            } else {
                if ((warp & 3) == 0 && lane == 0) waitb(b_tfull + buf * 8, (s >> 1) & 1, backoff);
                if (g == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (warp == 4 && lane == 0) arrive(b_empty + (s % NST) * 8);
            const uint32_t taddr = tmem + ((uint32_t) ((warp & 3) * 32) << 16) + buf * 256 + g * 128;
            for (int c = 0; c < 8; ++c) {
                uint32_t v[16];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]) : "r"(taddr + c * 16) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v[0]),"+r"(v[1]),"+r"(v[2]),"+r"(v[3]),"+r"(v[4]),"+r"(v[5]),"+r"(v[6]),"+r"(v[7]),"+r"(v[8]),"+r"(v[9]),"+r"(v[10]),"+r"(v[11]),"+r"(v[12]),"+r"(v[13]),"+r"(v[14]),"+r"(v[15]) :: "memory");
                if (c == 7) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) arrive(b_tempty + buf * 8);
                }
                if (fma_iters) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[(c * 8 + i) & 63] = fmaf(1.0001f, __uint_as_float(v[i]), acc[(c * 8 + i) & 63]);
                }
            }
        }
        float sum = 0; for (int i = 0; i < 64; ++i) sum += acc[i];
        if (sum == 12345.678f) out[7] = 1;
    }
    long long t1 = clock64();
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 128) out[0] = t1 - t0;
    if (warp == 12) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
}
static int run_all() {
    long long * d; cudaMalloc(&d, 64);
    cudaFuncSetAttribute(skel, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * 24576);
    const int steps = 400;
    for (int fma : {0, 1})
        for (int scheme : {0, 1, 2})
            for (int backoff : {0, 32, 100}) {
                skel<<<1, 512, 6 * 24576>>>(d, steps, scheme, backoff, fma);
                cudaError_t e = cudaDeviceSynchronize();
                long long h = 0; cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
                printf("fma %d scheme %d backoff %3d ns: %7.1f cycles per step (%s)\n", fma, scheme, backoff, (double) h / steps, cudaGetErrorString(e));
            }
    return 0;
}

}  // namespace probe_skeleton


int main(int argc, char ** argv) {
    const char * what = argc > 1 ? argv[1] : "";
    if (!strcmp(what, "tmem"))     return probe_tmem::run_all();
    if (!strcmp(what, "barrier"))  return probe_barrier::run_all();
    if (!strcmp(what, "barops"))   return probe_barops::run_all();
    if (!strcmp(what, "skeleton")) return probe_skeleton::run_all();
    fprintf(stderr, "usage: tc_probe tmem | barrier | barops | skeleton\n");
    return 2;
}
