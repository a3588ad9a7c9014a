#!/usr/bin/env python
"""One small, self-contained case per hot kernel, for captures under a profiler (a few launches, a few hundred MB at most).

    python whisper.cpp_b200/profile_case.py tc [M K N]        # tcgen05 quantised product, default 1280 x 1280 x 1500
    python whisper.cpp_b200/profile_case.py tc_cols [M K N]   # the same kernel in its per-column (decode) form, default 64 columns
    python whisper.cpp_b200/profile_case.py mma [M K N]       # mma.sync quantised product (packed operands), default 1280 x 1280 x 1500
    python whisper.cpp_b200/profile_case.py fa_enc            # encoder attention 1500 x 1536 x 20 heads
    python whisper.cpp_b200/profile_case.py topk              # top-k side output of 64 logits rows
    python whisper.cpp_b200/profile_case.py conv              # the two F16 products of the large-v3 conv stem

Each case runs the kernel five times and prints the CUDA-event time of the last three launches.
"""
import ctypes as C
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from kernel_bench import Col, Ep, load_pkg, ptr, q5_planes  # noqa: E402

i64, vp = C.c_int64, C.c_void_p


def timed(fn, name):
    if os.environ.get("B200_PROFILE_WARM", "1") != "0":      # bring the clocks up first (skipped under a profiler)
        w = torch.empty(1 << 26, device="cuda")
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < 0.6:
            w.add_(1.0)
            torch.cuda.synchronize()
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(f"{name}: {e0.elapsed_time(e1) * 1000 / 3:.1f} us per launch")


def main():
    K = load_pkg().kernels_lib()
    case = sys.argv[1] if len(sys.argv) > 1 else "tc"
    dims = [int(a) for a in sys.argv[2:5]]
    if case in ("tc", "tc_cols"):
        M, Kd, N = dims if len(dims) == 3 else ((1280, 1280, 1500) if case == "tc" else (1280, 1280, 64))
        nb = M * Kd // 32
        p = q5_planes(nb)
        x, out = torch.randn((N, Kd), device="cuda"), torch.zeros((N, M), device="cuda")
        xq, xd = torch.empty((N, Kd), dtype=torch.int8, device="cuda"), torch.empty((N, Kd // 32), device="cuda")
        assert K.b200_quantize_q8_0(ptr(x), i64(N), i64(Kd), i64(Kd * 4), ptr(xq), ptr(xd), None) == 0
        if case == "tc":
            timed(lambda: K.b200_mul_mat_tc_ep(6, ptr(p), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), i64(N), ptr(out), i64(M), None, None),
                  f"mul_mat_tc {M} x {Kd} x {N}")
        else:
            cols = (Col * N)()
            for n in range(N):
                cols[n].x, cols[n].dst = x[n].data_ptr(), out[n].data_ptr()
            ep = Ep(0, (C.c_int * 4)(0, 0, 0, 0), (C.c_float * 4)(0, 0, 0, 0), 0)
            timed(lambda: K.b200_mul_mat_tc_cols(6, ptr(p), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), cols, N, C.byref(ep), None),
                  f"mul_mat_tc_cols {M} x {Kd} x {N} columns")
        assert K.b200_mul_mat_tc_status() == 0
    elif case == "mma":
        M, Kd, N = dims if len(dims) == 3 else (1280, 1280, 1500)
        nb = M * Kd // 32
        p = q5_planes(nb)
        x, out = torch.randn((N, Kd), device="cuda"), torch.zeros((N, M), device="cuda")
        wh, wd = torch.empty((nb, 16), dtype=torch.int32, device="cuda"), torch.empty(nb, device="cuda")
        xh, xdh = torch.empty((N * Kd // 32, 16), dtype=torch.int32, device="cuda"), torch.empty(N * Kd // 32, device="cuda")
        assert K.b200_mma_pack_weights(6, ptr(p), i64(nb), ptr(wh), ptr(wd), None) == 0
        assert K.b200_mma_quantize(ptr(x), i64(N), i64(Kd), i64(Kd * 4), ptr(xh), ptr(xdh), None) == 0
        timed(lambda: K.b200_mul_mat_mma_ep(ptr(wh), ptr(wd), i64(M), i64(Kd), ptr(xh), ptr(xdh), i64(N), ptr(out), i64(M), None, None),
              f"mul_mat_mma {M} x {Kd} x {N}")
    elif case == "fa_enc":
        H, n_q, n_kv = 20, 1500, 1536
        q = torch.randn((n_q, H * 64), device="cuda")
        k, v = torch.randn((n_kv, H * 64), device="cuda").half(), torch.randn((n_kv, H * 64), device="cuda").half()
        o = torch.zeros((n_q, H, 64), device="cuda")
        timed(lambda: K.b200_flash_attn_ext(ptr(q), i64(H * 256), i64(256), ptr(k), i64(H * 128), i64(128), ptr(v), i64(H * 128), i64(128), None, i64(0),
                                            ptr(o), i64(n_q), i64(n_kv), i64(H), C.c_float(0.125), None), "flash_attn_ext 1500 x 1536 x 20")
    elif case == "topk":
        n, rows_n = 51866, 64
        x = torch.randn((rows_n, n), device="cuda")
        out = torch.zeros((rows_n, 128), dtype=torch.uint8, device="cuda")
        rows = (vp * rows_n)(*[x[i].data_ptr() for i in range(rows_n)])
        outs = (vp * rows_n)(*[out[i].data_ptr() for i in range(rows_n)])
        timed(lambda: K.b200_topk_rows(rows, outs, rows_n, i64(n), 5, None), "topk_rows 64 x 51866, k = 5")
    elif case == "conv":
        def arr4(v):
            return (C.c_int64 * 4)(*v)
        for (M, N, Kd) in ((3000, 1280, 384), (1500, 1280, 3840)):
            a, b = torch.randn((M, Kd), device="cuda").half(), torch.randn((N, Kd), device="cuda").half()
            o = torch.zeros((N, M), device="cuda")
            timed(lambda: K.b200_mul_mat_f16(ptr(a), arr4([Kd, M, 1, 1]), arr4([2, Kd * 2, Kd * M * 2, Kd * M * 2]), ptr(b), 1, arr4([Kd, N, 1, 1]),
                                             arr4([2, Kd * 2, Kd * N * 2, Kd * N * 2]), ptr(o), arr4([4, M * 4, M * N * 4, M * N * 4]), None),
                  f"mul_mat_f16 {M} x {N} x {Kd} ({2 * M * N * Kd / 1e9:.1f} GFLOP)")
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main()
