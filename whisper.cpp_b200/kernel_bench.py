#!/usr/bin/env python
"""Micro-benchmark of the decode- and encoder-shaped kernels through the C ABI (include/b200_whisper.h).

Shapes are those of Whisper large-v3 (d = 1280, 20 heads, 4d = 5120, vocabulary 51866, 1500 x 1536 encoder attention).
Every kernel is timed with CUDA events on the stream it is launched on, after warm-up; weight matrices are cycled
through ~200 MB of copies so that no launch finds its weights in L2.  torch only provides device memory and events.

    python whisper.cpp_b200/kernel_bench.py [n_columns]        # columns = decoder states that step together
"""
import ctypes as C
import os
import sys

import torch

import importlib.util  # noqa: E402


def load_pkg():
    """This file's own package, loaded by path (the directory name contains a dot)."""
    if "whisper_cpp_b200" not in sys.modules:
        pkg_dir = os.path.dirname(os.path.abspath(__file__))
        spec = importlib.util.spec_from_file_location("whisper_cpp_b200", os.path.join(pkg_dir, "__init__.py"),
                                                      submodule_search_locations=[pkg_dir])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["whisper_cpp_b200"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["whisper_cpp_b200"]


i64, vp = C.c_int64, C.c_void_p


class Col(C.Structure):
    _fields_ = [("x", vp), ("dst", vp), ("add", vp * 4)]


class Ep(C.Structure):
    _fields_ = [("n_steps", C.c_int), ("kind", C.c_int * 4), ("scalar", C.c_float * 4), ("store_f16", C.c_int)]


class Row(C.Structure):
    _fields_ = [("q", vp), ("k", vp), ("v", vp), ("mask", vp), ("dst", vp), ("n_kv", C.c_int64)]


class LnRow(C.Structure):
    _fields_ = [("x", vp), ("y", vp)]


def ptr(t):
    return vp(t.data_ptr())


def timeit(fn, iters=50):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000 / iters


def q5_planes(nb):
    p = torch.randint(0, 255, (nb * 22,), dtype=torch.uint8, device="cuda")
    p[20 * nb:] = (torch.rand(nb, device="cuda") * 0.01).to(torch.float16).view(torch.uint8)     # sane f16 scales
    return p


def main():
    K = load_pkg().kernels_lib()
    NC = int(sys.argv[1]) if len(sys.argv) > 1 else 32
    ep = Ep(0, (C.c_int * 4)(0, 0, 0, 0), (C.c_float * 4)(0, 0, 0, 0), 0)
    print(f"decode step, {NC} columns (decoder states in lock-step)")
    for (M, Kd, name) in [(1280, 1280, "d x d"), (5120, 1280, "mlp1"), (1280, 5120, "mlp2"), (51866, 1280, "logits")]:
        nb = M * Kd // 32
        ncopy = max(1, min(160, int(200e6 // (nb * 22))))
        planes = [q5_planes(nb) for _ in range(ncopy)]
        x, out = torch.randn((NC, Kd), device="cuda"), torch.zeros((NC, M), device="cuda")
        cols, xs = (Col * NC)(), (vp * NC)()
        for n in range(NC):
            cols[n].x, cols[n].dst, xs[n] = x[n].data_ptr(), out[n].data_ptr(), x[n].data_ptr()
        xq, xd = torch.empty((NC, Kd), dtype=torch.int8, device="cuda"), torch.empty((NC, Kd // 32), device="cuda")
        assert K.b200_quantize_cols(xs, NC, i64(Kd), ptr(xq), ptr(xd), None) == 0
        it = [0]
        cap = 16 if Kd > 2560 else 32

        def cols_q():
            p = planes[it[0] % ncopy]
            it[0] += 1
            for c0 in range(0, NC, cap):
                n = min(cap, NC - c0)
                assert K.b200_mul_mat_cols_q(6, ptr(p), i64(nb), i64(M), i64(Kd), vp(xq.data_ptr() + c0 * Kd), vp(xd.data_ptr() + c0 * (Kd // 32) * 4),
                                             C.byref(cols, c0 * C.sizeof(Col)), n, C.byref(ep), None) == 0

        t = timeit(cols_q)
        print(f"  mul_mat_cols_q {name:7s} M={M:6d} K={Kd:5d}: {t:8.1f} us   {nb * 22 / t / 1e3:7.1f} GB/s of weights")
        if NC >= 9:
            def tc():
                p = planes[it[0] % ncopy]
                it[0] += 1
                assert K.b200_mul_mat_tc_ep(6, ptr(p), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), i64(NC), ptr(out), i64(M), None, None) == 0
            t = timeit(tc)
            print(f"  mul_mat_tc     {name:7s} M={M:6d} K={Kd:5d}: {t:8.1f} us   {nb * 22 / t / 1e3:7.1f} GB/s of weights (tcgen05, {NC} columns)")
        print(f"  quantize_cols  K={Kd}: {timeit(lambda: K.b200_quantize_cols(xs, NC, i64(Kd), ptr(xq), ptr(xd), None)):.1f} us")
        if NC <= 8:
            def vec():
                p = planes[it[0] % ncopy]
                it[0] += 1
                assert K.b200_mul_mat_vec_q_cols(6, ptr(p), i64(nb), i64(M), i64(Kd), cols, NC, C.byref(ep), None) == 0
            t = timeit(vec)
            print(f"  mul_mat_vec_q_cols {name:7s}: {t:8.1f} us   {nb * 22 / t / 1e3:7.1f} GB/s of weights")
        del planes
    H, d = 20, 1280
    for n_kv in (1536, 120):
        rows, keep = (Row * NC)(), []
        for i in range(NC):
            q = torch.randn((H, 64), device="cuda")
            k, v = torch.randn((n_kv, H, 64), device="cuda").half(), torch.randn((n_kv, H, 64), device="cuda").half()
            o = torch.zeros((H, 64), device="cuda")
            keep += [q, k, v, o]
            rows[i].q, rows[i].k, rows[i].v, rows[i].dst, rows[i].n_kv, rows[i].mask = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), n_kv, None
        t = timeit(lambda: K.b200_flash_attn_decode_rows(rows, NC, i64(H), i64(256), i64(d * 2), i64(128), i64(d * 2), i64(128), C.c_float(0.35), None))
        print(f"  flash_attn_decode_rows n_kv={n_kv:5d}: {t:8.1f} us   {NC * n_kv * d * 2 * 2 / t / 1e3:7.1f} GB/s of K+V")
    x = torch.randn((NC, 1280), device="cuda")
    y, g, b = torch.zeros_like(x), torch.randn(1280, device="cuda"), torch.randn(1280, device="cuda")
    lr = (LnRow * NC)()
    for i in range(NC):
        lr[i].x, lr[i].y = x[i].data_ptr(), y[i].data_ptr()
    print(f"  layer_norm_rows: {timeit(lambda: K.b200_layer_norm_rows(lr, NC, ptr(g), ptr(b), i64(1280), C.c_float(1e-5), None)):.1f} us")

    print("encoder, one 30 s window (1500 columns)")
    for (M, Kd, N, name) in [(1280, 1280, 1500, "d x d"), (5120, 1280, 1500, "mlp1"), (1280, 5120, 1500, "mlp2")]:
        nb = M * Kd // 32
        p = q5_planes(nb)
        x, out = torch.randn((N, Kd), device="cuda"), torch.zeros((N, M), device="cuda")
        xq, xd = torch.empty((N, Kd), dtype=torch.int8, device="cuda"), torch.empty((N, Kd // 32), device="cuda")
        assert K.b200_quantize_q8_0(ptr(x), i64(N), i64(Kd), i64(Kd * 4), ptr(xq), ptr(xd), None) == 0
        t = timeit(lambda: K.b200_mul_mat_q(6, ptr(p), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), i64(N), ptr(out), i64(M), None), 10)
        print(f"  mul_mat_q {name:6s}: {t:8.1f} us   {2 * M * N * Kd / t / 1e6:7.2f} TFLOP/s")
        t = timeit(lambda: K.b200_mul_mat_tc_ep(6, ptr(p), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), i64(N), ptr(out), i64(M), None, None), 10)
        print(f"  mul_mat_tc {name:6s}: {t:7.1f} us   {2 * M * N * Kd / t / 1e6:7.2f} TFLOP/s  (tcgen05 + tensor memory)")
        wh, wd = torch.empty((nb, 16), dtype=torch.int32, device="cuda"), torch.empty(nb, device="cuda")
        xh, xdh = torch.empty((N * Kd // 32, 16), dtype=torch.int32, device="cuda"), torch.empty(N * Kd // 32, device="cuda")
        xf = torch.randn((N, Kd), device="cuda")
        assert K.b200_mma_pack_weights(6, ptr(p), i64(nb), ptr(wh), ptr(wd), None) == 0
        assert K.b200_mma_quantize(ptr(xf), i64(N), i64(Kd), i64(Kd * 4), ptr(xh), ptr(xdh), None) == 0
        t = timeit(lambda: K.b200_mul_mat_mma_ep(ptr(wh), ptr(wd), i64(M), i64(Kd), ptr(xh), ptr(xdh), i64(N), ptr(out), i64(M), None, None), 10)
        print(f"  mul_mat_mma {name:6s}: {t:6.1f} us   {2 * M * N * Kd / t / 1e6:7.2f} TFLOP/s")
        t = timeit(lambda: K.b200_mma_quantize(ptr(xf), i64(N), i64(Kd), i64(Kd * 4), ptr(xh), ptr(xdh), None), 10)
        print(f"  mma_quantize {name:6s}: {t:5.1f} us")
        print(f"  quantize_q8_0 [{N} x {Kd}]: {timeit(lambda: K.b200_quantize_q8_0(ptr(x), i64(N), i64(Kd), i64(Kd * 4), ptr(xq), ptr(xd), None), 10):.1f} us")
    n_q, n_kv = 1500, 1536
    q = torch.randn((n_q, H * 64), device="cuda")
    k, v = torch.randn((n_kv, H * 64), device="cuda").half(), torch.randn((n_kv, H * 64), device="cuda").half()
    o = torch.zeros((n_q, H, 64), device="cuda")
    t = timeit(lambda: K.b200_flash_attn_ext(ptr(q), i64(H * 256), i64(256), ptr(k), i64(H * 128), i64(128), ptr(v), i64(H * 128), i64(128), None, i64(0),
                                             ptr(o), i64(n_q), i64(n_kv), i64(H), C.c_float(0.125), None), 5)
    assert K.b200_mul_mat_tc_status() == 0, "a device-side wait of the tcgen05 product ran out"
    print(f"  flash_attn_ext 1500 x 1536 x 20 heads: {t:8.1f} us   {4 * 64 * n_q * n_kv * H / t / 1e6:7.2f} TFLOP/s")


if __name__ == "__main__":
    main()
