"""The allocation-free product entry point (b200_mul_mat_q_static) against the ordinary one.

Callers that are not allowed to allocate device memory where they need the product - code living inside
another framework's memory plan, latency-critical hosts that cannot take the device-wide stall of
cudaMalloc/cudaFree, callbacks that only receive input and output pointers - use the variant whose scratch is
a fixed array inside the library.  It must give the same bits as b200_quantize_q8_0 + b200_mul_mat_q with
caller-provided scratch, also on a second call that finds the first call's leftovers in the array.
This file is collected last on purpose, so a run that stops at the first failure has already run every other
test; it also passes when run alone in a fresh process (the first call then performs the per-device set-up).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
i64, vp = C.c_int64, C.c_void_p


def ptr(t):
    return vp(t.data_ptr())


def reference_product(lib, wtype, d_planes, nb, M, K, dx, N):
    qs = torch.empty((N, K), dtype=torch.int8, device="cuda")
    d = torch.empty((N, K // 32), device="cuda")
    dst = torch.zeros((N, M), device="cuda")
    assert lib.b200_quantize_q8_0(ptr(dx), i64(N), i64(K), i64(K * 4), ptr(qs), ptr(d), None) == 0
    assert lib.b200_mul_mat_q(wtype, ptr(d_planes), i64(nb), i64(M), i64(K), ptr(qs), ptr(d), i64(N), ptr(dst), i64(M), None) == 0
    torch.cuda.synchronize()
    return dst.cpu().numpy()


@pytest.mark.parametrize("wtype", [6, 8])
def test_static_scratch_product_matches_twice_in_a_row(pkg, wtype):
    lib = pkg.kernels_lib()
    lib.b200_static_scratch_bytes.restype = C.c_int64
    assert torch.cuda.is_available()
    quant = pkg.synth.quantize_q5_0 if wtype == 6 else pkg.synth.quantize_q8_0
    rng = np.random.default_rng(100 + wtype)
    # second call is smaller than the first, so stale bytes of call one lie right behind what call two writes
    for M, K, N in ((192, 1280, 300), (130, 384, 37)):
        w = (rng.standard_normal((M, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((N, K)).astype(np.float32)
        blocks = quant(w)
        nb = M * K // 32
        planes = np.zeros(blocks.size, np.uint8)
        assert lib.b200_blocks_to_planes(wtype, blocks.ctypes.data_as(vp), planes.ctypes.data_as(vp), i64(nb), i64(0), i64(nb)) == 0
        d_planes, dx = torch.from_numpy(planes).cuda(), torch.from_numpy(x).cuda()
        want = reference_product(lib, wtype, d_planes, nb, M, K, dx, N)
        got = torch.zeros((N, M), device="cuda")
        rc = lib.b200_mul_mat_q_static(wtype, ptr(d_planes), i64(nb), i64(M), i64(K), ptr(dx), i64(K * 4), i64(N), ptr(got), i64(M), None)
        assert rc == 0
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_static_scratch_rejects_oversize(pkg):
    lib = pkg.kernels_lib()
    lib.b200_static_scratch_bytes.restype = C.c_int64
    cap = lib.b200_static_scratch_bytes()
    assert 1 << 20 <= cap <= 64 << 20
    K = 5120
    N = cap // K + 1                       # N*K alone already exceeds the array
    rc = lib.b200_mul_mat_q_static(6, None, i64(0), i64(64), i64(K), None, i64(K * 4), i64(N), None, i64(64), None)
    assert rc == 10003
