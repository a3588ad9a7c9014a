"""Parity of the CUDA kernels called through the C ABI (include/b200_whisper.h) against the CPU restatement
(oracle/liboracle.so) on seeded inputs.  torch only provides device memory and the stream.  Bit-exact unless noted."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

i64, vp = C.c_int64, C.c_void_p


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return vp(t.data_ptr())


def arr4(v):
    return (i64 * 4)(*v)


def sync_ok(rc):
    assert rc == 0, f"kernel entry point returned {rc}"
    torch.cuda.synchronize()


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.fixture(scope="module")
def K(pkg):
    lib = pkg.kernels_lib()
    assert torch.cuda.is_available(), "these tests need the B200; the kernel library has no CPU path"
    return lib


def planes_of(lib, pkg, wtype, w):
    q = pkg.synth.quantize_q5_0 if wtype == 6 else pkg.synth.quantize_q8_0
    blocks = q(w)
    nb = blocks.shape[0] * blocks.shape[1]
    planes = np.zeros(blocks.size, np.uint8)
    assert lib.b200_blocks_to_planes(wtype, blocks.ctypes.data_as(vp), planes.ctypes.data_as(vp), i64(nb), i64(0), i64(nb)) == 0
    return blocks, planes, nb


@pytest.mark.parametrize("wtype", [6, 8])
def test_dequantize(K, pkg, wtype):
    blocks, planes, nb = planes_of(K, pkg, wtype, rnd(1, 16, 256, scale=0.02))
    d_planes, out = dev(planes), torch.empty(nb * 32, device="cuda")
    sync_ok(K.b200_dequantize(wtype, ptr(d_planes), i64(nb), i64(0), i64(nb), ptr(out), None))
    assert bits_equal(out.cpu().numpy(), O.dequantize(wtype, blocks))
    sync_ok(K.b200_dequantize(wtype, ptr(d_planes), i64(nb), i64(7), i64(3), ptr(out), None))   # ragged range
    assert bits_equal(out.cpu().numpy()[:96], O.dequantize(wtype, blocks).reshape(-1, 32)[7:10].reshape(-1))


def test_quantize_q8_0(K):
    x = rnd(2, 9, 384) * np.linspace(1e-4, 50, 9, dtype=np.float32)[:, None]
    x[3] = 0
    dx, qs, d = dev(x), torch.empty((9, 384), dtype=torch.int8, device="cuda"), torch.empty((9, 12), device="cuda")
    sync_ok(K.b200_quantize_q8_0(ptr(dx), i64(9), i64(384), i64(384 * 4), ptr(qs), ptr(d), None))
    rq, rd = O.quantize_row_q8_0(x)
    assert np.array_equal(qs.cpu().numpy().reshape(-1), rq) and bits_equal(d.cpu().numpy().reshape(-1), rd)


@pytest.mark.parametrize("wtype", [6, 8])
@pytest.mark.parametrize("Kd,M,N", [(384, 384, 1), (1280, 200, 8), (512, 130, 3), (384, 96, 40), (1280, 64, 33), (2048, 70, 9)])
def test_mul_mat_q_both_paths(K, pkg, wtype, Kd, M, N):
    w, x = rnd(3, M, Kd, scale=0.02), rnd(4, N, Kd)
    blocks, planes, nb = planes_of(K, pkg, wtype, w)
    ref = O.mul_mat_q(wtype, blocks, M, Kd, x)
    d_planes, dx, dst = dev(planes), dev(x), torch.zeros((N, M), device="cuda")
    if N <= 8:
        sync_ok(K.b200_mul_mat_vec_q(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(dx), i64(Kd * 4), i64(N), ptr(dst), i64(M), None))
        assert bits_equal(dst.cpu().numpy(), ref), "GEMV path"
    qs, d = torch.empty((N, Kd), dtype=torch.int8, device="cuda"), torch.empty((N, Kd // 32), device="cuda")
    sync_ok(K.b200_quantize_q8_0(ptr(dx), i64(N), i64(Kd), i64(Kd * 4), ptr(qs), ptr(d), None))
    dst.zero_()
    sync_ok(K.b200_mul_mat_q(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(dst), i64(M), None))
    assert bits_equal(dst.cpu().numpy(), ref), "GEMM path"


class EpStep(C.Structure):
    _fields_ = [("kind", C.c_int), ("ptr", vp), ("stride_n", i64), ("scalar", C.c_float)]


class Epilogue(C.Structure):
    _fields_ = [("n_steps", C.c_int), ("step", EpStep * 4), ("store_f16", C.c_int)]


@pytest.mark.parametrize("wtype", [6, 8])
@pytest.mark.parametrize("Kd,M,N", [(384, 96, 40), (1280, 130, 73), (512, 64, 72), (2048, 70, 9), (128, 200, 150)])
def test_mul_mat_mma_tensor_pipe_path(K, pkg, wtype, Kd, M, N):
    """f16-MMA product (packed operands) against the restatement, bit for bit, ragged M / N tiles included."""
    w, x = rnd(13, M, Kd, scale=0.02), rnd(14, N, Kd) * np.linspace(1e-3, 30, N, dtype=np.float32)[:, None]
    x[N // 2] = 0
    blocks, planes, nb = planes_of(K, pkg, wtype, w)
    ref = O.mul_mat_q(wtype, blocks, M, Kd, x)
    d_planes, dx, dst = dev(planes), dev(x), torch.zeros((N, M), device="cuda")
    wh, wd = torch.empty((nb, 16), dtype=torch.int32, device="cuda"), torch.empty(nb, device="cuda")
    xh, xd = torch.empty((N * Kd // 32, 16), dtype=torch.int32, device="cuda"), torch.empty(N * Kd // 32, device="cuda")
    sync_ok(K.b200_mma_pack_weights(wtype, ptr(d_planes), i64(nb), ptr(wh), ptr(wd), None))
    sync_ok(K.b200_mma_quantize(ptr(dx), i64(N), i64(Kd), i64(Kd * 4), ptr(xh), ptr(xd), None))
    sync_ok(K.b200_mul_mat_mma_ep(ptr(wh), ptr(wd), i64(M), i64(Kd), ptr(xh), ptr(xd), i64(N), ptr(dst), i64(M), None, None))
    assert bits_equal(dst.cpu().numpy(), ref)
    # epilogue: + bias (broadcast over columns), GELU table, + residual, stored as f32; same steps on the dp4a path
    bias, res = dev(rnd(15, M)), dev(rnd(16, N, M))
    ep = Epilogue()
    ep.n_steps = 3
    ep.step[0].kind, ep.step[0].ptr, ep.step[0].stride_n = 1, bias.data_ptr(), 0
    ep.step[1].kind = 3
    ep.step[2].kind, ep.step[2].ptr, ep.step[2].stride_n = 1, res.data_ptr(), M
    a, b = torch.zeros((N, M), device="cuda"), torch.zeros((N, M), device="cuda")
    sync_ok(K.b200_mul_mat_mma_ep(ptr(wh), ptr(wd), i64(M), i64(Kd), ptr(xh), ptr(xd), i64(N), ptr(a), i64(M), C.byref(ep), None))
    qs, d = torch.empty((N, Kd), dtype=torch.int8, device="cuda"), torch.empty((N, Kd // 32), device="cuda")
    sync_ok(K.b200_quantize_q8_0(ptr(dx), i64(N), i64(Kd), i64(Kd * 4), ptr(qs), ptr(d), None))
    sync_ok(K.b200_mul_mat_q_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(b), i64(M), C.byref(ep), None))
    assert bits_equal(a.cpu().numpy(), b.cpu().numpy())
    assert K.b200_mul_mat_mma_ep(ptr(wh), ptr(wd), i64(M), i64(96), ptr(xh), ptr(xd), i64(N), ptr(a), i64(M), None, None) != 0   # K % 128



@pytest.mark.parametrize("wtype", [6, 8])
@pytest.mark.parametrize("Kd,M,N", [(384, 96, 40), (1280, 130, 73), (512, 64, 72), (2048, 70, 9), (128, 200, 150), (32, 128, 32),
                                    (1280, 1280, 333), (5120, 257, 64)])
def test_mul_mat_tc_tcgen05_path(K, pkg, wtype, Kd, M, N):
    """tcgen05 / tensor-memory product (weights read as planes, Q5_0 unpacked in the shared-memory stage) against the
    restatement, bit for bit: ragged M / N tiles, one-block K, several tiles per CTA, and the fused epilogue steps."""
    w, x = rnd(23, M, Kd, scale=0.02), rnd(24, N, Kd) * np.linspace(1e-3, 30, N, dtype=np.float32)[:, None]
    x[N // 2] = 0
    blocks, planes, nb = planes_of(K, pkg, wtype, w)
    d_planes, dx, dst = dev(planes), dev(x), torch.zeros((N, M), device="cuda")
    qs, d = torch.empty((N, Kd), dtype=torch.int8, device="cuda"), torch.empty((N, Kd // 32), device="cuda")
    sync_ok(K.b200_quantize_q8_0(ptr(dx), i64(N), i64(Kd), i64(Kd * 4), ptr(qs), ptr(d), None))
    sync_ok(K.b200_mul_mat_tc_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(dst), i64(M), None, None))
    assert K.b200_mul_mat_tc_status() == 0, "a device-side wait ran out"
    if M * N * Kd <= 130 * 73 * 1280:
        ref = O.mul_mat_q(wtype, blocks, M, Kd, x)
    else:       # large cases: the dp4a kernel (itself checked against the restatement above) is the reference
        r = torch.zeros((N, M), device="cuda")
        sync_ok(K.b200_mul_mat_q(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(r), i64(M), None))
        ref = r.cpu().numpy()
    assert bits_equal(dst.cpu().numpy(), ref)
    bias, res = dev(rnd(25, M)), dev(rnd(26, N, M))
    ep = Epilogue()
    ep.n_steps = 3
    ep.step[0].kind, ep.step[0].ptr, ep.step[0].stride_n = 1, bias.data_ptr(), 0
    ep.step[1].kind = 3
    ep.step[2].kind, ep.step[2].ptr, ep.step[2].stride_n = 1, res.data_ptr(), M
    a, b = torch.zeros((N, M), device="cuda"), torch.zeros((N, M), device="cuda")
    sync_ok(K.b200_mul_mat_tc_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(a), i64(M), C.byref(ep), None))
    sync_ok(K.b200_mul_mat_q_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(b), i64(M), C.byref(ep), None))
    assert bits_equal(a.cpu().numpy(), b.cpu().numpy())
    # F16 store (the CPY into the K/V cache) with a scale step
    ep2 = Epilogue()
    ep2.n_steps, ep2.store_f16 = 1, 1
    ep2.step[0].kind, ep2.step[0].scalar = 2, 0.3535533845424652
    a16, b16 = torch.zeros((N, M), dtype=torch.float16, device="cuda"), torch.zeros((N, M), dtype=torch.float16, device="cuda")
    sync_ok(K.b200_mul_mat_tc_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(a16), i64(M), C.byref(ep2), None))
    sync_ok(K.b200_mul_mat_q_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(b16), i64(M), C.byref(ep2), None))
    assert np.array_equal(a16.cpu().numpy().view(np.uint16), b16.cpu().numpy().view(np.uint16))
    assert K.b200_mul_mat_tc_status() == 0
    assert K.b200_mul_mat_tc_ep(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd + 16), ptr(qs), ptr(d), i64(N), ptr(a), i64(M), None, None) != 0   # K % 32
    assert K.b200_mul_mat_tc_ep(wtype, None, i64(nb), i64(M), i64(Kd), ptr(qs), ptr(d), i64(N), ptr(a), i64(M), None, None) != 0            # NULL weights


def test_mul_mat_q_rejects_bad_arguments(K):
    assert K.b200_mul_mat_vec_q(6, None, i64(0), i64(4), i64(48), None, i64(0), i64(1), None, i64(4), None) != 0   # K % 32
    assert K.b200_mul_mat_vec_q(6, None, i64(0), i64(4), i64(64), None, i64(0), i64(9), None, i64(4), None) != 0   # N > 8
    assert K.b200_mul_mat_q(7, None, i64(0), i64(4), i64(64), None, None, i64(9), None, i64(4), None) != 0          # unknown type


@pytest.mark.parametrize("Kd,M,N", [(384, 50, 3), (240, 33, 20), (64, 8, 1)])
def test_mul_mat_f16(K, Kd, M, N):
    w, x = rnd(5, M, Kd, scale=0.02).astype(np.float16), rnd(6, N, Kd)
    dw, dx, dst = dev(w), dev(x), torch.zeros((N, M), device="cuda")
    sync_ok(K.b200_mul_mat_f16(ptr(dw), arr4([Kd, M, 1, 1]), arr4([2, Kd * 2, Kd * M * 2, Kd * M * 2]), ptr(dx), 0, arr4([Kd, N, 1, 1]),
                               arr4([4, Kd * 4, Kd * N * 4, Kd * N * 4]), ptr(dst), arr4([4, M * 4, M * N * 4, M * N * 4]), None))
    assert bits_equal(dst.cpu().numpy(), O.mul_mat_f16(w, x))


@pytest.mark.parametrize("n_q,n_kv,H,masked", [(1, 1536, 4, False), (3, 100, 2, True), (7, 33, 3, True), (2, 1, 1, False)])
def test_flash_attn_ext(K, n_q, n_kv, H, masked):
    d = 64 * H
    q, k, v = rnd(7, n_q, H, 64, scale=0.5), rnd(8, n_kv, H, 64, scale=0.5).astype(np.float16), rnd(9, n_kv, H, 64).astype(np.float16)
    mask = None
    if masked:
        mask = np.zeros((n_q, n_kv), np.float16)
        mask[np.random.default_rng(10).random((n_q, n_kv)) < 0.4] = -np.inf
        mask[:, 0] = 0
    dq, dk, dv, dst = dev(q), dev(k), dev(v), torch.zeros((n_q, H, 64), device="cuda")
    dm = dev(mask) if mask is not None else None
    sync_ok(K.b200_flash_attn_ext(ptr(dq), i64(d * 4), i64(64 * 4), ptr(dk), i64(d * 2), i64(128), ptr(dv), i64(d * 2), i64(128),
                                  ptr(dm) if dm is not None else None, i64(n_kv * 2), ptr(dst), i64(n_q), i64(n_kv), i64(H), C.c_float(0.125), None))
    assert bits_equal(dst.cpu().numpy(), O.flash_attn(q, k, v, mask, 0.125))


def test_norm_and_gelu(K):
    x = rnd(11, 37, 1280) * 2 + 0.3
    dx, dy = dev(x), torch.empty((37, 1280), device="cuda")
    nb = arr4([4, 1280 * 4, 1280 * 37 * 4, 1280 * 37 * 4])
    sync_ok(K.b200_norm(ptr(dx), ptr(dy), i64(1280), i64(37), i64(1), i64(1), nb, nb, C.c_float(1e-5), None))
    assert bits_equal(dy.cpu().numpy(), O.norm(x))
    g = np.concatenate([rnd(12, 5000) * 4, np.array([-10, 10, -10.5, 11, 0], np.float32)])
    dg, dgy = dev(g), torch.empty(g.size, device="cuda")
    sync_ok(K.b200_gelu(ptr(dg), ptr(dgy), i64(g.size), None))
    assert bits_equal(dgy.cpu().numpy(), O.gelu(g))


@pytest.mark.parametrize("mask_kind", [None, np.float32, np.float16])
def test_soft_max(K, mask_kind):
    x = rnd(13, 3, 5, 77, scale=2.0)
    mask = None
    if mask_kind is not None:
        mask = np.zeros((5, 77), np.float32)
        mask[np.random.default_rng(14).random((5, 77)) < 0.3] = -np.inf
        mask[:, 0] = 0
        mask = mask.astype(mask_kind)
    dx, dy = dev(x), torch.empty(x.shape, device="cuda")
    dm = dev(mask) if mask is not None else None
    mt = 0 if mask_kind in (None, np.float32) else 1
    sync_ok(K.b200_soft_max(ptr(dx), ptr(dm) if dm is not None else None, mt, i64(77 * (4 if mt == 0 else 2)), i64(5), ptr(dy), i64(77), i64(15), i64(5),
                            C.c_float(0.125), None))
    assert bits_equal(dy.cpu().numpy(), O.soft_max(x, mask, 0.125, 5))


@pytest.mark.parametrize("stride", [1, 2])
def test_im2col(K, stride):
    x = rnd(15, 80, 300)
    OW = (300 + 2 - 3) // stride + 1
    dx, dy = dev(x), torch.empty((OW, 240), dtype=torch.float16, device="cuda")
    sync_ok(K.b200_im2col_1d_f16(ptr(dx), i64(300 * 4), i64(300), i64(80), i64(3), i64(OW), stride, 1, 1, ptr(dy), None))
    assert bits_equal(dy.cpu().numpy(), O.im2col_1d(x, 3, stride))


def test_elementwise_and_copies(K, pkg):
    a, b = rnd(16, 7, 384), rnd(17, 1, 384)
    da, db, dd = dev(a), dev(b), torch.empty((7, 384), device="cuda")
    nba, nbb = arr4([4, 384 * 4, 384 * 7 * 4, 384 * 7 * 4]), arr4([4, 384 * 4, 384 * 4, 384 * 4])
    sync_ok(K.b200_binary(0, ptr(da), arr4([384, 7, 1, 1]), nba, ptr(db), arr4([384, 1, 1, 1]), nbb, ptr(dd), nba, None))
    assert bits_equal(dd.cpu().numpy(), a + b)
    sync_ok(K.b200_binary(1, ptr(da), arr4([384, 7, 1, 1]), nba, ptr(db), arr4([384, 1, 1, 1]), nbb, ptr(dd), nba, None))
    assert bits_equal(dd.cpu().numpy(), a * b)
    sync_ok(K.b200_scale(ptr(da), ptr(dd), i64(a.size), C.c_float(0.3535), None))
    assert bits_equal(dd.cpu().numpy(), a * np.float32(0.3535))
    # cont(transpose): src viewed as [7, 384] with swapped strides -> contiguous [7(fast), 384]
    dt = torch.empty((384, 7), device="cuda")
    sync_ok(K.b200_cpy(ptr(da), 0, arr4([7, 384, 1, 1]), arr4([384 * 4, 4, 7 * 384 * 4, 7 * 384 * 4]), ptr(dt), 0, arr4([7, 384, 1, 1]),
                       arr4([4, 7 * 4, 7 * 384 * 4, 7 * 384 * 4]), None))
    assert bits_equal(dt.cpu().numpy(), a.T)
    dh = torch.empty((7, 384), dtype=torch.float16, device="cuda")
    sync_ok(K.b200_cpy(ptr(da), 0, arr4([384, 7, 1, 1]), nba, ptr(dh), 1, arr4([384 * 7, 1, 1, 1]), arr4([2, 384 * 7 * 2, 384 * 7 * 2, 384 * 7 * 2]), None))
    assert bits_equal(dh.cpu().numpy(), a.astype(np.float16))
    # get_rows from a quantised table and an f32 table
    table = rnd(18, 50, 128, scale=0.02)
    ids = np.array([3, 49, 0, 3], np.int32)
    for wtype in (6, 8):
        blocks, planes, nb = planes_of(K, pkg, wtype, table)
        dp, di, dr = dev(planes), dev(ids), torch.empty((4, 128), device="cuda")
        sync_ok(K.b200_get_rows(wtype, ptr(dp), i64(nb), i64(128), ptr(di), i64(4), ptr(dr), None))
        assert bits_equal(dr.cpu().numpy(), O.dequantize(wtype, blocks).reshape(50, 128)[ids])
    dtab, di, dr = dev(table), dev(ids), torch.empty((4, 128), device="cuda")
    sync_ok(K.b200_get_rows(0, ptr(dtab), i64(128 * 4), i64(128), ptr(di), i64(4), ptr(dr), None))
    assert bits_equal(dr.cpu().numpy(), table[ids])
    # concat along dim 1
    x1, x2 = rnd(19, 3, 64), rnd(20, 5, 64)
    d1, d2, dc = dev(x1), dev(x2), torch.empty((8, 64), device="cuda")
    sync_ok(K.b200_concat(ptr(d1), arr4([64, 3, 1, 1]), arr4([4, 256, 768, 768]), ptr(d2), arr4([64, 5, 1, 1]), arr4([4, 256, 1280, 1280]),
                          ptr(dc), arr4([64, 8, 1, 1]), arr4([4, 256, 2048, 2048]), 1, None))
    assert bits_equal(dc.cpu().numpy(), np.concatenate([x1, x2], 0))


@pytest.mark.parametrize("n_mel,seconds", [(80, 1.0), (128, 30.0), (80, 11.0)])
def test_log_mel(K, pkg, n_mel, seconds):
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(21, seconds, n_tones=None, envelopes=True))
    filters = pkg.synth.mel_filterbank(n_mel)
    ref = O.log_mel(pcm, filters)
    out = np.empty_like(ref)
    nl, nlo = C.c_int(0), C.c_int(0)
    rc = K.b200_log_mel(0, pcm.ctypes.data_as(vp), i64(pcm.size), filters.ctypes.data_as(vp), n_mel, out.ctypes.data_as(vp), i64(out.size),
                        C.byref(nl), C.byref(nlo))
    assert rc == 0 and nl.value == ref.shape[1]
    mism = int((out.view(np.uint32) != ref.view(np.uint32)).sum())
    # log10 of the device maths library may differ from libm's in the last double bit; after rounding to float
    # that can flip an isolated value by one ulp.  Tolerance: at most 1e-5 of the values, each within 1 f32 ulp.
    assert mism <= max(1, out.size // 100000), f"{mism} of {out.size} mel values differ"
    assert np.abs(out - ref).max() <= 2.4e-7 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("wtype", [6, 8])
@pytest.mark.parametrize("Kd,M,N", [(1280, 200, 1), (384, 70, 2), (1280, 1280, 3), (512, 96, 7), (1280, 130, 16), (5120, 72, 13), (1280, 333, 32),
                                    (5120, 40, 5), (4096, 24, 8), (5120, 33, 12), (5120, 16, 16), (4096, 20, 21), (5120, 9, 24)])
def test_mul_mat_cols_q_scattered_columns(K, pkg, wtype, Kd, M, N):
    """Columns that live at unrelated addresses (as single-token steps of different decoder states do) are quantised
    together and multiplied in one launch; each column must equal the product computed for it alone."""
    w, x = rnd(30, M, Kd, scale=0.02), rnd(31, N, Kd)
    blocks, planes, nb = planes_of(K, pkg, wtype, w)
    ref = O.mul_mat_q(wtype, blocks, M, Kd, x)
    d_planes = dev(planes)
    big = torch.zeros((N, 3, Kd), device="cuda")            # columns spread out in memory
    big[:, 1, :] = dev(x)
    outs = torch.zeros((N, 2, M), device="cuda")
    bias = dev(rnd(32, M))

    class Col(C.Structure):
        _fields_ = [("x", vp), ("dst", vp), ("add", vp * 4)]

    class Ep(C.Structure):
        _fields_ = [("n_steps", C.c_int), ("kind", C.c_int * 4), ("scalar", C.c_float * 4), ("store_f16", C.c_int)]

    cols = (Col * N)()
    xs = (vp * N)()
    for n in range(N):
        cols[n].x = big[n, 1].data_ptr()
        cols[n].dst = outs[n, 1].data_ptr()
        cols[n].add[0] = bias.data_ptr()
        xs[n] = big[n, 1].data_ptr()
    ep = Ep(2, (C.c_int * 4)(1, 2, 0, 0), (C.c_float * 4)(0, 0.5, 0, 0), 0)     # + bias, then * 0.5
    xq = torch.empty((N, Kd), dtype=torch.int8, device="cuda")
    xd = torch.empty((N, Kd // 32), device="cuda")
    sync_ok(K.b200_quantize_cols(xs, N, i64(Kd), ptr(xq), ptr(xd), None))
    sync_ok(K.b200_mul_mat_cols_q(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), cols, N, C.byref(ep), None))
    want = (ref + bias.cpu().numpy()[None, :]) * np.float32(0.5)
    assert bits_equal(outs[:, 1].cpu().numpy(), want)
    if N <= 8:     # the f32-column entry point gives the same bits
        outs.zero_()
        sync_ok(K.b200_mul_mat_vec_q_cols(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), cols, N, C.byref(ep), None))
        assert bits_equal(outs[:, 1].cpu().numpy(), want)


@pytest.mark.parametrize("wtype", [6, 8])
@pytest.mark.parametrize("Kd,Ms,N", [(1280, (200, 200, 200), 16), (384, (96, 130, 64), 7), (512, (70, 33), 32)])
def test_mul_mat_cols_q_multi_shared_columns(K, pkg, wtype, Kd, Ms, N):
    """Several weight matrices on the same quantised columns in one launch (Q, K, V of a decoder layer): every job has its
    own outputs and epilogue (f32 + bias, f16 store, plain f32) and must equal the single-product entry point."""
    x = rnd(41, N, Kd)
    dx = dev(x)

    class Col(C.Structure):
        _fields_ = [("x", vp), ("dst", vp), ("add", vp * 4)]

    class Ep(C.Structure):
        _fields_ = [("n_steps", C.c_int), ("kind", C.c_int * 4), ("scalar", C.c_float * 4), ("store_f16", C.c_int)]

    xs = (vp * N)(*[dx[n].data_ptr() for n in range(N)])
    xq, xd = torch.empty((N, Kd), dtype=torch.int8, device="cuda"), torch.empty((N, Kd // 32), device="cuda")
    sync_ok(K.b200_quantize_cols(xs, N, i64(Kd), ptr(xq), ptr(xd), None))
    nj = len(Ms)
    eps = [Ep(1, (C.c_int * 4)(1, 0, 0, 0), (C.c_float * 4)(0, 0, 0, 0), 0), Ep(0, (C.c_int * 4)(), (C.c_float * 4)(), 1),
           Ep(1, (C.c_int * 4)(2, 0, 0, 0), (C.c_float * 4)(0.25, 0, 0, 0), 0)][:nj]
    keep, cols_l, planes_l, nbs, single = [], [], [], [], []
    for i, M in enumerate(Ms):
        blocks, planes, nb = planes_of(K, pkg, wtype, rnd(50 + i, M, Kd, scale=0.02))
        d_planes, bias = dev(planes), dev(rnd(60 + i, M))
        out_multi = torch.zeros((N, M), dtype=torch.float16 if eps[i].store_f16 else torch.float32, device="cuda")
        out_single = torch.zeros_like(out_multi)
        cm, cs = (Col * N)(), (Col * N)()
        for n in range(N):
            cm[n].dst, cs[n].dst = out_multi[n].data_ptr(), out_single[n].data_ptr()
            cm[n].add[0] = cs[n].add[0] = bias.data_ptr()
        sync_ok(K.b200_mul_mat_cols_q(wtype, ptr(d_planes), i64(nb), i64(M), i64(Kd), ptr(xq), ptr(xd), cs, N, C.byref(eps[i]), None))
        keep += [d_planes, bias, out_multi, out_single, cm, cs]
        cols_l.append(cm); planes_l.append(d_planes); nbs.append(nb); single.append((out_multi, out_single))
    wp = (vp * nj)(*[t.data_ptr() for t in planes_l])
    colp = (C.POINTER(Col) * nj)(*[C.cast(c, C.POINTER(Col)) for c in cols_l])
    epp = (C.POINTER(Ep) * nj)(*[C.pointer(e) for e in eps])
    sync_ok(K.b200_mul_mat_cols_q_multi(wtype, nj, wp, (i64 * nj)(*nbs), (i64 * nj)(*Ms), i64(Kd), ptr(xq), ptr(xd), colp, N, epp, None))
    for i, (a, b) in enumerate(single):
        assert bits_equal(a.cpu().numpy(), b.cpu().numpy()), f"job {i}"
        assert np.abs(b.float().cpu().numpy()).max() > 0


def test_decode_rows_attention_and_layer_norm_rows(K):
    """Row-descriptor entry points: every row has its own buffers and key count."""
    H, d = 3, 192
    rng = np.random.default_rng(33)

    class Row(C.Structure):
        _fields_ = [("q", vp), ("k", vp), ("v", vp), ("mask", vp), ("dst", vp), ("n_kv", C.c_int64)]

    rows = (Row * 3)()
    keep, want = [], []
    for i, n_kv in enumerate((37, 1536, 5)):
        q = (rng.standard_normal((H, 64)) * 0.5).astype(np.float32)
        k = (rng.standard_normal((n_kv, H, 64)) * 0.5).astype(np.float16)
        v = rng.standard_normal((n_kv, H, 64)).astype(np.float16)
        mask = None
        if i == 0:
            mask = np.zeros((1, n_kv), np.float16)
            mask[0, rng.random(n_kv) < 0.4] = -np.inf
            mask[0, 0] = 0
        dq, dk, dv, dd = dev(q), dev(k), dev(v), torch.zeros((H, 64), device="cuda")
        dm = dev(mask) if mask is not None else None
        keep += [dq, dk, dv, dd, dm]
        rows[i].q, rows[i].k, rows[i].v, rows[i].dst, rows[i].n_kv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dd.data_ptr(), n_kv
        rows[i].mask = dm.data_ptr() if dm is not None else None
        want.append(O.flash_attn(q[None], k, v, mask, 0.125)[0])
    sync_ok(K.b200_flash_attn_decode_rows(rows, 3, i64(H), i64(64 * 4), i64(d * 2), i64(128), i64(d * 2), i64(128), C.c_float(0.125), None))
    for i in range(3):
        assert bits_equal(keep[5 * i + 3].cpu().numpy(), want[i]), f"row {i}"
    # the variant that also leaves the rows quantised (layout of b200_quantize_cols) for the projection that follows
    xq, xd = torch.zeros((3, H * 64), dtype=torch.int8, device="cuda"), torch.zeros((3, H * 2), device="cuda")
    for i in range(3):
        keep[5 * i + 3].zero_()
    sync_ok(K.b200_flash_attn_decode_rows_q(rows, 3, i64(H), i64(64 * 4), i64(d * 2), i64(128), i64(d * 2), i64(128), C.c_float(0.125),
                                            ptr(xq), ptr(xd), None))
    for i in range(3):
        assert bits_equal(keep[5 * i + 3].cpu().numpy(), want[i]), f"row {i} (quantising variant)"
    rq, rd = O.quantize_row_q8_0(np.stack([w_.reshape(-1) for w_ in want]))
    assert np.array_equal(xq.cpu().numpy().reshape(-1), rq) and bits_equal(xd.cpu().numpy().reshape(-1), rd)

    class LnRow(C.Structure):
        _fields_ = [("x", vp), ("y", vp)]

    x = rnd(34, 5, 1280) * 2 + 0.1
    gamma, beta = rnd(35, 1280), rnd(36, 1280)
    dx, dy, dg, db = dev(x), torch.zeros((5, 1280), device="cuda"), dev(gamma), dev(beta)
    lr = (LnRow * 5)()
    for i in range(5):
        lr[i].x, lr[i].y = dx[i].data_ptr(), dy[4 - i].data_ptr()
    sync_ok(K.b200_layer_norm_rows(lr, 5, ptr(dg), ptr(db), i64(1280), C.c_float(1e-5), None))
    assert bits_equal(dy.cpu().numpy()[::-1], O.norm(x) * gamma + beta)
    # the variant that also leaves the rows quantised (layout of b200_quantize_cols) for the product that follows
    dy2 = torch.zeros((5, 1280), device="cuda")
    for i in range(5):
        lr[i].y = dy2[4 - i].data_ptr()
    xq, xd = torch.zeros((5, 1280), dtype=torch.int8, device="cuda"), torch.zeros((5, 40), device="cuda")
    sync_ok(K.b200_layer_norm_rows_q(lr, 5, ptr(dg), ptr(db), i64(1280), C.c_float(1e-5), ptr(xq), ptr(xd), None))
    assert bits_equal(dy2.cpu().numpy(), dy.cpu().numpy())
    rq, rd = O.quantize_row_q8_0(dy.cpu().numpy()[::-1].copy())       # row i of the launch wrote dy[4 - i]
    assert np.array_equal(xq.cpu().numpy().reshape(-1), rq) and bits_equal(xd.cpu().numpy().reshape(-1), rd)
    assert K.b200_layer_norm_rows_q(lr, 5, ptr(dg), ptr(db), i64(1290), C.c_float(1e-5), ptr(xq), ptr(xd), None) != 0


class TopkResult(C.Structure):
    _fields_ = [("n", C.c_int32), ("k", C.c_int32), ("max", C.c_float), ("logsumexp", C.c_float), ("ids", C.c_int32 * 8), ("vals", C.c_float * 8)]


@pytest.mark.parametrize("n,k,n_rows", [(51866, 5, 3), (1024, 8, 1), (70000, 1, 64), (40, 8, 2)])
def test_topk_rows(K, n, k, n_rows):
    """Top-k / max / log-sum-exp side output of logits rows against a host scan (ties resolved towards the lower index,
    as the reference's forward scan does)."""
    rng = np.random.default_rng(n + k)
    x = rng.standard_normal((n_rows, n)).astype(np.float32) * 4
    x[0, 7] = x[0, n - 3] = x[0].max() + 1          # a tie for the maximum
    if n_rows > 1:
        x[1, : min(n, 20)] = 2.5                    # a run of equal values
    dx = dev(x)
    out = torch.zeros((n_rows, C.sizeof(TopkResult)), dtype=torch.uint8, device="cuda")
    rows = (vp * n_rows)(*[dx[i].data_ptr() for i in range(n_rows)])
    outs = (vp * n_rows)(*[out[i].data_ptr() for i in range(n_rows)])
    sync_ok(K.b200_topk_rows(rows, outs, n_rows, i64(n), k, None))
    raw = out.cpu().numpy()
    for i in range(n_rows):
        r = TopkResult.from_buffer_copy(raw[i].tobytes())
        order = np.lexsort((np.arange(n), -x[i].astype(np.float64)))[:k]
        assert r.n == n and r.k == k
        assert list(r.ids)[:k] == order.tolist(), f"row {i}: {list(r.ids)[:k]} vs {order.tolist()}"
        assert np.array_equal(np.array(list(r.vals)[:k], np.float32), x[i][order])
        assert r.max == x[i].max()
        lse = float(np.log(np.exp(x[i].astype(np.float64) - float(x[i].max())).sum()) + float(x[i].max()))
        assert abs(r.logsumexp - lse) <= 1e-5 * max(1.0, abs(lse))
    assert K.b200_topk_rows(rows, outs, n_rows, i64(n), 9, None) != 0       # k beyond the maximum
    assert K.b200_topk_rows(rows, outs, 65, i64(n), 1, None) != 0           # too many rows


@pytest.mark.parametrize("wtype,bs", [(6, 22), (8, 34)])
def test_blocks_planes_on_the_device(K, wtype, bs):
    """Raw ggml blocks -> planes -> raw blocks on the device equals the host conversion, whole tensors and partial ranges."""
    nb = 3001
    blocks = np.random.default_rng(bs).integers(0, 256, (nb, bs), dtype=np.uint8)
    want = np.zeros(nb * bs, np.uint8)
    assert K.b200_blocks_to_planes(wtype, blocks.ctypes.data_as(vp), want.ctypes.data_as(vp), i64(nb), i64(0), i64(nb)) == 0
    d_blocks, d_planes = dev(blocks), torch.zeros(nb * bs, dtype=torch.uint8, device="cuda")
    sync_ok(K.b200_blocks_to_planes_device(wtype, ptr(d_blocks), ptr(d_planes), i64(nb), i64(0), i64(nb), None))
    assert np.array_equal(d_planes.cpu().numpy(), want)
    # a partial range (blocks 100..699) lands where the host puts it and leaves the rest alone
    part, want_p = torch.zeros(nb * bs, dtype=torch.uint8, device="cuda"), np.zeros(nb * bs, np.uint8)
    assert K.b200_blocks_to_planes(wtype, blocks[100:700].ctypes.data_as(vp), want_p.ctypes.data_as(vp), i64(nb), i64(100), i64(600)) == 0
    sync_ok(K.b200_blocks_to_planes_device(wtype, ptr(dev(blocks[100:700])), ptr(part), i64(nb), i64(100), i64(600), None))
    assert np.array_equal(part.cpu().numpy(), want_p)
    back = torch.zeros((nb, bs), dtype=torch.uint8, device="cuda")
    sync_ok(K.b200_planes_to_blocks_device(wtype, ptr(d_planes), ptr(back), i64(nb), i64(0), i64(nb), None))
    assert np.array_equal(back.cpu().numpy(), blocks)
    assert K.b200_blocks_to_planes_device(wtype, ptr(d_blocks), ptr(d_planes), i64(nb), i64(3000), i64(2), None) != 0
