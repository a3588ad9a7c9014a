"""Per-operator parity: the B200 plugin against the reference's own CPU backend, same graph, same bytes.

Every case builds the operator the way src/whisper.cpp builds it (oracle/op_harness.cpp), runs it on
device "CPU" and on device "B200_0", and demands identical bits unless a tolerance is stated.
"""
import numpy as np
import pytest

import ref_ops as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.have_ref(), reason="reference build (oracle/_ref) missing")]

GPU = "B200_0"


@pytest.fixture(scope="module", autouse=True)
def plugin():
    n = R.load_plugin()
    assert n >= 1, "the B200 plugin exposes no device"


def both(op, p, f=(), inputs=(), out_shape=None, out_dtype=np.float32):
    a = R.run("CPU", op, p, f, inputs, out_shape, out_dtype)
    b = R.run(GPU, op, p, f, inputs, out_shape, out_dtype)
    return a, b


def assert_bits(a, b, what):
    av, bv = a.view(np.uint8).reshape(-1), b.view(np.uint8).reshape(-1)
    if not np.array_equal(av, bv):
        a32, b32 = a.astype(np.float64).reshape(-1), b.astype(np.float64).reshape(-1)
        bad = np.flatnonzero(a32 != b32)
        rel = np.abs(a32 - b32).max() / (np.abs(a32).max() + 1e-30)
        raise AssertionError(f"{what}: {bad.size}/{a32.size} elements differ, max rel {rel:.3e}, first at {bad[:5]}: "
                             f"cpu {a32[bad[:5]]} gpu {b32[bad[:5]]}")


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


@pytest.mark.parametrize("wtype", [R.Q5_0, R.Q8_0])
def test_weight_roundtrip_bytes(wtype):
    w = R.quantize(wtype, rnd(1, 96, 256, scale=0.02))
    back = R.run(GPU, "ROUNDTRIP", [wtype, 256, 96], inputs=[w], out_shape=w.shape, out_dtype=np.uint8)
    assert np.array_equal(w, back)


@pytest.mark.parametrize("wtype", [R.Q5_0, R.Q8_0])
@pytest.mark.parametrize("K,M,N", [(384, 384, 1), (512, 2048, 1), (1280, 1280, 5), (1280, 1000, 8), (384, 51865, 1),
                                    (512, 512, 37), (2048, 512, 100), (1280, 5120, 1500 // 4), (64, 70, 33)])
def test_mul_mat_quant(wtype, K, M, N):
    w = R.quantize(wtype, rnd(2, M, K, scale=0.02))
    x = rnd(3, N, K)
    a, b = both("MUL_MAT", [wtype, K, M, N], inputs=[w, x], out_shape=(N, M))
    assert_bits(a, b, f"mul_mat type {wtype} K{K} M{M} N{N}")


@pytest.mark.parametrize("overwrite", [0, 1])
@pytest.mark.parametrize("wtype,K,M,N", [(R.Q5_0, 1280, 256, 64), (R.Q8_0, 384, 100, 40), (R.Q5_0, 512, 96, 12)])
def test_two_products_on_the_same_activations(wtype, K, M, N, overwrite):
    """The plugin quantises activations once for products that follow each other on the same source - and again when a node
    in between wrote into that memory (here: an in-place scale)."""
    w = R.quantize(wtype, rnd(12, M, K, scale=0.02))
    x = rnd(13, N, K)
    a, b = both("MM_TWICE", [wtype, K, M, N, overwrite], inputs=[w, x], out_shape=(N, M))
    assert_bits(a, b, f"two products, overwrite {overwrite}")


@pytest.mark.parametrize("K,M,N", [(384, 384, 1), (384, 1536, 3), (1536, 384, 40), (240, 300, 384), (384, 51865, 1), (100, 7, 5)])
def test_mul_mat_f16_weights(K, M, N):
    w = rnd(4, M, K, scale=0.02).astype(np.float16)
    x = rnd(5, N, K)
    a, b = both("MUL_MAT", [R.F16, K, M, N], inputs=[w, x], out_shape=(N, M))
    assert_bits(a, b, f"mul_mat f16 K{K} M{M} N{N}")


@pytest.mark.parametrize("K,OW,OC", [(240, 3000 // 10, 384), (1152, 150, 384)])
def test_mul_mat_conv_f16_f16(K, OW, OC):
    cols = rnd(6, OW, K).astype(np.float16)
    w = rnd(7, OC, K, scale=0.02).astype(np.float16)
    a, b = both("MUL_MAT_CONV", [K, OW, OC], inputs=[cols, w], out_shape=(OC, OW))
    assert_bits(a, b, "conv product")


@pytest.mark.parametrize("n_q,n_kv,H,mask", [(1, 1536, 6, 0), (1, 37, 6, 1), (5, 77, 8, 1), (40, 1536, 6, 0), (4, 448, 20, 1), (33, 65, 2, 1)])
def test_flash_attn_ext(n_q, n_kv, H, mask):
    d = 64 * H
    q = rnd(8, n_q, d, scale=0.5)
    k = rnd(9, n_kv, d, scale=0.5).astype(np.float16)
    v = rnd(10, n_kv, d).astype(np.float16)
    inputs = [q, k, v]
    if mask:
        rows = (n_q + 63) // 64 * 64
        m = np.zeros((rows, n_kv), np.float16)
        rng = np.random.default_rng(11)
        m[rng.random((rows, n_kv)) < 0.3] = -np.inf
        m[:, 0] = 0
        inputs.append(m)
    a, b = both("FLASH_ATTN", [n_q, n_kv, H, mask, n_kv], f=[0.125], inputs=inputs, out_shape=(n_q, H, 64))
    assert_bits(a, b, f"flash_attn n_q{n_q} n_kv{n_kv} H{H} mask{mask}")


@pytest.mark.parametrize("ne0,ne1", [(384, 1), (1280, 7), (512, 1500)])
def test_norm(ne0, ne1):
    x = rnd(12, ne1, ne0) * 3 + 0.5
    a, b = both("NORM", [ne0, ne1], f=[1e-5], inputs=[x], out_shape=(ne1, ne0))
    assert_bits(a, b, "norm")


@pytest.mark.parametrize("op", ["ADD", "MUL"])
@pytest.mark.parametrize("a_shape,b_shape", [((1500, 384), (1500, 384)), ((7, 384), (1, 384)), ((384, 3000), (384, 1))])
def test_binary_broadcast(op, a_shape, b_shape):
    x, y = rnd(13, *a_shape), rnd(14, *b_shape)
    a, b = both(op, [a_shape[1], a_shape[0], b_shape[1], b_shape[0]], inputs=[x, y], out_shape=a_shape)
    assert_bits(a, b, op)


def test_scale():
    x = rnd(15, 9, 384)
    a, b = both("SCALE", [384, 9], f=[64 ** -0.25], inputs=[x], out_shape=(9, 384))
    assert_bits(a, b, "scale")


def test_gelu_every_f16_input():
    h = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    h = h[np.isfinite(h)]
    extra = rnd(16, 4096) * 4
    x = np.concatenate([h, extra, np.array([-10.0, 10.0, -11.0, 12.5, 0.0], np.float32)])
    x = np.resize(x, (x.size // 64 + 1) * 64).reshape(-1, 64)
    a, b = both("GELU", [64, x.shape[0]], inputs=[x], out_shape=x.shape)
    assert_bits(a, b, "gelu")


def test_cpy_f32_to_f16_into_kv_view():
    x = rnd(17, 5, 384)
    a, b = both("CPY_F16", [384, 5, 384 * 3, 384 * 16], inputs=[x, None], out_shape=(384 * 16,), out_dtype=np.float16)
    assert_bits(a, b, "cpy f32->f16")


def test_cpy_transposed_store():
    x = rnd(18, 40, 384)
    a, b = both("CPY_F16_T", [384, 40, 64], inputs=[x, None], out_shape=(384 * 64,), out_dtype=np.float16)
    assert_bits(a, b, "cpy transposed")


def test_cont_transpose():
    x = rnd(19, 384, 1500)
    a, b = both("CONT_T", [1500, 384], inputs=[x], out_shape=(1500, 384))
    assert_bits(a, b, "cont(transpose)")


@pytest.mark.parametrize("ttype", [R.Q5_0, R.Q8_0, R.F16, R.F32])
def test_get_rows(ttype):
    table = rnd(20, 1000, 384, scale=0.02)
    if ttype in (R.Q5_0, R.Q8_0):
        t = R.quantize(ttype, table)
    elif ttype == R.F16:
        t = table.astype(np.float16)
    else:
        t = table
    ids = np.array([0, 999, 5, 5, 123, 77, 500], np.int32)
    a, b = both("GET_ROWS", [ttype, 384, 1000, len(ids)], inputs=[t, ids], out_shape=(len(ids), 384))
    assert_bits(a, b, "get_rows")


@pytest.mark.parametrize("IC,IW,stride", [(80, 3000, 1), (384, 3000, 2), (128, 300, 1)])
def test_im2col(IC, IW, stride):
    x = rnd(21, IC, IW)
    OW = (IW + 2 - 3) // stride + 1
    a, b = both("IM2COL", [IC, 8, IW, stride], inputs=[None, x], out_shape=(OW, IC * 3), out_dtype=np.float16)
    assert_bits(a, b, "im2col")


@pytest.mark.parametrize("ne0,ne1,ne2,mask", [(1500, 10, 6, 0), (37, 5, 6, 1), (448, 3, 2, 2), (1501, 4, 2, 0)])
def test_soft_max(ne0, ne1, ne2, mask):
    x = rnd(22, ne2, ne1, ne0, scale=2.0)
    inputs = [x]
    if mask:
        rows = (ne1 + 63) // 64 * 64
        m = np.zeros((rows, ne0), np.float32)
        m[np.random.default_rng(23).random((rows, ne0)) < 0.3] = -np.inf
        m[:, 0] = 0
        inputs.append(m.astype(np.float16) if mask == 2 else m)
    a, b = both("SOFT_MAX", [ne0, ne1, ne2, mask], f=[0.125], inputs=inputs, out_shape=x.shape)
    assert_bits(a, b, "soft_max")


def test_concat():
    x, y = rnd(24, 5, 64), rnd(25, 9, 64)
    a, b = both("CONCAT", [64, 5, 9, 1], inputs=[x, y], out_shape=(14, 64))
    assert_bits(a, b, "concat")


@pytest.mark.parametrize("n_q,n_kv,H", [(1, 77, 6), (40, 1500 // 10, 6)])
def test_nonflash_scores(n_q, n_kv, H):
    d = 64 * H
    k = rnd(26, n_kv, d, scale=0.5).astype(np.float16)
    q = rnd(27, n_q, d, scale=0.5)
    a, b = both("KQ_NOFA", [n_q, n_kv, H], inputs=[k, q], out_shape=(H, n_q, n_kv))
    assert_bits(a, b, "non-flash KQ")


@pytest.mark.parametrize("n_q,n_kv,H", [(1, 77, 6), (20, 150, 6)])
def test_nonflash_pv(n_q, n_kv, H):
    n_ctx = 160
    v = rnd(28, 64 * H, n_ctx).astype(np.float16)
    p = np.abs(rnd(29, H, n_q, n_kv))
    a, b = both("KQV_NOFA", [n_q, n_kv, H, n_ctx], inputs=[v, p], out_shape=(H, n_q, 64))
    assert_bits(a, b, "non-flash PV")


def test_error_paths_return_values_instead_of_aborting():
    """An allocation the device cannot satisfy comes back as a NULL buffer, and a graph with an operator the plugin does
    not implement comes back as a failed status (the scheduler never sends one; here it is handed over directly) - the
    process keeps running in both cases, and ordinary work still succeeds afterwards."""
    assert R.load_plugin() > 0
    L = R.lib()
    assert L.oph_try_alloc(b"B200_0", 1 << 20) == 1
    assert L.oph_try_alloc(b"B200_0", 1 << 46) == 0          # 64 TiB: cudaMalloc fails, alloc_buffer returns NULL
    st = L.oph_unsupported_status(b"B200_0")
    assert st == -1, f"graph_compute returned {st} for an unsupported operator, expected GGML_STATUS_FAILED (-1)"
    assert L.oph_try_alloc(b"B200_0", 1 << 20) == 1          # the device is still usable
