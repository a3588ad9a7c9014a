"""Pins the CPU restatement (oracle/restatement.c) and the generator's quantisers against the reference:
always against the committed golden vectors (tests/golden/, produced from the unmodified reference
libraries by tests/golden/make_golden.py) and, where oracle/_ref exists, against the reference run live.
All comparisons are bit-exact."""
import os

import numpy as np
import pytest

import oracle_lib as O
import ref_ops as R

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def gold(name):
    return dict(np.load(os.path.join(GOLD, name + ".npz")))


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("name,t", [("q5_0", 6), ("q8_0", 8)])
def test_quantiser_and_dequant_golden(pkg, name, t):
    g = gold(f"quant_{name}")
    q = pkg.synth.quantize_q5_0 if t == 6 else pkg.synth.quantize_q8_0
    assert np.array_equal(q(g["w"]), g["blocks"]), "generator quantiser differs from ggml_quantize_chunk"
    assert bits_equal(O.dequantize(t, g["blocks"]), g["deq"])
    dq = pkg.synth.dequantize_q5_0 if t == 6 else pkg.synth.dequantize_q8_0
    assert bits_equal(dq(g["blocks"]).reshape(-1), g["deq"])


def test_activation_quantisation_golden():
    g = gold("act_q8_0")
    qs, d = O.quantize_row_q8_0(g["x"])
    blocks = g["blocks"]
    assert np.array_equal(qs.reshape(-1, 32), blocks[:, 2:].view(np.int8))
    assert bits_equal(d.astype(np.float16), blocks[:, :2].copy().view(np.float16).reshape(-1))


@pytest.mark.parametrize("name,t", [("q5_0", 6), ("q8_0", 8)])
def test_mul_mat_q_golden(name, t):
    g = gold(f"mul_mat_{name}")
    M, nb, _ = g["blocks"].shape
    assert bits_equal(O.mul_mat_q(t, g["blocks"], M, nb * 32, g["x"]), g["dst"])


@pytest.mark.parametrize("K", [128, 80])
def test_mul_mat_f16_golden(K):
    g = gold(f"mul_mat_f16_k{K}")
    assert bits_equal(O.mul_mat_f16(g["w"], g["x"]), g["dst"])


def test_norm_golden():
    g = gold("norm")
    assert bits_equal(O.norm(g["x"]), g["y"])


def test_gelu_golden_every_f16_input():
    g = gold("gelu")
    assert bits_equal(O.gelu(g["x"].astype(np.float32)).astype(np.float16), g["y"])


@pytest.mark.parametrize("name", ["nomask", "mask"])
def test_flash_attn_golden(name):
    g = gold(f"flash_attn_{name}")
    n_q, H = g["dst"].shape[0], g["dst"].shape[1]
    mask = g["mask"] if g["mask"].size else None
    out = O.flash_attn(g["q"].reshape(n_q, H, 64), g["k"].reshape(-1, H, 64), g["v"].reshape(-1, H, 64), mask, 0.125)
    assert bits_equal(out, g["dst"])


def test_soft_max_golden():
    g = gold("soft_max")
    assert bits_equal(O.soft_max(g["x"], g["mask"], 0.125, g["x"].shape[1]), g["y"])


@pytest.mark.parametrize("s", [1, 2])
def test_im2col_golden(s):
    g = gold(f"im2col_s{s}")
    assert bits_equal(O.im2col_1d(g["x"], 3, s), g["y"])


def test_log_mel_golden():
    g = gold("log_mel")
    mel = O.log_mel(g["pcm"], g["filters"])
    assert mel.shape[1] == int(g["n_len"])
    assert bits_equal(mel[:, :120], g["mel_head"])
    assert float(mel[:, 120:].max()) == float(g["tail"])


def test_mel_filterbank_properties(pkg):
    for n in (80, 128):
        f = pkg.synth.mel_filterbank(n)
        assert f.shape == (n, 201) and (f >= 0).all() and (f.sum(1) > 0).all()
        centers = (f * np.arange(201)).sum(1) / f.sum(1)
        assert (np.diff(centers) >= 0).all() and centers[-1] > 150


# ---- live against the reference build, when it is here -------------------------------------------
live = pytest.mark.skipif(not R.have_ref(), reason="reference build (oracle/_ref) missing")


@live
@pytest.mark.parametrize("t", [6, 8])
@pytest.mark.parametrize("K,M,N", [(384, 40, 5), (1280, 16, 2)])
def test_mul_mat_q_live(t, K, M, N):
    w = (np.random.default_rng(1).standard_normal((M, K)) * 0.02).astype(np.float32)
    x = np.random.default_rng(2).standard_normal((N, K)).astype(np.float32)
    blocks = R.quantize(t, w)
    assert bits_equal(O.mul_mat_q(t, blocks, M, K, x), R.run("CPU", "MUL_MAT", [t, K, M, N], inputs=[blocks, x], out_shape=(N, M)))


@live
def test_flash_attn_live_long():
    n_q, n_kv, H = 2, 1536, 3
    rng = np.random.default_rng(3)
    q = (rng.standard_normal((n_q, 64 * H)) * 0.5).astype(np.float32)
    k = (rng.standard_normal((n_kv, 64 * H)) * 0.5).astype(np.float16)
    v = rng.standard_normal((n_kv, 64 * H)).astype(np.float16)
    ref = R.run("CPU", "FLASH_ATTN", [n_q, n_kv, H, 0, n_kv], f=[0.125], inputs=[q, k, v], out_shape=(n_q, H, 64))
    out = O.flash_attn(q.reshape(n_q, H, 64), k.reshape(-1, H, 64), v.reshape(-1, H, 64), None, 0.125)
    assert bits_equal(out, ref)


@live
def test_generated_model_equals_reference_quantize_tool(pkg, tmp_path):
    import subprocess
    f16 = str(tmp_path / "t-f16.bin")
    pkg.synth.write_model(f16, "tiny", "f16", seed=0)
    tool = os.path.join(R.REF, "quantize")
    for wt in ("q5_0", "q8_0"):
        mine, ref = str(tmp_path / f"t-{wt}.bin"), str(tmp_path / f"t-{wt}.ref.bin")
        pkg.synth.write_model(mine, "tiny", wt, seed=0)
        subprocess.run([tool, f16, ref, wt], check=True, capture_output=True)
        assert open(mine, "rb").read() == open(ref, "rb").read()
