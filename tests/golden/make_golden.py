"""Generates tests/golden/*.npz from the UNMODIFIED reference libraries in oracle/_ref (built by oracle/Makefile).

Run where a whisper.cpp checkout exists:  make -C oracle && python tests/golden/make_golden.py
Every vector is the output of the reference's own code: ggml_quantize_chunk, the type-traits to_float /
from_float, single-operator graphs on the ggml CPU backend (oracle/op_harness.cpp), and whisper_pcm_to_mel.
Inputs are seeded; both inputs and outputs are stored, so the tests need no reference at run time.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import ref_ops as R  # noqa: E402
from conftest import load_pkg  # noqa: E402


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def main():
    out = {}
    # block formats
    w = rnd(1, 8, 128, scale=0.02)
    for name, t in (("q5_0", R.Q5_0), ("q8_0", R.Q8_0)):
        blocks = R.quantize(t, w)
        out[f"quant_{name}"] = dict(w=w, blocks=blocks, deq=R.dequantize(t, blocks))
    x = rnd(2, 4, 128) * np.array([[1.0], [1e-3], [30.0], [0.0]], np.float32)
    out["act_q8_0"] = dict(x=x, blocks=R.cpu_quantize_row_q8_0(x))
    # matrix products
    K, M, N = 128, 24, 3
    wq, xx = rnd(3, M, K, scale=0.02), rnd(4, N, K)
    for name, t in (("q5_0", R.Q5_0), ("q8_0", R.Q8_0)):
        blocks = R.quantize(t, wq)
        out[f"mul_mat_{name}"] = dict(blocks=blocks, x=xx, dst=R.run("CPU", "MUL_MAT", [t, K, M, N], inputs=[blocks, xx], out_shape=(N, M)))
    for K2 in (128, 80):
        w16, x2 = rnd(5, M, K2, scale=0.02).astype(np.float16), rnd(6, N, K2)
        out[f"mul_mat_f16_k{K2}"] = dict(w=w16, x=x2, dst=R.run("CPU", "MUL_MAT", [R.F16, K2, M, N], inputs=[w16, x2], out_shape=(N, M)))
    # row-wise
    xn = rnd(7, 5, 384) * 3 + 0.5
    out["norm"] = dict(x=xn, y=R.run("CPU", "NORM", [384, 5], f=[1e-5], inputs=[xn], out_shape=(5, 384)))
    h = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    h = h[np.isfinite(h)]
    h = np.resize(h, (h.size // 64 + 1) * 64).reshape(-1, 64)
    out["gelu"] = dict(x=h.astype(np.float16), y=R.run("CPU", "GELU", [64, h.shape[0]], inputs=[h], out_shape=h.shape).astype(np.float16))
    # attention
    n_q, n_kv, H = 3, 70, 2
    q, k, v = rnd(8, n_q, 64 * H, scale=0.5), rnd(9, n_kv, 64 * H, scale=0.5).astype(np.float16), rnd(10, n_kv, 64 * H).astype(np.float16)
    m = np.zeros((64, n_kv), np.float16)
    m[np.random.default_rng(11).random((64, n_kv)) < 0.3] = -np.inf
    m[:, 0] = 0
    for name, mask in (("nomask", None), ("mask", m)):
        ins = [q, k, v] + ([mask] if mask is not None else [])
        out[f"flash_attn_{name}"] = dict(q=q, k=k, v=v, mask=mask if mask is not None else np.zeros(0, np.float16),
                                         dst=R.run("CPU", "FLASH_ATTN", [n_q, n_kv, H, int(mask is not None), n_kv], f=[0.125], inputs=ins, out_shape=(n_q, H, 64)))
    xs = rnd(12, 2, 5, 37, scale=2.0)
    ms = np.zeros((64, 37), np.float32)
    ms[np.random.default_rng(13).random((64, 37)) < 0.3] = -np.inf
    ms[:, 0] = 0
    out["soft_max"] = dict(x=xs, mask=ms, y=R.run("CPU", "SOFT_MAX", [37, 5, 2, 1], f=[0.125], inputs=[xs, ms], out_shape=xs.shape))
    xi = rnd(14, 6, 50)
    for s in (1, 2):
        OW = (50 + 2 - 3) // s + 1
        out[f"im2col_s{s}"] = dict(x=xi, y=R.run("CPU", "IM2COL", [6, 4, 50, s], inputs=[None, xi], out_shape=(OW, 18), out_dtype=np.float16))
    # log-mel through whisper_pcm_to_mel (tiny model file only carries the filterbank)
    pkg = load_pkg()
    path = "/tmp/golden_tiny_f16.bin"
    pkg.synth.write_model(path, "tiny", "f16", seed=0)
    wsp = pkg.Whisper(path, use_gpu=False, probe=True)
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(3, seconds=1.0))
    mel = wsp.pcm_to_mel(pcm)
    out["log_mel"] = dict(pcm=pcm, filters=wsp.filters(), mel_head=mel[:, :120].copy(), n_len=np.array(mel.shape[1]), tail=mel[:, 120:].max())
    wsp.close()
    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
        print(name, {k: getattr(v, "shape", v) for k, v in d.items()})


if __name__ == "__main__":
    main()
