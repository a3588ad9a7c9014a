"""Synthetic Whisper model files and audio clips.

Writes model files in the legacy "ggml" container that whisper.cpp loads
(container layout: whisper.cpp models/convert-pt-to-ggml.py:273-338; loader:
src/whisper.cpp:1508-1960) with random-init weights, and seeded noise+tone clips.
Quantised files follow the rules of the reference quantize tool
(examples/quantize/quantize.cpp:158-170, examples/common-ggml.cpp:120-192): every
2-D tensor except the conv biases and the two positional embeddings is quantised
row by row from its F16 values; block arithmetic restates
ggml/src/ggml-quants.c:105-146 (Q5_0) and :194-216 (Q8_0).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

GGML_FILE_MAGIC = 0x67676D6C
GGML_TYPE_F32, GGML_TYPE_F16, GGML_TYPE_Q5_0, GGML_TYPE_Q8_0 = 0, 1, 6, 8
FTYPE = {"f16": 1, "q5_0": 2 * 1000 + 8, "q8_0": 2 * 1000 + 7}
WTYPE = {"f16": GGML_TYPE_F16, "q5_0": GGML_TYPE_Q5_0, "q8_0": GGML_TYPE_Q8_0}
N_VOCAB_FILE = 50257
SAMPLE_RATE = 16000
N_FFT = 400


@dataclass(frozen=True)
class Arch:
    name: str
    d: int
    n_head: int
    n_enc: int
    n_dec: int
    n_mels: int = 80
    n_vocab: int = 51865
    n_audio_ctx: int = 1500
    n_text_ctx: int = 448


ARCHS = {
    "tiny": Arch("tiny", 384, 6, 4, 4),
    "base": Arch("base", 512, 8, 6, 6),
    "small": Arch("small", 768, 12, 12, 12),
    "medium": Arch("medium", 1024, 16, 24, 24),
    "large-v3": Arch("large-v3", 1280, 20, 32, 32, n_mels=128, n_vocab=51866),
    "large-v3-turbo": Arch("large-v3-turbo", 1280, 20, 32, 4, n_mels=128, n_vocab=51866),
}


# ----------------------------------------------------------------------------- quantisers
def quantize_q5_0(x: np.ndarray) -> np.ndarray:
    """f32 [rows, k] -> bytes [rows, k/32, 22] = {f16 d, u32 qh, 16 nibble bytes}."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    assert k % 32 == 0
    b = x.reshape(rows, k // 32, 32)
    idx = np.argmax(np.abs(b), axis=-1)  # first index of the absolute maximum
    mx = np.take_along_axis(b, idx[..., None], axis=-1)[..., 0]
    d = (mx / np.float32(-16.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    xs = (b * inv[..., None]).astype(np.float32) + np.float32(16.5)
    q = np.minimum(31, xs.astype(np.int8).astype(np.uint8)).astype(np.uint8)  # C cast truncates
    lo, hi = q[..., :16], q[..., 16:]
    qs = (lo & 0x0F) | ((hi & 0x0F) << 4)
    sh = np.arange(16, dtype=np.uint32)
    qh = ((lo >> 4).astype(np.uint32) << sh).sum(-1, dtype=np.uint32) | (
        ((hi >> 4).astype(np.uint32) << (sh + 16)).sum(-1, dtype=np.uint32))
    out = np.empty((rows, k // 32, 22), dtype=np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, k // 32, 2)
    out[..., 2:6] = qh.view(np.uint8).reshape(rows, k // 32, 4)
    out[..., 6:22] = qs
    return out


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [rows, k] -> bytes [rows, k/32, 34] = {f16 d, 32 int8}; rounding = roundf."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    assert k % 32 == 0
    b = x.reshape(rows, k // 32, 32)
    amax = np.abs(b).max(-1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    v = (b * inv[..., None]).astype(np.float32)
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)  # roundf: half away from zero
    out = np.empty((rows, k // 32, 34), dtype=np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, k // 32, 2)
    out[..., 2:34] = q.view(np.uint8)
    return out


def dequantize_q5_0(blocks: np.ndarray) -> np.ndarray:
    """bytes [..., 22] -> f32 [..., 32]  (ggml-quants.c:296-320)."""
    d = blocks[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    qh = blocks[..., 2:6].copy().view(np.uint32)[..., 0]
    qs = blocks[..., 6:22]
    sh = np.arange(16, dtype=np.uint32)
    h0 = ((qh[..., None] >> sh) & 1).astype(np.int32) << 4
    h1 = ((qh[..., None] >> (sh + 16)) & 1).astype(np.int32) << 4
    x0 = ((qs & 0x0F).astype(np.int32) | h0) - 16
    x1 = ((qs >> 4).astype(np.int32) | h1) - 16
    return np.concatenate([x0, x1], -1).astype(np.float32) * d[..., None]


def dequantize_q8_0(blocks: np.ndarray) -> np.ndarray:
    d = blocks[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    return blocks[..., 2:34].view(np.int8).astype(np.float32) * d[..., None]


# ----------------------------------------------------------------------------- model pieces
def mel_filterbank(n_mels: int, n_fft: int = N_FFT, sr: int = SAMPLE_RATE) -> np.ndarray:
    """Slaney-scale triangular mel filters with area normalisation, f32 [n_mels, n_fft/2+1]."""
    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        lin = f / (200.0 / 3)
        log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
        return np.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))

    freqs = np.linspace(0, sr / 2, n_fft // 2 + 1)
    pts = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(sr / 2), n_mels + 2))
    fdiff = np.diff(pts)
    ramps = pts[:, None] - freqs[None, :]
    lower = -ramps[:-2] / fdiff[:-1, None]
    upper = ramps[2:] / fdiff[1:, None]
    w = np.maximum(0, np.minimum(lower, upper))
    w *= (2.0 / (pts[2:n_mels + 2] - pts[:n_mels]))[:, None]
    return w.astype(np.float32)


def sinusoids(length: int, channels: int) -> np.ndarray:
    inc = np.log(10000.0) / (channels // 2 - 1)
    inv = np.exp(-inc * np.arange(channels // 2))
    t = np.arange(length)[:, None] * inv[None, :]
    return np.concatenate([np.sin(t), np.cos(t)], axis=1).astype(np.float32)


def _vocab_token(i: int) -> bytes:
    return b" " if i == 220 else (b"<%d>" % i)  # id 220 must be " " (looked up by src/whisper.cpp:5057)


def tensor_list(a: Arch):
    """(name, numpy-shape, kind) in file order; numpy shape is ggml ne reversed."""
    d = a.d
    out = [
        ("encoder.positional_embedding", (a.n_audio_ctx, d), "sin"),
        ("encoder.conv1.weight", (d, a.n_mels, 3), "conv"),
        ("encoder.conv1.bias", (d, 1), "bias"),
        ("encoder.conv2.weight", (d, d, 3), "conv"),
        ("encoder.conv2.bias", (d, 1), "bias"),
        ("encoder.ln_post.weight", (d,), "one"),
        ("encoder.ln_post.bias", (d,), "zero"),
    ]

    def block(p, cross):
        t = [
            (f"{p}.mlp_ln.weight", (d,), "one"), (f"{p}.mlp_ln.bias", (d,), "zero"),
            (f"{p}.mlp.0.weight", (4 * d, d), "lin"), (f"{p}.mlp.0.bias", (4 * d,), "bias"),
            (f"{p}.mlp.2.weight", (d, 4 * d), "lin"), (f"{p}.mlp.2.bias", (d,), "bias"),
        ]
        for att in (["attn", "cross_attn"] if cross else ["attn"]):
            t += [
                (f"{p}.{att}_ln.weight", (d,), "one"), (f"{p}.{att}_ln.bias", (d,), "zero"),
                (f"{p}.{att}.query.weight", (d, d), "lin"), (f"{p}.{att}.query.bias", (d,), "bias"),
                (f"{p}.{att}.key.weight", (d, d), "lin"),
                (f"{p}.{att}.value.weight", (d, d), "lin"), (f"{p}.{att}.value.bias", (d,), "bias"),
                (f"{p}.{att}.out.weight", (d, d), "lin"), (f"{p}.{att}.out.bias", (d,), "bias"),
            ]
        return t

    for i in range(a.n_enc):
        out += block(f"encoder.blocks.{i}", False)
    out += [
        ("decoder.positional_embedding", (a.n_text_ctx, d), "pos"),
        ("decoder.token_embedding.weight", (a.n_vocab, d), "lin"),
        ("decoder.ln.weight", (d,), "one"), ("decoder.ln.bias", (d,), "zero"),
    ]
    for i in range(a.n_dec):
        out += block(f"decoder.blocks.{i}", True)
    return out


def write_model(path: str, arch: str | Arch, wtype: str = "f16", seed: int = 0) -> dict:
    """Random-init model: linear/embedding/conv weights N(0,0.02) (stored F16, then quantised to
    `wtype` from the F16 values), biases N(0,0.02) F32, LayerNorm gain 1 / bias 0, sinusoidal
    encoder positions, decoder positions N(0,0.01).  Returns {"bytes": file size}."""
    a = ARCHS[arch] if isinstance(arch, str) else arch
    rng = np.random.default_rng(seed)
    with open(path, "wb") as f:
        f.write(struct.pack("<I", GGML_FILE_MAGIC))
        f.write(struct.pack("<11i", a.n_vocab, a.n_audio_ctx, a.d, a.n_head, a.n_enc,
                            a.n_text_ctx, a.d, a.n_head, a.n_dec, a.n_mels, FTYPE[wtype]))
        f.write(struct.pack("<2i", a.n_mels, N_FFT // 2 + 1))
        f.write(mel_filterbank(a.n_mels).tobytes())
        f.write(struct.pack("<i", N_VOCAB_FILE))
        for i in range(N_VOCAB_FILE):
            t = _vocab_token(i)
            f.write(struct.pack("<I", len(t)))
            f.write(t)
        for name, shape, kind in tensor_list(a):
            if kind == "sin":
                data, tt = sinusoids(*shape), GGML_TYPE_F32
            elif kind == "one":
                data, tt = np.ones(shape, np.float32), GGML_TYPE_F32
            elif kind == "zero":
                data, tt = np.zeros(shape, np.float32), GGML_TYPE_F32
            elif kind == "bias":
                data, tt = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)), GGML_TYPE_F32
            elif kind == "pos":
                data, tt = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.01)), GGML_TYPE_F32
            else:  # "lin" / "conv": stored F16
                w16 = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
                if kind == "lin" and wtype != "f16":
                    q = quantize_q5_0 if wtype == "q5_0" else quantize_q8_0
                    data, tt = q(w16.astype(np.float32)), WTYPE[wtype]
                else:
                    data, tt = w16, GGML_TYPE_F16
            nb = name.encode()
            ne = shape[::-1]
            f.write(struct.pack("<3i", len(ne), len(nb), tt))
            f.write(struct.pack("<%di" % len(ne), *ne))
            f.write(nb)
            f.write(np.ascontiguousarray(data).tobytes())
        size = f.tell()
    return {"bytes": size}


# ----------------------------------------------------------------------------- audio
def make_clip(seed: int, seconds: float = 30.0, n_tones: int | None = 3, envelopes: bool = False) -> np.ndarray:
    """int16 mono 16 kHz: Gaussian noise sigma=0.05 + sine tones (100-4000 Hz, amplitude 0.2).
    n_tones=None draws 1..5 tones; envelopes=True multiplies each tone by a slow seeded AM envelope."""
    rng = np.random.default_rng(seed)
    n = int(seconds * SAMPLE_RATE)
    t = np.arange(n, dtype=np.float64) / SAMPLE_RATE
    x = rng.standard_normal(n) * 0.05
    k = int(rng.integers(1, 6)) if n_tones is None else n_tones
    for _ in range(k):
        fr = rng.uniform(100.0, 4000.0)
        tone = 0.2 * np.sin(2 * np.pi * fr * t + rng.uniform(0, 2 * np.pi))
        if envelopes:
            tone *= 0.5 * (1.0 + np.sin(2 * np.pi * rng.uniform(0.2, 3.0) * t + rng.uniform(0, 2 * np.pi)))
        x += tone
    return np.clip(np.round(x * 32768.0), -32768, 32767).astype(np.int16)


def pcm_f32(clip_i16: np.ndarray) -> np.ndarray:
    return (clip_i16.astype(np.float32) / np.float32(32768.0)).astype(np.float32)
