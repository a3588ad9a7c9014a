"""Whole-path parity through whisper.h: the same synthetic model file and clip run on the reference CPU
backend (use_gpu=false) and on the B200 plugin (use_gpu=true), flash_attn flag alike on both sides.

Gates (from the north star): encoder output relative L2 <= 1e-3; teacher-forced logits max relative
error <= 1e-2; greedy token ids identical except where the reference's top-2 margin is below 1e-3.
"""
import os

import numpy as np
import pytest

import ref_ops as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.have_ref(), reason="reference build (oracle/_ref) missing")]

ENC_TOL = 1e-3
LOGIT_TOL = 1e-2
MARGIN = 1e-3


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / np.linalg.norm(a.astype(np.float64)))


def run_pair(pkg, model_dir, arch, wtype, flash, n_new=32, seed=1):
    path = os.path.join(model_dir, f"{arch}-{wtype}.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, arch, wtype, seed=0)
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(seed))
    out = {}
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=flash, probe=True)
    mel = cpu.pcm_to_mel(pcm)[:, :3000].copy()
    from whisper_cpp_b200.host import backend_stat
    for name, w in (("cpu", cpu), ("gpu", None)):
        if w is None:
            w = pkg.Whisper(path, use_gpu=True, flash_attn=flash, probe=True)
            nodes0, launches0 = backend_stat("b200_stat_nodes", True), pkg.kernels_lib().b200_launch_count()
        w.set_mel(mel)
        enc = w.encode()
        force = out["cpu"]["tokens"] if name == "gpu" else None
        toks, margins, logits = w.greedy(n_new, force=force, want_logits=True)
        out[name] = dict(enc=enc, tokens=toks, margins=margins, logits=logits)
        if name == "gpu":   # free-running ids as well
            w.set_mel(mel)
            out[name]["free_tokens"] = w.greedy(n_new)[0]
            # the plugin, not the CPU backend, must have executed the graphs
            n_layers = {"tiny": 4, "base": 6, "large-v3": 32}[arch]
            assert backend_stat("b200_stat_nodes", True) - nodes0 > 2 * (20 * n_layers * (n_new + 1))
            assert pkg.kernels_lib().b200_launch_count() - launches0 > 0
        w.close()
    return out


def check(out, what):
    e = rel_l2(out["cpu"]["enc"], out["gpu"]["enc"])
    same = float((out["cpu"]["enc"] == out["gpu"]["enc"]).mean())
    lc, lg = out["cpu"]["logits"].astype(np.float64), out["gpu"]["logits"].astype(np.float64)
    lerr = float(np.abs(lc - lg).max() / np.abs(lc).max())
    print(f"{what}: encoder rel-L2 {e:.3e} (bit-identical fraction {same:.4f}); logits max-rel {lerr:.3e}; "
          f"bit-identical logits fraction {float((lc == lg).mean()):.4f}")
    assert e <= ENC_TOL, f"{what}: encoder rel-L2 {e}"
    assert lerr <= LOGIT_TOL, f"{what}: logits max-rel {lerr}"
    for name in ("tokens", "free_tokens"):
        diff = np.flatnonzero(out["cpu"]["tokens"] != out["gpu"][name])
        if name == "free_tokens" and diff.size:
            diff = diff[:1]   # after the first divergence the histories differ; only that step is comparable
        assert all(out["cpu"]["margins"][i] < MARGIN for i in diff), f"{what}: {name} differ at {diff} with margins {out['cpu']['margins'][diff]}"


@pytest.mark.parametrize("wtype", ["f16", "q5_0", "q8_0"])
def test_tiny_flash(pkg, model_dir, wtype):
    check(run_pair(pkg, model_dir, "tiny", wtype, True), f"tiny {wtype} flash_attn")


@pytest.mark.parametrize("wtype", ["f16", "q5_0"])
def test_tiny_no_flash(pkg, model_dir, wtype):
    check(run_pair(pkg, model_dir, "tiny", wtype, False), f"tiny {wtype} no flash_attn")


def test_base_q5_0_flash(pkg, model_dir):
    check(run_pair(pkg, model_dir, "base", "q5_0", True, n_new=16), "base q5_0 flash_attn")


def test_concurrent_states_are_batched_and_match_the_oracle(pkg, model_dir):
    """Several whisper_states decode at once; their steps are merged below graph_compute.  Every clip must still get
    exactly the token ids the reference CPU backend produces for it alone."""
    from whisper_cpp_b200.host import backend_stat
    path = os.path.join(model_dir, "tiny-q5_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "tiny", "q5_0", seed=0)
    pcm = np.stack([pkg.synth.pcm_f32(pkg.synth.make_clip(40 + i)) for i in range(6)])
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    want, _ = cpu.greedy_batch(24, pcm=pcm, device_mel=False)
    cpu.close()
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, n_states=6, threads=1)
    b0, g0 = backend_stat("b200_stat_batches"), backend_stat("b200_stat_batched_graphs")
    got, _ = gpu.greedy_batch(24, pcm=pcm, device_mel=True)
    b1, g1 = backend_stat("b200_stat_batches"), backend_stat("b200_stat_batched_graphs")
    gpu.close()
    assert np.array_equal(got, want), f"token ids differ under batching:\n{got}\n{want}"
    assert g1 - g0 > b1 - b0 > 0, f"no decode steps were merged (batches {b1 - b0}, graphs {g1 - g0})"


@pytest.mark.parametrize("beam", [1, 5])
def test_whisper_full_beam_search_token_ids(pkg, model_dir, beam):
    """whisper_full end to end (host log-mel, encoder, beam search with several decoders per step, KV cache sequence
    copies, the host sampler): the plugin's logits are bit-identical to the reference CPU backend's, so every beam takes
    the same decisions and the emitted token ids are equal.  Also with the mel computed on the device front-end."""
    path = os.path.join(model_dir, "tiny-q8_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "tiny", "q8_0", seed=0)
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(7))[: 16000 * 11]
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    want = cpu.full(pcm, beam_size=beam, max_tokens=48)
    cpu.close()
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True)
    launches0 = pkg.kernels_lib().b200_launch_count()
    got = gpu.full(pcm, beam_size=beam, max_tokens=48)
    assert pkg.kernels_lib().b200_launch_count() > launches0
    gpu.close()
    assert len(want) > 0 and np.array_equal(want, got), f"beam {beam}: {want[:16]} vs {got[:16]}"


def test_large_v3_q5_0_benchmark_shapes(pkg, model_dir):
    """The benchmark's own model size (d = 1280, 32 + 32 layers, 128 mel bins, vocabulary 51866): encoder output and the
    logits of a few teacher-forced steps against the reference CPU backend; this is where the tensor-pipe product runs at
    its real shapes (1280 x 1280, 5120 x 1280, 1280 x 5120 by 1500 columns)."""
    check(run_pair(pkg, model_dir, "large-v3", "q5_0", True, n_new=4), "large-v3 q5_0 flash")
