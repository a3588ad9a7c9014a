#!/usr/bin/env python
"""How far does a different summation order move the model outputs?  (run by hand on a B200; prints one JSON line)

    python tests/relaxed_drift.py ARCH WTYPE [N_NEW]

The plugin's kernels replay the reference CPU backend's arithmetic order, which costs throughput.  With
GGML_B200_RELAXED=1 two of them switch to what a plain tensor-core formulation would compute: the quantised product
applies ONE fma per 32-block to the whole block sum (instead of eight per-lane chains), and encoder attention rounds
the softmax weights to F16 once and keeps the V accumulator in f32 (instead of an F16 accumulator rounded after every
key).  This script measures, against the reference CPU backend on the same model file and clip:
  * encoder output relative L2 and teacher-forced logits max relative error of the relaxed plugin,
  * the first step at which its free-running greedy ids leave the reference's, with the reference's top-2 margin there,
  * the reference's own noise floor: its flash-attention path against its non-flash path on the same input.
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from conftest import load_pkg  # noqa: E402


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / np.linalg.norm(a.astype(np.float64)))


def max_rel(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(np.abs(a - b).max() / np.abs(a).max())


def leg(pkg, path, mel, use_gpu, flash, n_new, force):
    w = pkg.Whisper(path, use_gpu=use_gpu, flash_attn=flash, probe=True)
    w.set_mel(mel)
    enc = w.encode()
    toks, margins, logits = w.greedy(n_new, force=force, want_logits=True)
    free = None
    if use_gpu:
        w.set_mel(mel)
        free = w.greedy(n_new)[0]
    w.close()
    return dict(enc=enc, tokens=toks, margins=margins, logits=logits, free=free)


def main():
    arch, wtype = sys.argv[1], sys.argv[2]
    n_new = int(sys.argv[3]) if len(sys.argv) > 3 else 8
    pkg = load_pkg()
    d = os.environ.get("B200_MODEL_DIR", "/tmp/b200_models")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{arch}-{wtype}.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, arch, wtype, seed=0)
    if len(sys.argv) > 4:          # child: the plugin leg, exact or relaxed as the environment says
        z = np.load(sys.argv[4])
        out = leg(pkg, path, z["mel"], True, True, n_new, z["tokens"])
        np.savez(sys.argv[5], enc=out["enc"], logits=out["logits"], free=out["free"])
        return
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(1))
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True, probe=True)
    mel = cpu.pcm_to_mel(pcm)[:, :3000].copy()
    cpu.close()
    ref = leg(pkg, path, mel, False, True, n_new, None)
    nofa = leg(pkg, path, mel, False, False, n_new, ref["tokens"])
    res = {"arch": arch, "wtype": wtype, "n_new": n_new,
           "reference_flash_vs_reference_non_flash": {"encoder_rel_l2": rel_l2(ref["enc"], nofa["enc"]),
                                                      "logits_max_rel": max_rel(ref["logits"], nofa["logits"])},
           "reference_top2_margins": {"min": float(ref["margins"].min()), "median": float(np.median(ref["margins"]))},
           "reference_logit_abs_max": float(np.abs(ref["logits"]).max())}
    tmp_in, tmp_out = f"/tmp/relaxed_in_{os.getpid()}.npz", f"/tmp/relaxed_out_{os.getpid()}.npz"
    np.savez(tmp_in, mel=mel, tokens=ref["tokens"])
    for name, env in (("plugin_exact", {}), ("plugin_relaxed", {"GGML_B200_RELAXED": "1"})):
        r = subprocess.run([sys.executable, os.path.abspath(__file__), arch, wtype, str(n_new), tmp_in, tmp_out],
                           env=dict(os.environ, **env), capture_output=True, text=True)
        if r.returncode != 0:
            res[name] = {"error": r.stderr[-1500:]}
            continue
        z = np.load(tmp_out)
        diff = np.flatnonzero(z["free"] != ref["tokens"])
        res[name] = {"encoder_rel_l2": rel_l2(ref["enc"], z["enc"]), "logits_max_rel": max_rel(ref["logits"], z["logits"]),
                     "logits_bit_identical_fraction": float((ref["logits"] == z["logits"]).mean()),
                     "first_free_running_divergence": int(diff[0]) if diff.size else None,
                     "reference_margin_there": float(ref["margins"][diff[0]]) if diff.size else None}
    for f in (tmp_in, tmp_out):
        if os.path.exists(f):
            os.remove(f)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
