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
            n_layers = pkg.synth.ARCHS[arch].n_dec
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
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, n_states=6, threads=1, probe=True)
    b0, g0 = backend_stat("b200_stat_batches", True), backend_stat("b200_stat_batched_graphs", True)
    got, _ = gpu.greedy_batch(24, pcm=pcm, device_mel=True)
    b1, g1 = backend_stat("b200_stat_batches", True), backend_stat("b200_stat_batched_graphs", True)
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
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, probe=True)
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


def test_every_node_runs_on_the_plugin_and_every_graph_is_one_split(pkg, model_dir):
    """Equality, not a lower bound: the computing nodes of the graphs whisper.cpp builds (conv, encoder, cross, one
    prompt step, single-token steps) are exactly the nodes the plugin reports, every graph reached the plugin as a
    whole (one scheduler split), so the CPU backend that sits last in the scheduler computed nothing."""
    from whisper_cpp_b200.host import backend_stat
    path = os.path.join(model_dir, "tiny-q5_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "tiny", "q5_0", seed=0)
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(3))
    w = pkg.Whisper(path, use_gpu=True, flash_attn=True, probe=True)
    w.set_mel(w.pcm_to_mel(pcm)[:, :3000].copy())
    n0, g0 = backend_stat("b200_stat_nodes", True), backend_stat("b200_stat_graphs", True)
    w.encode()
    expect_nodes = sum(w.graph_nodes(i) for i in range(3))
    expect_graphs = 3
    logits = w.decode(w.prefix(), 0)
    expect_nodes += w.graph_nodes(3)
    expect_graphs += 1
    n_past = 4
    for _ in range(5):
        logits = w.decode([int(np.argmax(logits))], n_past)
        n_past += 1
        expect_nodes += w.graph_nodes(3)
        expect_graphs += 1
    assert w.sched_splits() == [1, 1, 1, 1], f"a graph was split between backends: {w.sched_splits()}"
    got_nodes, got_graphs = backend_stat("b200_stat_nodes", True) - n0, backend_stat("b200_stat_graphs", True) - g0
    w.close()
    assert got_graphs == expect_graphs, f"graphs on the plugin {got_graphs}, graphs whisper.cpp ran {expect_graphs}"
    assert got_nodes == expect_nodes, f"nodes on the plugin {got_nodes}, computing nodes of the graphs {expect_nodes}"


@pytest.mark.parametrize("n_states", [14, 33])
def test_more_states_than_a_group_holds(pkg, model_dir, n_states):
    """More states than one merged group takes (the cap is 12 by default, 32 columns per launch): several leaders in
    flight, groups of 9..32 columns, a second flush.  Every clip must get the reference CPU backend's token ids."""
    from whisper_cpp_b200.host import backend_stat
    path = os.path.join(model_dir, "tiny-q5_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "tiny", "q5_0", seed=0)
    pcm = np.stack([pkg.synth.pcm_f32(pkg.synth.make_clip(200 + i, 8.0)) for i in range(n_states + 3)])
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    want, _ = cpu.greedy_batch(20, pcm=pcm, device_mel=False)
    cpu.close()
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, n_states=n_states, threads=1, probe=True)
    b0, g0 = backend_stat("b200_stat_batches", True), backend_stat("b200_stat_batched_graphs", True)
    got, _ = gpu.greedy_batch(20, pcm=pcm, device_mel=True)
    b1, g1 = backend_stat("b200_stat_batches", True), backend_stat("b200_stat_batched_graphs", True)
    gpu.close()
    bad = [i for i in range(len(pcm)) if not np.array_equal(got[i], want[i])]
    assert not bad, f"clips {bad} differ from the reference CPU backend under batching with {n_states} states"
    assert g1 - g0 > b1 - b0 > 0


def _encode_all(w, mels):
    """whisper_encode of len(mels) clips on as many states at once (one host thread per state)."""
    import threading
    out, err = [None] * len(mels), []

    def work(i):
        try:
            w.set_mel(mels[i], state=i)
            out[i] = w.encode(state=i)
        except Exception as e:      # noqa: BLE001
            err.append(e)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(mels))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not err, err
    return out


def test_config1_base_q5_0_encoder_16_clips(pkg, model_dir):
    """Benchmark configuration 1: base Q5_0, encoder only, a batch of 16 clips (here: 16 states encoding at once on
    their own streams) - conv stem, quantised products and 1500 x 1536 flash attention against the CPU backend."""
    path = os.path.join(model_dir, "base-q5_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "base", "q5_0", seed=0)
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    mels = [cpu.pcm_to_mel(pkg.synth.pcm_f32(pkg.synth.make_clip(300 + i)))[:, :3000].copy() for i in range(16)]
    want = []
    for m in mels:
        cpu.set_mel(m)
        want.append(cpu.encode())
    cpu.close()
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, n_states=16, threads=1, probe=True)
    got = _encode_all(gpu, mels)
    gpu.close()
    errs = [rel_l2(want[i], got[i]) for i in range(16)]
    print(f"base q5_0, 16 clips: encoder rel-L2 max {max(errs):.3e}")
    assert max(errs) <= ENC_TOL


def test_config2_small_q8_0_whisper_full_beam5(pkg, model_dir):
    """Benchmark configuration 2: small Q8_0 through whisper_full with beam search of width 5 (token budget shortened
    to bound the CPU time of the oracle), two clips: decoder KV-cache attention with several sequences per step,
    cross-attention, the 51865-wide logits and the host top-k sampler."""
    path = os.path.join(model_dir, "small-q8_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "small", "q8_0", seed=0)
    clips = [pkg.synth.pcm_f32(pkg.synth.make_clip(400 + i)) for i in range(2)]
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    want = [cpu.full(c, beam_size=5, max_tokens=40) for c in clips]
    cpu.close()
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, probe=True)
    got = [gpu.full(c, beam_size=5, max_tokens=40) for c in clips]
    gpu.close()
    for i in range(2):
        assert len(want[i]) > 0 and np.array_equal(want[i], got[i]), f"clip {i}: {want[i][:16]} vs {got[i][:16]}"


def test_config4_large_v3_turbo_q8_0(pkg, model_dir):
    """Benchmark configuration 4's model: large-v3-turbo Q8_0 (32 encoder + 4 decoder layers, F16 KV and attention):
    encoder output and 8 teacher-forced steps against the CPU backend."""
    check(run_pair(pkg, model_dir, "large-v3-turbo", "q8_0", True, n_new=8), "large-v3-turbo q8_0 flash")


def _unbatched_reference(pkg, path, pcm_file, n_new, out_file):
    """The same plugin with cross-state batching switched off and one state, in a process of its own (the switch is read
    once per process): the clip-by-clip result that the batched run must reproduce."""
    import subprocess
    import sys
    code = (
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.abspath(__file__))!r})\n"
        "from conftest import load_pkg\n"
        "pkg = load_pkg()\n"
        f"pcm = np.load({pcm_file!r})\n"
        f"w = pkg.Whisper({path!r}, use_gpu=True, flash_attn=True, n_states=1, threads=1, probe=True)\n"
        f"toks, _ = w.greedy_batch({n_new}, pcm=pcm, device_mel=True)\n"
        "w.close()\n"
        f"np.save({out_file!r}, toks)\n")
    env = dict(os.environ, GGML_B200_NO_BATCHING="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stderr[-3000:]
    return np.load(out_file)


def test_large_v3_states_at_different_positions_in_one_group(pkg, model_dir, tmp_path):
    """The benchmark's regime: large-v3 Q5_0, 16 states, more clips than states, encoders admitted three at a time so that
    the states reach their decode loops at different times - merged groups then hold states at different positions (own
    key counts, own masks), and a state that takes its second clip joins others that are mid-decode.  Every clip must
    reproduce what the same plugin computes for it alone without batching; two clips are also checked against the
    reference CPU backend."""
    from whisper_cpp_b200.host import backend_stat
    path = os.path.join(model_dir, "large-v3-q5_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "large-v3", "q5_0", seed=0)
    n_clips, n_new = 20, 24
    pcm = np.stack([pkg.synth.pcm_f32(pkg.synth.make_clip(500 + i)) for i in range(n_clips)])
    pcm_file, out_file = str(tmp_path / "pcm.npy"), str(tmp_path / "alone.npy")
    np.save(pcm_file, pcm)
    alone = _unbatched_reference(pkg, path, pcm_file, n_new, out_file)
    os.environ["DRV_MAX_ENC"] = "3"
    try:
        gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, n_states=16, threads=1, probe=True)
        b0, g0 = backend_stat("b200_stat_batches", True), backend_stat("b200_stat_batched_graphs", True)
        got, _ = gpu.greedy_batch(n_new, pcm=pcm, device_mel=True)
        b1, g1 = backend_stat("b200_stat_batches", True), backend_stat("b200_stat_batched_graphs", True)
        gpu.close()
    finally:
        del os.environ["DRV_MAX_ENC"]
    bad = [i for i in range(n_clips) if not np.array_equal(got[i], alone[i])]
    assert not bad, f"clips {bad} differ between the batched and the unbatched plugin"
    assert g1 - g0 > b1 - b0 > 0, "nothing was merged"
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    want, _ = cpu.greedy_batch(n_new, pcm=pcm[:2], device_mel=False)
    cpu.close()
    assert np.array_equal(want, got[:2]), f"{want} vs {got[:2]}"


def test_product_driver_in_its_own_process(pkg, model_dir, tmp_path):
    """The product build of the driver (linked against baseline/_ref, not the oracle's copy of the host libraries) in a
    process of its own: token ids equal to the oracle's, and no library under oracle/ is mapped in that process."""
    import subprocess
    import sys
    path = os.path.join(model_dir, "tiny-q5_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "tiny", "q5_0", seed=0)
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(11))[None, :]
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    want, _ = cpu.greedy_batch(12, pcm=pcm, device_mel=False)
    cpu.close()
    pcm_file, out_file = str(tmp_path / "pcm.npy"), str(tmp_path / "toks.npy")
    np.save(pcm_file, pcm)
    code = (
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.abspath(__file__))!r})\n"
        "from conftest import load_pkg\n"
        "pkg = load_pkg()\n"
        f"w = pkg.Whisper({path!r}, use_gpu=True, flash_attn=True)\n"
        f"toks, _ = w.greedy_batch(12, pcm=np.load({pcm_file!r}), device_mel=True)\n"
        "w.close()\n"
        f"np.save({out_file!r}, toks)\n"
        "maps = open('/proc/self/maps').read()\n"
        "assert '/baseline/_ref/libwhisper.so' in maps and '/oracle/' not in maps, [l for l in maps.splitlines() if '_ref' in l]\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert np.array_equal(np.load(out_file), want)


def test_logits_side_output_equals_host_scan(pkg, model_dir):
    """The plugin's top-k / max side output of every decode step equals a host scan of the reference CPU backend's logits
    for 32 steps (the logits themselves are bit-identical, so ids and values must be equal); the driver's greedy loop gives
    the same token ids whether it samples from the side output (with and without the logits read-back) or from the row."""
    import whisper_cpp_b200.host as H
    path = os.path.join(model_dir, "tiny-q8_0.bin")
    if not os.path.exists(path):
        pkg.synth.write_model(path, "tiny", "q8_0", seed=0)
    pcm = pkg.synth.pcm_f32(pkg.synth.make_clip(5))
    cpu = pkg.Whisper(path, use_gpu=False, flash_attn=True)
    mel = cpu.pcm_to_mel(pcm)[:, :3000].copy()
    cpu.set_mel(mel)
    want_toks, _, want_logits = cpu.greedy(32, want_logits=True)
    cpu.close()
    gpu = pkg.Whisper(path, use_gpu=True, flash_attn=True, probe=True)
    try:
        H.logits_side_output(5, skip_readback=False, probe=True, use_in_driver=False)
        gpu.set_mel(mel)
        gpu.encode()
        gpu.decode(gpu.prefix(), 0)
        n_past, row = 4, 3
        for step in range(32):
            r = H.last_topk(row, probe=True)
            order = np.lexsort((np.arange(gpu.n_vocab), -want_logits[step].astype(np.float64)))[:5]
            assert list(r.ids)[:5] == order.tolist(), f"step {step}"
            assert np.array_equal(np.array(list(r.vals)[:5], np.float32), want_logits[step][order]), f"step {step}"
            assert r.max == want_logits[step].max() and r.n == gpu.n_vocab
            if step + 1 < 32:
                gpu.decode([int(want_toks[step])], n_past)
                n_past, row = n_past + 1, 0
        d2h = []
        for skip in (False, True):
            H.logits_side_output(2, skip_readback=skip, probe=True, use_in_driver=True)
            gpu.set_mel(mel)
            b0 = H.backend_stat("b200_stat_d2h", True)
            toks = gpu.greedy(32)[0]
            d2h.append(H.backend_stat("b200_stat_d2h", True) - b0)
            assert np.array_equal(toks, want_toks), f"skip_readback={skip}: {toks} vs {want_toks}"
        assert d2h[1] < d2h[0] / 50, f"the logits rows still crossed the bus with the read-back switched off: {d2h}"
    finally:
        H.logits_side_output(0, probe=True)
        gpu.close()


def test_tcgen05_product_at_model_level(pkg, model_dir):
    """The tcgen05 / tensor-memory form of the many-column product is opt-in (GGML_B200_TC=1, read once per process): with it
    a whole tiny model - encoder, cross K/V and prompt products all go through it - is still bit-identical to the reference
    CPU backend.  Runs tests/relaxed_drift.py in a process of its own and reads its exact-arithmetic leg."""
    import json
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, GGML_B200_TC="1", B200_MODEL_DIR=model_dir)
    r = subprocess.run([sys.executable, os.path.join(here, "relaxed_drift.py"), "tiny", "q5_0", "8"], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    res = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    exact = res["plugin_exact"]
    assert "error" not in exact, exact
    assert exact["encoder_rel_l2"] == 0.0 and exact["logits_max_rel"] == 0.0 and exact["first_free_running_divergence"] is None, exact
