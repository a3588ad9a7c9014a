#!/usr/bin/env python
"""Throughput benchmark of the whisper.cpp hot path on the B200 ggml backend plugin.

Workload: Whisper large-v3, Q5_0 weights (random init, quantised by the rules of
the reference tool), a batch of 64 seeded 30 s clips, each: log-mel -> encoder -> greedy decode of 224 tokens
after the forced prefix [SOT, en, transcribe, notimestamps], driven through the unmodified whisper.h API
(whisper_set_mel / whisper_encode / whisper_decode).  The batch is split evenly over the ranks (one rank per
GPU, strong scaling: 64 clips in total at every N), no collective on the data path.

One "step" = one pass over the rank's share of the batch.
  value : audio-seconds / second with the log-mel inputs prepared before the timed region (they still enter
          through whisper_set_mel, the only input door of the plugin boundary);
  e2e   : the same from host PCM buffers: PCM -> device log-mel -> host mel -> whisper_set_mel -> encode ->
          decode -> token ids on the host, everything inside the timed region.

`--impl reference` times the reference's own CPU backend (the unmodified host libraries of baseline/_ref with the
CPU variant that suits the host, all host cores) on a bounded sample of the same workload (one clip per step).
`--impl oracle-tokens` (internal) runs clip 0 on the parity oracle (oracle/_ref, pinned AVX2 arithmetic) in a process
of its own and saves its token ids: the main run compares the ids of the same clip from its timed steps with them.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import resource
import subprocess
import sys
import threading
import time

import numpy as np

import importlib.util

ROOT = os.path.dirname(os.path.abspath(__file__))


def load_pkg():
    """The package directory name contains a dot, so it is loaded by path under an importable name."""
    if "whisper_cpp_b200" not in sys.modules:
        pkg_dir = os.path.join(ROOT, "whisper.cpp_b200")
        spec = importlib.util.spec_from_file_location("whisper_cpp_b200", os.path.join(pkg_dir, "__init__.py"),
                                                      submodule_search_locations=[pkg_dir])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["whisper_cpp_b200"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["whisper_cpp_b200"]


N_NEW = 224
CLIP_SECONDS = 30.0
TOTAL_CLIPS = 64

# What limits each kernel class (ncu counters of small cases of the same kernels): the reference's summation orders are
# replayed exactly, which keeps the attention kernels and the float chain of the products off the MMA accumulators.
LIMITER = {
    "flash_attn_ext":    "F16 accumulation chain and 32-way score sums replayed exactly: instruction issue, tensor pipe unused by design",
    "mul_mat_q":         "mma.sync lane sums (zero-expanded f16 operands), float chain of 8 FMAs per block and output on the FMA pipe",
    "mul_mat_vec_q":     "launch and load latency of small dependent launches, not bandwidth",
    "flash_attn_decode": "sequential F16 chain over the keys of each (row, head)",
}
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one representative launch of each class, from an ncu capture
TRAFFIC_NCU = {
    "mul_mat_vec_q":     {"bytes": 1.177e6, "launch": "1280 x 1280 Q5_0 weights x 12 columns, the group size of the run (algorithmic 1.205e6: columns and output stay in L2)"},
    "flash_attn_decode": {"bytes": 251.9e6, "launch": "32 rows x 20 heads x 1536 keys (algorithmic 251.7e6)"},
    "flash_attn_ext":    {"bytes": 15.6e6,  "launch": "1500 x 1536 keys x 20 heads (Q + K/V once; K/V re-reads hit L2)"},
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """nvidia-smi clocks / throttle reasons during the timed region."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.rows = index, threading.Event(), []

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.25)

    def summary(self):
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows for i in range(4) if len(r) > 2 + i and r[2 + i].lower().startswith("active")})
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_file(pkg, arch, wtype, rank, barrier):
    d = os.environ.get("B200_MODEL_DIR", "/tmp/b200_models")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{arch}-{wtype}.bin")
    if rank == 0 and not os.path.exists(path):
        tmp = path + ".tmp"
        pkg.synth.write_model(tmp, arch, wtype, seed=0)
        os.replace(tmp, path)
    barrier()
    return path


def make_pcm(pkg, n, first_seed):
    return np.stack([pkg.synth.pcm_f32(pkg.synth.make_clip(first_seed + i, CLIP_SECONDS, n_tones=None, envelopes=True))
                     for i in range(n)])


def timing_table(lib):
    def proc(name, restype, argtypes):
        p = lib.drv_backend_proc(b"B200", name.encode())
        return C.CFUNCTYPE(restype, *argtypes)(p)
    n = proc("b200_timing_classes", C.c_int, [])()
    name = proc("b200_timing_name", C.c_char_p, [C.c_int])
    get = proc("b200_timing_get", None, [C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_double), C.POINTER(C.c_double)])
    out = {}
    for c in range(n):
        cnt, ms, work = C.c_int64(0), C.c_double(0), C.c_double(0)
        get(c, C.byref(cnt), C.byref(ms), C.byref(work))
        if cnt.value:
            out[name(c).decode()] = {"launch_groups": cnt.value, "ms": ms.value, "work": work.value}
    return out


def run_reference(args, pkg):
    """The reference's own CPU implementation (unmodified whisper.cpp + ggml CPU backend, the variant that suits this
    host), rank 0 only.  No library of this repository's kernels is loaded in this process."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    path = model_file(pkg, args.arch, args.wtype, 0, lambda: None)
    w = pkg.Whisper(path, use_gpu=False, flash_attn=True, threads=cores, oracle=False)
    info = w.lib.drv_system_info().decode()
    pcm = make_pcm(pkg, 1, 1000)
    times = []
    for s in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        w.greedy_batch(N_NEW, pcm=pcm, device_mel=False)
        dt = time.perf_counter() - t0
        if s >= args.warmup:
            times.append(dt)
    w.close()
    total = sum(times)
    value = CLIP_SECONDS * len(times) / total
    sample = (f"1 clip per step (log-mel + encoder + {N_NEW} greedy tokens), {cores} threads, {args.warmup} warm-up + {len(times)} timed steps; "
              f"{info.strip()}")
    print(json.dumps({
        "impl": "reference", "metric": "audio_seconds_per_second", "value": value, "unit": "audio-s/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * total / len(times), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "q5_0 weights x q8_0 activations (i8 dot, f32 accumulate)" if args.wtype != "f16" else "f16",
        "data": "synthetic", "config": {"workload": f"whisper {args.arch} {args.wtype}: encode + greedy {N_NEW} tokens per 30 s clip",
                                        "clips_per_step": 1, "l2": "weights (1.1 GB) exceed L2"},
        "cpu_baseline": {"value": value, "unit": "audio-s/s", "cores": cores, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": "audio-s/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_oracle_tokens(args, pkg):
    """Clip 0 of the benchmark batch on the parity oracle (pinned AVX2 build of the reference CPU backend)."""
    cores = len(os.sched_getaffinity(0))
    path = model_file(pkg, args.arch, args.wtype, 0, lambda: None)
    w = pkg.Whisper(path, use_gpu=False, flash_attn=True, threads=cores)
    toks, _ = w.greedy_batch(N_NEW, pcm=make_pcm(pkg, 1, 1000), device_mel=False)
    w.close()
    np.save(args.out, toks[0])


def child(args, impl, extra, timeout=1800):
    """Runs this script again as `--impl <impl>` in a process of its own and returns its stdout."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", impl, "--arch", args.arch, "--wtype", args.wtype, "--n-new", str(N_NEW)] + extra
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)} failed: {r.stderr[-2000:]}")
    return r.stdout


def run_whisper_bench(path, plugin, pkg_dir, host_dir):
    """The reference's own benchmark tool (examples/bench/bench.cpp), unmodified, on the plugin: Enc / Dec / Bch5 / PP in
    ms as scripts/bench-all.sh reports them (encode per run, decode per token, batched per token, prompt per token)."""
    import re
    env = dict(os.environ, LD_PRELOAD=os.path.join(pkg_dir, "libb200_autoload.so"), GGML_BACKEND_PATH=plugin)
    try:
        r = subprocess.run([os.path.join(host_dir, "whisper-bench"), "-m", path, "-t", "1", "-fa"], capture_output=True, text=True, timeout=600, env=env)
    except Exception as e:      # noqa: BLE001
        return {"error": str(e)}
    out = r.stdout + r.stderr
    if r.returncode != 0:
        return {"error": out[-400:]}
    res = {}
    for key, name in (("encode", "enc_ms"), ("decode", "dec_ms"), ("batchd", "bch5_ms"), ("prompt", "pp_ms")):
        m = re.search(rf"{key} time =\s*[\d.]+ ms /\s*\d+ runs \(\s*([\d.]+) ms per run\)", out)
        res[name] = float(m.group(1)) if m else None
    res["device"] = "B200 plugin" if "B200" in out else "unknown (plugin not reported in the tool's log)"
    res["published_v100_large_v2_q5_0"] = {"enc_ms": 89.24, "dec_ms": 6.48, "bch5_ms": 1.48, "pp_ms": 0.11}
    return res


def main():
    global N_NEW
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "oracle-tokens"])
    ap.add_argument("--out", default="", help="--impl oracle-tokens: where the token ids go")
    ap.add_argument("--arch", default="large-v3")
    ap.add_argument("--wtype", default="q5_0")
    ap.add_argument("--clips", type=int, default=TOTAL_CLIPS, help="clips in the whole batch (all ranks)")
    ap.add_argument("--states", type=int, default=0, help="whisper_states (host threads / streams) per GPU; 0 = auto")
    ap.add_argument("--n-new", type=int, default=N_NEW, help="greedy tokens per clip (224 = the benchmark workload; smaller only for profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="timed arms only: no per-operator passes, CPU legs or whisper-bench (parameter sweeps)")
    ap.add_argument("--no-side-output", action="store_true", help="sample from the logits rows read back to the host instead of the plugin's top-k side output")
    args = ap.parse_args()
    N_NEW = args.n_new
    pkg = load_pkg()

    if args.impl == "reference":
        run_reference(args, pkg)
        return
    if args.impl == "oracle-tokens":
        run_oracle_tokens(args, pkg)
        return

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    gpu_index = local
    if world > 1:
        # One process per GPU, and each process sees only its own GPU: whisper.cpp (src/whisper.cpp:1384-1405) always puts
        # the first GPU-type device first in its weight buffer list, so weights would land on device 0 whatever gpu_device
        # says; with a single visible device per process "device 0" is the right one.
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        ids = visible.split(",") if visible else [str(i) for i in range(64)]
        os.environ["CUDA_VISIBLE_DEVICES"] = ids[local]
        gpu_index = int(ids[local]) if ids[local].isdigit() else local
        local = 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cores = len(os.sched_getaffinity(0))
    # one whisper_state per clip, at most 64: their decode steps are merged by the plugin into groups, and several groups
    # in flight keep the device busy while the host threads of the others build their next step
    n_states = args.states or min(64, max(1, args.clips // world))
    path = model_file(pkg, args.arch, args.wtype, rank, barrier)
    clips_rank = args.clips // world
    pcm = make_pcm(pkg, clips_rank, 1000 + rank * clips_rank)
    w = pkg.Whisper(path, use_gpu=True, flash_attn=True, gpu_device=local, n_states=n_states, threads=1)
    lib = w.lib
    # greedy sampling from the plugin's logits side output (top-2 per step) instead of reading 200 KB of logits per state
    # and step back to the host; the full-logits path stays available (--no-side-output)
    side_output = not args.no_side_output
    if side_output:
        pkg.host.logits_side_output(2, skip_readback=True)

    def stat(name):
        return C.CFUNCTYPE(C.c_int64)(lib.drv_backend_proc(b"B200", name.encode()))()

    # inputs of the `value` arm: log-mels prepared once by the device front-end (not timed)
    f = w.filters()
    kl = pkg.kernels_lib()
    kl.b200_mel_create.restype = C.c_void_p
    kl.b200_mel_create.argtypes = [C.c_int, C.c_void_p, C.c_int]
    kl.b200_mel_compute.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    kl.b200_mel_destroy.argtypes = [C.c_void_p]
    plan = kl.b200_mel_create(local, f.ctypes.data, f.shape[0])
    if not plan:
        raise SystemExit("b200_mel_create failed")
    mels = np.empty((clips_rank, w.n_mels, 3000), np.float32)
    tmp = np.empty((w.n_mels, 6000), np.float32)
    for i in range(clips_rank):
        nl, nlo = C.c_int(0), C.c_int(0)
        e = kl.b200_mel_compute(plan, pcm[i].ctypes.data, pcm.shape[1], tmp.ctypes.data, tmp.size, C.byref(nl), C.byref(nlo))
        if e != 0:
            raise SystemExit(f"b200_mel_compute failed: {e}")
        mels[i] = tmp[:, :3000]
    kl.b200_mel_destroy(plan)

    def run_steps(kind):
        """W warm-up + K timed steps; returns (seconds of the timed steps (max over ranks), launches, h2d, d2h)."""
        sampler = ClockSampler(gpu_index)
        times = []
        for s in range(args.warmup + args.steps):
            if s == args.warmup:
                barrier()
                sampler.start()
                l0, h0, d0 = kl.b200_launch_count(), stat("b200_stat_h2d"), stat("b200_stat_d2h")
                ru0 = resource.getrusage(resource.RUSAGE_SELF)
                t0 = time.perf_counter()
            # every call returns when the last state has synchronised its stream and read its last logits back: the host
            # clock brackets all device work of the step (the plugin's streams are not torch's, so torch events see nothing)
            if kind == "value":
                toks, _ = w.greedy_batch(N_NEW, mels=mels)
            else:
                toks, _ = w.greedy_batch(N_NEW, pcm=pcm, device_mel=True)
            if s >= args.warmup:
                timed_tokens.append(toks[0].copy())
        barrier()
        dt = time.perf_counter() - t0
        ru1 = resource.getrusage(resource.RUSAGE_SELF)
        host_cpu[kind] = ((ru1.ru_utime - ru0.ru_utime) + (ru1.ru_stime - ru0.ru_stime)) / dt      # host cores busy in this rank
        sampler.stop_flag.set()
        sampler.join()
        l1, h1, d1 = kl.b200_launch_count(), stat("b200_stat_h2d"), stat("b200_stat_d2h")
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        counts = torch.tensor([l1 - l0, h1 - h0, d1 - d0], device="cuda", dtype=torch.float64)      # whole-job sums
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(counts, op=dist.ReduceOp.SUM)
        n_l, n_h, n_d = (int(v) for v in counts.tolist())
        return float(t.item()), n_l, n_h, n_d, sampler.summary()

    host_cpu = {}
    timed_tokens = []      # clip 0 of every timed step (both arms)
    sec_v, launches, _, _, clocks = run_steps("value")
    if args.quick:
        sec_e, h2d, d2h = sec_v, 0, 0
    else:
        sec_e, _, h2d, d2h, _ = run_steps("e2e")
    audio = CLIP_SECONDS * clips_rank * world * args.steps
    value, e2e = audio / sec_v, audio / sec_e
    # the device mel front-end moves PCM in and the mel out, besides what crosses the plugin boundary
    mel_h2d = pcm.shape[1] * 4 + 400 * 4
    mel_d2h = w.n_mels * 6000 * 4
    h2d_step = h2d / args.steps + clips_rank * world * mel_h2d
    d2h_step = d2h / args.steps + clips_rank * world * mel_d2h

    # Roofline of the dominant kernel: per-operator CUDA events on the backend's own streams (b200_timing_*), two extra
    # passes inside this run.  Encoder-side classes are timed with ONE state on two clips (concurrent states would run
    # their kernels side by side and inflate each other's event times); decode-side classes are timed with all states
    # stepping together, as in the timed region.  Times are reported per clip.
    roof = None
    per_clip = {}
    encoder_ms = None
    if rank == 0 and not args.quick:
        en = C.CFUNCTYPE(None, C.c_int)(lib.drv_backend_proc(b"B200", b"b200_timing_enable"))
        rs = C.CFUNCTYPE(None)(lib.drv_backend_proc(b"B200", b"b200_timing_reset"))
        one = pkg.Whisper.__new__(pkg.Whisper)  # the same context with a single state
        one.__dict__.update(w.__dict__)
        one.states = w.states[:1]
        n_serial = min(2, clips_rank)
        rs(); en(1)
        one.greedy_batch(min(N_NEW, 4), mels=mels[:n_serial])
        en(0)
        t_serial = timing_table(lib)
        # encoder alone: whisper_encode (conv + encoder + cross graphs) of one state with nothing else on the device; the call
        # returns after the backend has synchronised, so the host clock covers launch + device time of the three graphs
        one.set_mel(mels[0])
        enc_ms = []
        for _ in range(6):
            t0 = time.perf_counter()
            if lib.drv_encode(one.ctx, one.states[0], 0, 1) != 0:
                raise SystemExit("whisper_encode failed")
            enc_ms.append(1000.0 * (time.perf_counter() - t0))
        encoder_ms = float(np.median(enc_ms[1:]))
        # decode loop of ONE group (the plugin merges the states of a group): the states meet after their prompt step and
        # timing is switched on there, so encoders and other groups do not run beside the kernels that are timed
        n_batched = min(int(os.environ.get("GGML_B200_MAX_GROUP", "12")), n_states, clips_rank)
        grp = pkg.Whisper.__new__(pkg.Whisper)
        grp.__dict__.update(w.__dict__)
        grp.states = w.states[:n_batched]
        hook_t = C.CFUNCTYPE(None, C.c_int)
        lib.drv_set_decode_phase_hook.argtypes = [C.c_void_p, C.c_int]
        lib.drv_set_decode_phase_hook.restype = None
        rs()
        lib.drv_set_decode_phase_hook(lib.drv_backend_proc(b"B200", b"b200_timing_enable"), n_batched)
        grp.greedy_batch(N_NEW, mels=mels[:n_batched])
        en(0)
        lib.drv_set_decode_phase_hook(None, 0)
        t_batched = timing_table(lib)
        decode_side = ("mul_mat_vec_q", "flash_attn_decode", "norm", "get_rows", "binary")
        for k, v in t_batched.items():
            per_clip[k] = {"launch_groups": v["launch_groups"] / n_batched, "ms": v["ms"] / n_batched, "work": v["work"] / n_batched,
                           "timed": f"decode loop, {n_batched} states stepping together"}
        for k, v in t_serial.items():
            name = k if k not in decode_side else k + " (encoder, prompt and first steps)"
            per_clip[name] = {"launch_groups": v["launch_groups"] / n_serial, "ms": v["ms"] / n_serial, "work": v["work"] / n_serial,
                              "timed": "one state alone"}
        hbm, tf, which = peaks()
        top = max(per_clip.items(), key=lambda kv: kv[1]["ms"])[0] if per_clip else None
        if top:
            r = per_clip[top]
            per_launch_work = r["work"] / r["launch_groups"]
            per_launch_s = r["ms"] / 1000.0 / r["launch_groups"]
            top = top.split(" (")[0]
            if top in ("mul_mat_q", "mul_mat_f16", "flash_attn_ext"):
                ach, peak, unit, bound = per_launch_work / per_launch_s / 1e12, tf, "TFLOP/s", "tensor"
            else:
                ach, peak, unit, bound = per_launch_work / per_launch_s / 1e9, hbm, "GB/s", "hbm"
            roof = {"kernel": top, "bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                    "traffic": TRAFFIC_NCU.get(top), "peak_source": which, "avg_us": per_launch_s * 1e6,
                    "share_of_gpu_time": r["ms"] / sum(v["ms"] for v in per_clip.values()), "timed": r["timed"],
                    "note": LIMITER.get(top)}

    cpu_base, parity, wbench = None, None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.quick:      # reported at N = 1 only
        # the reference arm in a process of its own (its host libraries never share a process with the product's):
        # one warm-up clip, two timed clips
        line = [ln for ln in child(args, "reference", ["--steps", "2", "--warmup", "1"]).splitlines() if ln.startswith("{")][-1]
        cpu_base = json.loads(line)["cpu_baseline"]
        # parity inside the run: clip 0 of every timed step against the parity oracle's ids for the same clip
        tok_file = f"/tmp/b200_bench_oracle_tokens_{os.getpid()}.npy"
        child(args, "oracle-tokens", ["--out", tok_file])
        want = np.load(tok_file)
        os.remove(tok_file)
        equal = min(int((t == want).sum()) for t in timed_tokens)
        parity = {"clip": 0, "tokens_equal": equal, "of": int(len(want)), "timed_steps_checked": len(timed_tokens),
                  "distinct_token_ids": int(len(set(want.tolist()))),
                  "against": "reference CPU backend, pinned AVX2 build (oracle/_ref), same clip, own process"}
    if rank == 0 and world == 1 and not args.quick:
        w.close()
        w = None
        wbench = run_whisper_bench(path, pkg.host.PLUGIN_PATH, pkg.PKG_DIR, pkg.HOST_DIR)
    if w is not None:
        w.close()

    if rank == 0:
        print(json.dumps({
            "metric": "audio_seconds_per_second", "value": value, "unit": "audio-s/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * sec_v / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "q5_0 weights x q8_0 activations (i8 dot, f32 accumulate)" if args.wtype != "f16" else "f16",
            "data": "synthetic",
            "config": {"workload": f"whisper {args.arch} {args.wtype}: encode + greedy {N_NEW} tokens per 30 s clip",
                       "clips_total": clips_rank * world, "clips_per_gpu": clips_rank, "states_per_gpu": n_states, "flash_attn": True,
                       "sampling": "greedy from the plugin's top-k side output (b200_last_topk), logits read-back off" if side_output
                                   else "greedy from the logits rows read back to the host",
                       "l2": "inputs larger than L2: 1.1 GB of weights are streamed per decode step per state",
                       "timed_region": "value: encoder + decoder with the log-mels prepared beforehand; e2e: PCM on the host -> log-mel on the "
                                       "device -> encoder -> decoder -> token ids on the host"},
            "e2e": {"value": e2e, "unit": "audio-s/s", "h2d_bytes_per_step": int(h2d_step), "d2h_bytes_per_step": int(d2h_step),
                    "ms_per_step": 1000.0 * sec_e / args.steps},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu_base,
            "host": {"cpus": os.cpu_count(), "cores_busy_value": round(host_cpu.get("value", 0.0), 2),
                     "cores_busy_e2e": round(host_cpu.get("e2e", 0.0), 2), "threads": n_states},
            "parity_in_run": parity, "encoder_ms_per_30s": encoder_ms, "whisper_bench": wbench,
            "kernel_classes_per_clip": {k: {"launch_groups": round(v["launch_groups"], 1), "ms": round(v["ms"], 3), "timed": v["timed"]}
                                        for k, v in sorted(per_clip.items(), key=lambda kv: -kv[1]["ms"])},
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
