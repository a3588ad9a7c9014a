"""CPU-only checks of the host side: the C-ABI library loads without a GPU and exports every symbol the
header declares, the plugin refuses to load without a device, the plane layout round-trips, and the
clip sharding over ranks (gloo, world size 2) covers the batch exactly once."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import ref_ops as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "whisper.cpp_b200")


def test_kernel_library_exports_every_declared_symbol(pkg):
    lib = pkg.kernels_lib()
    header = open(os.path.join(ROOT, "include", "b200_whisper.h")).read()
    code = re.sub(r"/\*.*?\*/", "", header, flags=re.S)           # declarations only; comments name plugin procs too
    names = sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", code)))
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert b"sm_100a" in lib.b200_version()
    # the optional entry points the header documents for the plugin are exported by the plugin
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(PKG, "libggml-b200.so")], capture_output=True, text=True).stdout
    for proc in ("b200_logits_side_output", "b200_last_topk"):
        assert proc in header and f" {proc}" in out


def test_plugin_exports_entry_points_and_refuses_without_gpu():
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(PKG, "libggml-b200.so")], capture_output=True, text=True).stdout
    assert " ggml_backend_init" in out and " ggml_backend_score" in out
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu and R.have_ref():
        assert R.load_plugin() == 0      # score 0: no device, no CPU fallback


@pytest.mark.parametrize("t,bs", [(6, 22), (8, 34)])
def test_plane_layout_roundtrip(pkg, t, bs):
    lib = pkg.kernels_lib()
    nb = 37
    blocks = np.random.default_rng(0).integers(0, 256, (nb, bs), dtype=np.uint8)
    planes = np.zeros(nb * bs, np.uint8)
    back = np.zeros_like(blocks)
    i64 = C.c_int64
    assert lib.b200_blocks_to_planes(t, blocks.ctypes.data_as(C.c_void_p), planes.ctypes.data_as(C.c_void_p), i64(nb), i64(0), i64(nb)) == 0
    assert lib.b200_planes_to_blocks(t, planes.ctypes.data_as(C.c_void_p), back.ctypes.data_as(C.c_void_p), i64(nb), i64(0), i64(nb)) == 0
    assert np.array_equal(blocks, back)
    qs = 16 if t == 6 else 32
    assert np.array_equal(planes[:qs], blocks[0, bs - qs:])            # first plane = packed quants of block 0
    assert np.array_equal(planes[-2:], blocks[-1, :2])                 # last plane = scales
    # partial range lands in the same place
    part = np.zeros(nb * bs, np.uint8)
    assert lib.b200_blocks_to_planes(t, blocks[5:9].ctypes.data_as(C.c_void_p), part.ctypes.data_as(C.c_void_p), i64(nb), i64(5), i64(4)) == 0
    assert np.array_equal(part[qs * 5: qs * 9], planes[qs * 5: qs * 9])
    assert lib.b200_blocks_to_planes(t, blocks.ctypes.data_as(C.c_void_p), planes.ctypes.data_as(C.c_void_p), i64(nb), i64(30), i64(10)) != 0


def test_clip_generator_is_seeded(pkg):
    a, b = pkg.synth.make_clip(5, 1.0), pkg.synth.make_clip(5, 1.0)
    assert a.dtype == np.int16 and np.array_equal(a, b) and not np.array_equal(a, pkg.synth.make_clip(6, 1.0))
    c = pkg.synth.make_clip(9, 1.0, n_tones=None, envelopes=True)
    assert c.shape == (16000,) and np.abs(c).max() > 1000


def test_sharding_two_ranks_gloo(tmp_path):
    """Strong-scaling split used by bench.py: rank r owns clips [r*n/W, (r+1)*n/W); checked with 2 gloo ranks."""
    script = tmp_path / "shard.py"
    script.write_text(
        "import os, torch, torch.distributed as dist\n"
        "dist.init_process_group('gloo')\n"
        "r, w = dist.get_rank(), dist.get_world_size()\n"
        "n = 64; per = n // w\n"
        "mine = torch.zeros(n, dtype=torch.int64); mine[r*per:(r+1)*per] = 1\n"
        "seeds = torch.zeros(n, dtype=torch.int64); seeds[r*per:(r+1)*per] = torch.arange(1000 + r*per, 1000 + (r+1)*per)\n"
        "dist.all_reduce(mine); dist.all_reduce(seeds)\n"
        "t = torch.tensor([1.0 + r]); dist.all_reduce(t, op=dist.ReduceOp.MAX)\n"
        "assert mine.tolist() == [1]*n and seeds.tolist() == list(range(1000, 1064)) and t.item() == float(w)\n"
        "dist.destroy_process_group()\n")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29531", str(script)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]


def test_static_scratch_entry_point_rejects_bad_arguments_without_a_device(pkg):
    """b200_mul_mat_q_static validates everything before its first launch, so bad arguments come back as error codes on
    a machine without a GPU as well (no device access happens)."""
    lib = pkg.kernels_lib()
    i64, vp = C.c_int64, C.c_void_p
    buf = np.zeros(1 << 16, np.uint8)
    p = buf.ctypes.data + (-buf.ctypes.data % 256)
    ok = dict(w=vp(p), nb=i64(64 * 2), M=i64(64), K=i64(64), x=vp(p + 4096), xs=i64(256), N=i64(4), dst=vp(p + 8192), ds=i64(64))

    def call(**kw):
        a = dict(ok, **kw)
        return lib.b200_mul_mat_q_static(6, a["w"], a["nb"], a["M"], a["K"], a["x"], a["xs"], a["N"], a["dst"], a["ds"], None)
    assert call(x=None) == 10001 and call(dst=None) == 10001 and call(w=None) == 10001
    assert call(w=vp(p + 4)) == 10001                      # weights not 16-byte aligned
    assert call(xs=i64(128)) == 10001                      # row stride shorter than a row
    assert call(ds=i64(32)) == 10001                       # destination stride shorter than M
    assert call(nb=i64(64)) == 10001                       # weight tensor smaller than M x K
    assert call(N=i64(1 << 60)) == 10003                   # absurd N: too large, and no overflow on the way
    assert call(K=i64(48)) == 10001


@pytest.mark.skipif(not R.have_ref(), reason="reference build (oracle/_ref) missing")
def test_truncated_model_file_fails_cleanly(pkg, tmp_path):
    """A model file cut off in the middle of its tensors makes whisper_init_* return NULL (the loader's own checks,
    src/whisper.cpp:1874-1960); the harness turns that into an exception, nothing crashes."""
    good = tmp_path / "tiny.bin"
    pkg.synth.write_model(str(good), "tiny", "q5_0", seed=0)
    data = good.read_bytes()
    bad = tmp_path / "cut.bin"
    bad.write_bytes(data[: len(data) // 2])
    with pytest.raises(RuntimeError):
        pkg.Whisper(str(bad), use_gpu=False)
    bad.write_bytes(data[: len(data) * 3 // 4 + 5])          # cut inside a tensor's data
    with pytest.raises(RuntimeError):
        pkg.Whisper(str(bad), use_gpu=False)


@pytest.mark.skipif(not R.have_ref(), reason="reference build (oracle/_ref) missing")
def test_cached_plan_is_refused_for_a_graph_with_other_consumers():
    """Plans are cached by a signature of operators, types and shapes.  Two graphs with the same signature: in one the
    product feeds only the bias addition (the plugin fuses them), in the other a later node reads the product itself, so
    the product must reach memory.  The plugin has to refuse the cached fused plan for the second graph (no device work:
    the plugin's test hook only builds and compares plans)."""
    lib = R.lib()
    lib.oph_plan_probe.argtypes = [C.c_char_p, C.c_int]
    same = lib.oph_plan_probe(R.PLUGIN.encode(), 0)
    other = lib.oph_plan_probe(R.PLUGIN.encode(), 1)
    assert same >= 0 and other >= 0, (same, other)       # -1: signatures differ (the test graphs would be wrong), -10/-11: set-up
    assert same & 2 and other & 2, "the product + bias pair is expected to be fused"
    assert same & 1, "an identical graph must fit its own plan"
    assert not (other & 1), "a graph whose product has a second consumer must not run on the fused plan"
