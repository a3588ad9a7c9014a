"""ctypes bindings: the whisper.h driver (csrc/driver.cpp) and the kernel C ABI (include/b200_whisper.h).

Nothing here computes: every call lands either in the unmodified whisper.cpp host library or in
libb200_kernels.so.  Loading fails loudly when a library is missing.

Two builds of the driver exist and a process uses exactly one of them:
  product  libb200_driver.so, linked against the unmodified reference host libraries in baseline/_ref - what an
           application that loads the plugin looks like (bench.py, smoke);
  oracle   oracle/_ref/libb200_driver_probe.so with the checker's own copy of the reference libraries - the CPU
           backend used as parity oracle, and the probe into whisper_state internals that the tests read.
Loading both would put two copies of libggml / libwhisper into one process, so the second request is refused.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(os.path.dirname(PKG_DIR), "oracle", "_ref")        # checker: oracle CPU backend + probe driver
HOST_DIR = os.path.join(os.path.dirname(PKG_DIR), "baseline", "_ref")     # product: host libraries the driver links
PLUGIN_PATH = os.path.join(PKG_DIR, "libggml-b200.so")

_kernels = None
_drivers = {}


def kernels_lib() -> C.CDLL:
    """libb200_kernels.so with argument types set for the entry points used from Python."""
    global _kernels
    if _kernels is None:
        path = os.path.join(PKG_DIR, "libb200_kernels.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with `make -C {PKG_DIR}/csrc` (no CPU fallback exists)")
        lib = C.CDLL(path)
        lib.b200_launch_count.restype = C.c_int64
        lib.b200_version.restype = C.c_char_p
        _kernels = lib
    return _kernels


def _driver(probe: bool) -> C.CDLL:
    if probe not in _drivers:
        if (not probe) in _drivers:
            raise RuntimeError("this process already loaded the other build of the driver (product vs oracle/probe); "
                               "two copies of the reference host libraries must not share a process")
        path = os.path.join(REF_DIR, "libb200_driver_probe.so") if probe else os.path.join(PKG_DIR, "libb200_driver.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `make -C oracle` and `make -C {PKG_DIR}/csrc`")
        lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        vp, ci, cf = C.c_void_p, C.c_int, C.c_float
        lib.drv_open.restype = vp
        lib.drv_open.argtypes = [C.c_char_p, ci, ci, ci]
        lib.drv_close.argtypes = [vp]
        lib.drv_state_new.restype = vp
        lib.drv_state_new.argtypes = [vp]
        lib.drv_state_free.argtypes = [vp]
        lib.drv_load_backend.argtypes = [C.c_char_p]
        lib.drv_load_host_backends.argtypes = [C.c_char_p]
        if not probe and lib.drv_load_host_backends(HOST_DIR.encode()) < 1:
            raise RuntimeError(f"no CPU backend variant could be loaded from {HOST_DIR} (run `make -C baseline`)")
        lib.drv_backend_proc.restype = vp
        lib.drv_backend_proc.argtypes = [C.c_char_p, C.c_char_p]
        for f in ("drv_n_vocab", "drv_n_mels", "drv_n_audio_state", "drv_n_audio_ctx"):
            getattr(lib, f).argtypes = [vp]
        lib.drv_prefix.argtypes = [vp, C.POINTER(ci)]
        lib.drv_pcm_to_mel.argtypes = [vp, vp, C.c_void_p, ci, ci]
        lib.drv_set_mel.argtypes = [vp, vp, C.c_void_p, ci, ci]
        lib.drv_n_len.argtypes = [vp]
        lib.drv_encode.argtypes = [vp, vp, ci, ci]
        lib.drv_decode.argtypes = [vp, vp, C.c_void_p, ci, ci, ci]
        lib.drv_logits.restype = C.POINTER(cf)
        lib.drv_logits.argtypes = [vp]
        lib.drv_probe_mel.restype = C.c_int64
        lib.drv_probe_mel.argtypes = [vp, C.c_void_p, C.c_int64]
        lib.drv_probe_embd_enc.restype = C.c_int64
        lib.drv_probe_embd_enc.argtypes = [vp, C.c_void_p, C.c_int64]
        lib.drv_greedy.argtypes = [vp, vp, ci, ci, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.drv_full.argtypes = [vp, vp, C.c_void_p, ci, ci, ci, ci, C.c_void_p, ci]
        lib.drv_greedy_batch.argtypes = [vp, C.POINTER(vp), ci, C.c_void_p, C.c_void_p, ci, C.c_void_p, ci, ci, ci, ci, ci,
                                         C.c_void_p, C.POINTER(C.c_double)]
        lib.drv_read_filters.argtypes = [C.c_char_p, C.c_void_p, ci, C.POINTER(ci), C.POINTER(ci)]
        lib.drv_set_mel_compute.argtypes = [vp]
        lib.drv_set_last_topk.argtypes = [vp]
        lib.drv_probe_splits.argtypes = [vp, C.POINTER(ci)]
        lib.drv_probe_graph_nodes.restype = C.c_int64
        lib.drv_probe_graph_nodes.argtypes = [vp, vp, ci]
        lib.drv_system_info.restype = C.c_char_p
        _drivers[probe] = lib
    return _drivers[probe]


def load_plugin(probe: bool = False) -> int:
    """ggml_backend_load(libggml-b200.so); returns the number of B200 devices (0 without a GPU)."""
    lib = _driver(probe)
    if not os.path.exists(PLUGIN_PATH):
        raise RuntimeError(f"{PLUGIN_PATH} is missing (no CPU fallback exists)")
    key = ("plugin", probe)
    if key not in _drivers:
        _drivers[key] = lib.drv_load_backend(PLUGIN_PATH.encode())
    return _drivers[key]


class TopkResult(C.Structure):
    """b200_topk_result of include/b200_whisper.h"""
    _fields_ = [("n", C.c_int32), ("k", C.c_int32), ("max", C.c_float), ("logsumexp", C.c_float),
                ("ids", C.c_int32 * 8), ("vals", C.c_float * 8)]


def logits_side_output(top_k: int, skip_readback: bool = False, probe: bool = False, use_in_driver: bool = True):
    """Switches the plugin's logits side output on (top_k > 0) or off; with use_in_driver the driver's greedy loop samples
    from it (b200_last_topk) instead of scanning whisper_get_logits on the host."""
    lib = _driver(probe)
    fn = lib.drv_backend_proc(b"B200", b"b200_logits_side_output")
    last = lib.drv_backend_proc(b"B200", b"b200_last_topk")
    if not fn or not last:
        raise RuntimeError("the plugin does not offer the logits side output (plugin not loaded?)")
    C.CFUNCTYPE(None, C.c_int, C.c_int)(fn)(int(top_k), int(bool(skip_readback)))
    lib.drv_set_last_topk(C.c_void_p(last if (top_k > 0 and use_in_driver) else None))


def last_topk(row: int = 0, probe: bool = False) -> TopkResult:
    lib = _driver(probe)
    last = lib.drv_backend_proc(b"B200", b"b200_last_topk")
    r = TopkResult()
    rc = C.CFUNCTYPE(C.c_int, C.c_int, C.POINTER(TopkResult))(last)(row, C.byref(r))
    if rc != 0:
        raise RuntimeError(f"b200_last_topk failed: {rc}")
    return r


def backend_stat(name: str, probe: bool = False) -> int:
    lib = _driver(probe)
    p = lib.drv_backend_proc(b"B200", name.encode())
    if not p:
        raise RuntimeError(f"backend proc {name} not found (plugin not loaded?)")
    return C.CFUNCTYPE(C.c_int64)(p)()


class Whisper:
    """One whisper_context (+ states) on the B200 plugin (use_gpu=True) or on the reference CPU backend (use_gpu=False:
    the oracle build unless oracle=False).  probe=True selects the oracle/probe build of the driver for a plugin run."""

    def __init__(self, model_path: str, use_gpu: bool, flash_attn: bool = True, gpu_device: int = 0,
                 probe: bool = False, n_states: int = 1, threads: int | None = None, quiet: bool = True,
                 oracle: bool | None = None):
        # oracle=False with use_gpu=False: the reference CPU path through the product's host libraries (best CPU variant
        # for this host) - what `bench.py --impl reference` times; the parity oracle is the pinned AVX2 build instead
        probe = probe or (oracle if oracle is not None else not use_gpu)
        self.lib = _driver(probe)
        self.probe = probe
        self.model_path = model_path
        self.gpu_device = gpu_device
        self.use_gpu = use_gpu
        self.mel_plans = []
        self.lib.drv_set_quiet(1 if quiet else 0)
        if use_gpu and load_plugin(probe) <= 0:
            raise RuntimeError("B200 plugin exposes no device: refusing to run (there is no CPU fallback in the product path)")
        self.threads = threads or os.cpu_count() or 1
        self.ctx = self.lib.drv_open(model_path.encode(), int(use_gpu), int(flash_attn), gpu_device)
        if not self.ctx:
            raise RuntimeError(f"whisper_init_from_file failed for {model_path}")
        self.states = [self.lib.drv_state_new(self.ctx) for _ in range(n_states)]
        if not all(self.states):
            raise RuntimeError("whisper_init_state failed")
        self.n_vocab = self.lib.drv_n_vocab(self.ctx)
        self.n_mels = self.lib.drv_n_mels(self.ctx)
        self.d = self.lib.drv_n_audio_state(self.ctx)
        self.n_audio_ctx = self.lib.drv_n_audio_ctx(self.ctx)

    def close(self):
        for p in self.mel_plans:
            kernels_lib().b200_mel_destroy(C.c_void_p(p))
        self.mel_plans = []
        for s in self.states:
            self.lib.drv_state_free(s)
        self.states = []
        if self.ctx:
            self.lib.drv_close(self.ctx)
            self.ctx = None

    def prefix(self):
        a = (C.c_int * 4)()
        self.lib.drv_prefix(self.ctx, a)
        return list(a)

    def pcm_to_mel(self, pcm: np.ndarray, state: int = 0) -> np.ndarray:
        pcm = np.ascontiguousarray(pcm, np.float32)
        if self.lib.drv_pcm_to_mel(self.ctx, self.states[state], pcm.ctypes.data, len(pcm), self.threads) != 0:
            raise RuntimeError("whisper_pcm_to_mel failed")
        n = self.lib.drv_probe_mel(self.states[state], None, 0)
        if n <= 0:
            raise RuntimeError(f"mel probe unavailable ({n}); use probe=True")
        out = np.empty((self.n_mels, n // self.n_mels), np.float32)
        self.lib.drv_probe_mel(self.states[state], out.ctypes.data, out.size)
        return out

    def set_mel(self, mel: np.ndarray, state: int = 0):
        mel = np.ascontiguousarray(mel, np.float32)
        assert mel.shape[0] == self.n_mels
        if self.lib.drv_set_mel(self.ctx, self.states[state], mel.ctypes.data, mel.shape[1], mel.shape[0]) != 0:
            raise RuntimeError("whisper_set_mel failed")

    def encode(self, state: int = 0) -> np.ndarray | None:
        if self.lib.drv_encode(self.ctx, self.states[state], 0, self.threads) != 0:
            raise RuntimeError("whisper_encode failed")
        if not self.probe:
            return None
        out = np.empty((self.n_audio_ctx, self.d), np.float32)
        n = self.lib.drv_probe_embd_enc(self.states[state], out.ctypes.data, out.size)
        if n != out.size:
            raise RuntimeError(f"embd_enc probe returned {n}, expected {out.size}")
        return out

    def decode(self, tokens, n_past: int, state: int = 0) -> np.ndarray:
        t = np.ascontiguousarray(tokens, np.int32)
        if self.lib.drv_decode(self.ctx, self.states[state], t.ctypes.data, len(t), n_past, self.threads) != 0:
            raise RuntimeError("whisper_decode failed")
        p = self.lib.drv_logits(self.states[state])
        rows = np.ctypeslib.as_array(p, shape=(len(t), self.n_vocab))
        return rows[len(t) - 1].copy()  # only the last fed token's row is filled (src/whisper.cpp:2960-2966)

    def greedy(self, n_new: int, force=None, state: int = 0, want_logits: bool = False):
        out = np.zeros(n_new, np.int32)
        margins = np.zeros(n_new, np.float32)
        logits = np.zeros((n_new, self.n_vocab), np.float32) if want_logits else None
        f = np.ascontiguousarray(force, np.int32) if force is not None else None
        e = self.lib.drv_greedy(self.ctx, self.states[state], n_new, self.threads,
                                f.ctypes.data if f is not None else None, out.ctypes.data, margins.ctypes.data,
                                logits.ctypes.data if logits is not None else None)
        if e != 0:
            raise RuntimeError(f"drv_greedy failed: {e}")
        return out, margins, logits

    def filters(self) -> np.ndarray:
        """mel filterbank [n_mel, 201] as stored in the model file."""
        buf = np.empty(256 * 201, np.float32)
        nm, nf = C.c_int(0), C.c_int(0)
        if self.lib.drv_read_filters(self.model_path.encode(), buf.ctypes.data, buf.size, C.byref(nm), C.byref(nf)) != 0:
            raise RuntimeError("cannot read mel filters from the model file")
        return buf[: nm.value * nf.value].reshape(nm.value, nf.value).copy()

    def _ensure_mel_plans(self):
        if not self.mel_plans:
            f = self.filters()
            kl = kernels_lib()
            kl.b200_mel_create.restype = C.c_void_p
            kl.b200_mel_create.argtypes = [C.c_int, C.c_void_p, C.c_int]
            kl.b200_mel_destroy.argtypes = [C.c_void_p]
            self.mel_plans = [kl.b200_mel_create(self.gpu_device, f.ctypes.data, f.shape[0]) for _ in self.states]
            if not all(self.mel_plans):
                raise RuntimeError("b200_mel_create failed (no CUDA device?)")
            # the driver's worker threads call the device front-end through this pointer
            self.lib.drv_set_mel_compute(C.cast(kl.b200_mel_compute, C.c_void_p))

    def greedy_batch(self, n_new: int, mels: np.ndarray | None = None, pcm: np.ndarray | None = None, device_mel: bool = True):
        """Encode + greedy-decode a batch of clips spread over all states.
        mels [n_clips, n_mel, n_len] or pcm [n_clips, n_samples] (mel on the B200 when device_mel, else
        whisper_pcm_to_mel on host threads).  Returns (tokens [n_clips, n_new], seconds)."""
        arr = (C.c_void_p * len(self.states))(*self.states)
        secs = C.c_double(0)
        if pcm is not None:
            pcm = np.ascontiguousarray(pcm, np.float32)
            n_clips, n_samples = pcm.shape
            toks = np.zeros((n_clips, n_new), np.int32)
            plans = None
            if device_mel:
                self._ensure_mel_plans()
                plans = (C.c_void_p * len(self.mel_plans))(*self.mel_plans)
            e = self.lib.drv_greedy_batch(self.ctx, arr, len(self.states), plans, pcm.ctypes.data, n_samples, None, 0, self.n_mels,
                                          n_clips, n_new, self.threads, toks.ctypes.data, C.byref(secs))
        else:
            mels = np.ascontiguousarray(mels, np.float32)
            n_clips, n_mel, n_len = mels.shape
            toks = np.zeros((n_clips, n_new), np.int32)
            e = self.lib.drv_greedy_batch(self.ctx, arr, len(self.states), None, None, 0, mels.ctypes.data, n_len, n_mel,
                                          n_clips, n_new, self.threads, toks.ctypes.data, C.byref(secs))
        if e != 0:
            raise RuntimeError(f"drv_greedy_batch failed: {e}")
        return toks, secs.value

    def sched_splits(self, state: int = 0):
        """Splits of the last conv / encoder / cross / decoder graph of a state (probe build); 1 = one backend ran it all."""
        a = (C.c_int * 4)()
        if self.lib.drv_probe_splits(self.states[state], a) != 0:
            raise RuntimeError("scheduler probe unavailable; use probe=True")
        return list(a)

    def graph_nodes(self, which: int, state: int = 0) -> int:
        """Computing nodes of the conv (0) / encoder (1) / cross (2) / last decoder (3) graph of a state (probe build)."""
        n = self.lib.drv_probe_graph_nodes(self.ctx, self.states[state], which)
        if n < 0:
            raise RuntimeError(f"graph probe unavailable ({n}); use probe=True")
        return int(n)

    def full(self, pcm: np.ndarray | None, beam_size: int = 1, max_tokens: int = 0, state: int = 0):
        out = np.zeros(1024, np.int32)
        if pcm is not None:
            pcm = np.ascontiguousarray(pcm, np.float32)
        n = self.lib.drv_full(self.ctx, self.states[state], pcm.ctypes.data if pcm is not None else None,
                              len(pcm) if pcm is not None else 0, beam_size, max_tokens, self.threads, out.ctypes.data, len(out))
        if n < 0:
            raise RuntimeError("whisper_full failed")
        return out[:min(n, len(out))].copy()
