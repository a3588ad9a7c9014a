"""B200-native ggml backend for the whisper.cpp inference hot path.

The product is two shared libraries built from csrc/:
  libb200_kernels.so  sm_100a kernels behind the C ABI of include/b200_whisper.h
  libggml-b200.so     the ggml backend plugin (ggml_backend_init) that whisper.cpp loads
plus libb200_driver.so, a flat C wrapper over whisper.h used by the Python harness (host.py).
"""
from . import synth  # noqa: F401
from .host import Whisper, kernels_lib, load_plugin, PKG_DIR, REF_DIR, HOST_DIR  # noqa: F401
