// Pre-load shim for UNMODIFIED reference executables (whisper-bench, whisper-cli) that were linked against host
// libraries with dynamically loaded backends: it asks the registry to load every backend it can find before main()
// runs - the CPU variants next to the executable and the out-of-tree backend named by GGML_BACKEND_PATH
// (ggml_backend_load_all, ggml/src/ggml-backend-reg.cpp:558-586).  The reference's own examples call whisper_init_*
// first, which looks for the CPU device before anything has been loaded (src/whisper.cpp:1384-1425); loading from a
// static initialiser is one of the registry's supported ways in and needs no change to the executable.
//
//   LD_PRELOAD=libb200_autoload.so GGML_BACKEND_PATH=/path/to/libggml-b200.so whisper-bench -m model.bin
#include "ggml-backend.h"

__attribute__((constructor)) static void b200_autoload(void) { ggml_backend_load_all(); }
