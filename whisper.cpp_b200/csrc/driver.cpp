// Host driver over the public whisper.h API (include/whisper.h of the reference), with flat C entry
// points that a Python harness can call through ctypes.  It is the caller side of the drop-in: it
// loads the B200 plugin with ggml_backend_load() and then uses whisper_init_*, whisper_set_mel,
// whisper_encode, whisper_decode and whisper_full exactly as any whisper.cpp application does.
//
// Two builds of this one file:
//   default           links the unmodified libwhisper.so and uses only whisper.h;
//   -DDRV_WITH_PROBE  compiles the unmodified src/whisper.cpp into the same translation unit so that a
//                     test can read whisper_state::embd_enc (the encoder output has no public getter).
#ifdef DRV_WITH_PROBE
#include "whisper.cpp"
#else
#include "whisper.h"
#include "ggml-backend.h"
#endif

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <condition_variable>
#include <mutex>
#include <vector>

extern "C" {

static void drv_quiet_log(enum ggml_log_level level, const char * text, void *) {
    if (level == GGML_LOG_LEVEL_ERROR || level == GGML_LOG_LEVEL_WARN) fputs(text, stderr);
}

void drv_set_quiet(int quiet) {
    if (quiet) whisper_log_set(drv_quiet_log, nullptr);
    else       whisper_log_set(nullptr, nullptr);
}

// Host libraries built with dynamically loaded backends (baseline/Makefile) find their CPU backend variants next to
// the executable; a process whose executable is an interpreter points the registry at the library directory instead.
// Returns the number of registered backends afterwards.
int drv_load_host_backends(const char * dir) {
    ggml_backend_load_all_from_path(dir);
    return (int) ggml_backend_reg_count();
}

// Registers the plugin; returns the number of devices it exposes (0 = load failed / no GPU).
int drv_load_backend(const char * path) {
    ggml_backend_reg_t reg = ggml_backend_load(path);
    if (!reg) return 0;
    return (int) ggml_backend_reg_dev_count(reg);
}

void * drv_backend_proc(const char * reg_name, const char * proc) {
    ggml_backend_reg_t reg = ggml_backend_reg_by_name(reg_name);
    return reg ? ggml_backend_reg_get_proc_address(reg, proc) : nullptr;
}

void * drv_open(const char * model_path, int use_gpu, int flash_attn, int gpu_device) {
    struct whisper_context_params cp = whisper_context_default_params();
    cp.use_gpu    = use_gpu != 0;
    cp.flash_attn = flash_attn != 0;
    cp.gpu_device = gpu_device;
    return whisper_init_from_file_with_params_no_state(model_path, cp);
}
void   drv_close(void * ctx)       { whisper_free((struct whisper_context *) ctx); }
void * drv_state_new(void * ctx)   { return whisper_init_state((struct whisper_context *) ctx); }
void   drv_state_free(void * st)   { whisper_free_state((struct whisper_state *) st); }

int drv_n_vocab(void * ctx)     { return whisper_n_vocab((struct whisper_context *) ctx); }
int drv_n_mels(void * ctx)      { return whisper_model_n_mels((struct whisper_context *) ctx); }
int drv_n_audio_state(void * ctx) { return whisper_model_n_audio_state((struct whisper_context *) ctx); }
int drv_n_audio_ctx(void * ctx) { return whisper_model_n_audio_ctx((struct whisper_context *) ctx); }

// forced prefix [SOT, lang=en, transcribe, notimestamps]
int drv_prefix(void * vctx, int * out4) {
    struct whisper_context * ctx = (struct whisper_context *) vctx;
    out4[0] = whisper_token_sot(ctx);
    out4[1] = whisper_token_lang(ctx, whisper_lang_id("en"));
    out4[2] = whisper_token_transcribe(ctx);
    out4[3] = whisper_token_not(ctx);
    return 4;
}

int drv_pcm_to_mel(void * ctx, void * st, const float * pcm, int n, int threads) {
    return whisper_pcm_to_mel_with_state((struct whisper_context *) ctx, (struct whisper_state *) st, pcm, n, threads);
}
int drv_set_mel(void * ctx, void * st, const float * mel, int n_len, int n_mel) {
    return whisper_set_mel_with_state((struct whisper_context *) ctx, (struct whisper_state *) st, mel, n_len, n_mel);
}
int drv_n_len(void * st) { return whisper_n_len_from_state((struct whisper_state *) st); }
int drv_encode(void * ctx, void * st, int offset, int threads) {
    return whisper_encode_with_state((struct whisper_context *) ctx, (struct whisper_state *) st, offset, threads);
}
int drv_decode(void * ctx, void * st, const int * tokens, int n, int n_past, int threads) {
    return whisper_decode_with_state((struct whisper_context *) ctx, (struct whisper_state *) st, tokens, n, n_past, threads);
}
const float * drv_logits(void * st) { return whisper_get_logits_from_state((struct whisper_state *) st); }

// mel spectrogram held by the state: needs the probe build (no public getter)
int64_t drv_probe_mel(void * st, float * out, int64_t cap) {
#ifdef DRV_WITH_PROBE
    struct whisper_state * s = (struct whisper_state *) st;
    const int64_t n = (int64_t) s->mel.data.size();
    if (out && cap >= n) memcpy(out, s->mel.data.data(), n * sizeof(float));
    return n;
#else
    (void) st; (void) out; (void) cap;
    return -1;
#endif
}

// encoder output [n_audio_state, n_audio_ctx] f32 of the last whisper_encode call (probe build only)
int64_t drv_probe_embd_enc(void * st, float * out, int64_t cap) {
#ifdef DRV_WITH_PROBE
    struct whisper_state * s = (struct whisper_state *) st;
    if (!s->embd_enc) return -2;
    const int64_t n = ggml_nelements(s->embd_enc);
    if (out && cap >= n) ggml_backend_tensor_get(s->embd_enc, out, 0, n * sizeof(float));
    return n;
#else
    (void) st; (void) out; (void) cap;
    return -1;
#endif
}

// Scheduler evidence (probe build only): number of splits of the last graph each of the state's four schedulers ran
// (conv, encoder, cross, decoder).  One split = the whole graph went to a single backend.
int drv_probe_splits(void * st, int * out4) {
#ifdef DRV_WITH_PROBE
    struct whisper_state * s = (struct whisper_state *) st;
    out4[0] = ggml_backend_sched_get_n_splits(s->sched_conv.sched);
    out4[1] = ggml_backend_sched_get_n_splits(s->sched_encode.sched);
    out4[2] = ggml_backend_sched_get_n_splits(s->sched_cross.sched);
    out4[3] = ggml_backend_sched_get_n_splits(s->sched_decode.sched);
    return 0;
#else
    (void) st; (void) out4;
    return -1;
#endif
}

// Number of computing nodes (not views, not empty) of a graph as whisper.cpp builds it for this state (probe build only):
// which = 0 conv, 1 encoder, 2 cross, 3 decoder for the batch of the state's last whisper_decode call.  Only the graph
// description is rebuilt in the scheduler's metadata buffer; nothing is allocated or computed.
int64_t drv_probe_graph_nodes(void * vctx, void * st, int which) {
#ifdef DRV_WITH_PROBE
    struct whisper_context * ctx = (struct whisper_context *) vctx;
    struct whisper_state * s = (struct whisper_state *) st;
    struct ggml_cgraph * g = nullptr;
    if (which == 0)      g = whisper_build_graph_conv(*ctx, *s);
    else if (which == 1) g = whisper_build_graph_encoder(*ctx, *s);
    else if (which == 2) g = whisper_build_graph_cross(*ctx, *s);
    else if (which == 3) g = whisper_build_graph_decoder(*ctx, *s, s->batch, false, false);
    if (!g) return -2;
    int64_t n = 0;
    for (int i = 0; i < ggml_graph_n_nodes(g); ++i) {
        const struct ggml_tensor * t = ggml_graph_node(g, i);
        const bool view = t->op == GGML_OP_NONE || t->op == GGML_OP_RESHAPE || t->op == GGML_OP_VIEW || t->op == GGML_OP_PERMUTE || t->op == GGML_OP_TRANSPOSE;
        if (!view && !ggml_is_empty(t)) ++n;
    }
    return n;
#else
    (void) vctx; (void) st; (void) which;
    return -1;
#endif
}

static int argmax_f32(const float * x, int n) {
    int best = 0;
    float bv = x[0];
    for (int i = 1; i < n; ++i) if (x[i] > bv) { bv = x[i]; best = i; }
    return best;
}

// encode (mel must be set) + forced prefix + greedy decode of n_new tokens through whisper_decode,
// argmax on the host over the raw logits; EOT is not special, so every clip costs the same work.
// If force != NULL the fed-back token at step i is force[i] (teacher forcing) while out[i] still
// reports this run's argmax.  margins (optional) receives top1-top2 of every step; logits_out
// (optional) receives the raw logits of every step, n_vocab floats each.
// Admission gate for encoders: at most `limit` states run whisper_encode at a time (0 = no limit), so that the rest of
// the states keep decoding together while a few encoders fill the GPU, instead of all states encoding, then all decoding.
struct enc_gate {
    std::mutex mu;
    std::condition_variable cv;
    int limit = 0, busy = 0;
    void enter() { if (limit <= 0) return; std::unique_lock<std::mutex> lk(mu); cv.wait(lk, [&] { return busy < limit; }); ++busy; }
    void leave() { if (limit <= 0) return; { std::lock_guard<std::mutex> lk(mu); --busy; } cv.notify_one(); }
};
static enc_gate g_enc_gate;

// Measurement aid: when a hook is set, the states of a batch meet after their prompt step and the last one to arrive
// calls hook(1) before anybody takes the first single-token step (per-operator timing of the decode loop alone).
static void (*g_phase_hook)(int) = nullptr;
static int g_phase_parties = 0, g_phase_arrived = 0;
static std::mutex g_phase_mu;
static std::condition_variable g_phase_cv;
void drv_set_decode_phase_hook(void (*hook)(int), int parties) {
    std::lock_guard<std::mutex> lk(g_phase_mu);
    g_phase_hook = hook; g_phase_parties = parties; g_phase_arrived = 0;
}
static void decode_phase_meet() {
    std::unique_lock<std::mutex> lk(g_phase_mu);
    if (!g_phase_hook || g_phase_parties <= 0) return;
    if (++g_phase_arrived >= g_phase_parties) { g_phase_hook(1); g_phase_cv.notify_all(); }
    // bounded: a state that failed before the meeting point must not leave the others waiting for ever
    else g_phase_cv.wait_for(lk, std::chrono::seconds(120), [&] { return g_phase_arrived >= g_phase_parties || !g_phase_hook; });
}

// Optional: sample from the plugin's logits side output (get_proc_address "b200_last_topk", include/b200_whisper.h)
// instead of scanning the row whisper_get_logits returns.  fn = NULL switches back to the host scan.
struct drv_topk_result { int32_t n, k; float max, logsumexp; int32_t ids[8]; float vals[8]; };
typedef int (*drv_last_topk_fn)(int row, drv_topk_result * out);
static drv_last_topk_fn g_last_topk = nullptr;
void drv_set_last_topk(void * fn) { g_last_topk = (drv_last_topk_fn) fn; }

int drv_greedy(void * vctx, void * vst, int n_new, int threads, const int * force, int * out, float * margins, float * logits_out) {
    struct whisper_context * ctx = (struct whisper_context *) vctx;
    struct whisper_state *   st  = (struct whisper_state *) vst;
    g_enc_gate.enter();
    const int enc = whisper_encode_with_state(ctx, st, 0, threads);
    g_enc_gate.leave();
    if (enc != 0) return -1;
    int prefix[4];
    drv_prefix(ctx, prefix);
    const int n_vocab = whisper_n_vocab(ctx);
    if (whisper_decode_with_state(ctx, st, prefix, 4, 0, threads) != 0) return -2;
    decode_phase_meet();
    int n_past = 4;
    for (int i = 0; i < n_new; ++i) {
        // logits of the last fed token: row n_tokens-1 of the state's logits buffer
        const float * lg = whisper_get_logits_from_state(st) + (i == 0 ? (size_t) 3 * n_vocab : 0);
        if (g_last_topk && !logits_out) {
            drv_topk_result r;
            if (g_last_topk(i == 0 ? 3 : 0, &r) != 0 || r.n != n_vocab || r.k < 2) return -4;
            out[i] = r.ids[0];
            if (margins) margins[i] = r.vals[0] - r.vals[1];
            if (i + 1 == n_new) break;
            const int feed = force ? force[i] : r.ids[0];
            if (whisper_decode_with_state(ctx, st, &feed, 1, n_past, threads) != 0) return -3;
            ++n_past;
            continue;
        }
        const int tok = argmax_f32(lg, n_vocab);
        out[i] = tok;
        if (margins) {
            float second = -INFINITY;
            for (int j = 0; j < n_vocab; ++j) if (j != tok && lg[j] > second) second = lg[j];
            margins[i] = lg[tok] - second;
        }
        if (logits_out) memcpy(logits_out + (size_t) i * n_vocab, lg, sizeof(float) * n_vocab);
        if (i + 1 == n_new) break;
        const int feed = force ? force[i] : tok;
        if (whisper_decode_with_state(ctx, st, &feed, 1, n_past, threads) != 0) return -3;
        ++n_past;
    }
    return 0;
}

// whisper_full on PCM (or on the mel already set in the state when pcm == NULL), beam or greedy,
// temperature 0 with no fallback ladder; returns the number of tokens written to out.
int drv_full(void * vctx, void * vst, const float * pcm, int n_samples, int beam_size, int max_tokens, int threads, int * out, int cap) {
    struct whisper_context * ctx = (struct whisper_context *) vctx;
    struct whisper_state *   st  = (struct whisper_state *) vst;
    struct whisper_full_params p = whisper_full_default_params(beam_size > 1 ? WHISPER_SAMPLING_BEAM_SEARCH : WHISPER_SAMPLING_GREEDY);
    p.n_threads        = threads;
    p.print_progress   = false;
    p.print_realtime   = false;
    p.print_timestamps = false;
    p.print_special    = false;
    p.no_context       = true;
    p.no_timestamps    = true;
    p.single_segment   = true;
    p.suppress_blank   = true;
    p.language         = "en";
    p.temperature      = 0.0f;
    p.temperature_inc  = 0.0f;
    p.max_tokens       = max_tokens;
    if (beam_size > 1) p.beam_search.beam_size = beam_size;
    else               p.greedy.best_of = 1;
    if (whisper_full_with_state(ctx, st, p, pcm, pcm ? n_samples : 0) != 0) return -1;
    int n = 0;
    const int n_seg = whisper_full_n_segments_from_state(st);
    for (int s = 0; s < n_seg; ++s) {
        const int nt = whisper_full_n_tokens_from_state(st, s);
        for (int t = 0; t < nt; ++t) {
            if (n < cap) out[n] = whisper_full_get_token_id_from_state(st, s, t);
            ++n;
        }
    }
    return n;
}

// Mel filterbank stored in a legacy ggml model file (header layout: src/whisper.cpp:1508-1607).
// whisper.h has no getter for it; an application that computes the mel itself reads it from the file.
int drv_read_filters(const char * model_path, float * out, int cap, int * n_mel, int * n_fft) {
    FILE * f = fopen(model_path, "rb");
    if (!f) return -1;
    uint32_t magic = 0;
    int32_t hp[11];
    int32_t nm = 0, nf = 0;
    int rc = -2;
    if (fread(&magic, 4, 1, f) == 1 && magic == 0x67676d6c && fread(hp, 4, 11, f) == 11 && fread(&nm, 4, 1, f) == 1 && fread(&nf, 4, 1, f) == 1) {
        *n_mel = nm; *n_fft = nf;
        if (nm > 0 && nf > 0 && (int64_t) nm * nf <= cap && fread(out, 4, (size_t) nm * nf, f) == (size_t) nm * nf) rc = 0;
    }
    fclose(f);
    return rc;
}

// The device log-mel front-end (b200_mel_compute of libb200_kernels.so, include/b200_whisper.h) is handed in as a
// function pointer by the caller that loaded the kernel library, so that this driver links nothing but the
// reference's own host libraries.
typedef int (*drv_mel_compute_fn)(void * plan, const float * pcm_host, int64_t n_samples, float * out_host, int64_t out_capacity, int * n_len, int * n_len_org);
static drv_mel_compute_fn g_mel_compute = nullptr;
void drv_set_mel_compute(void * fn) { g_mel_compute = (drv_mel_compute_fn) fn; }

// A batch of clips on one context: n_states worker threads, each with its own whisper_state (and so
// its own backend stream), pull clips from a shared counter.  Input is either PCM
// [n_clips][n_samples] (mel computed per clip: on the device when mel_plans != NULL, else by
// whisper_pcm_to_mel on the host threads) or ready mels [n_clips][n_mel][n_len] when pcm == NULL.
// tokens_out = [n_clips][n_new].  Returns 0 or the first error; *seconds = wall time of the batch.
int drv_greedy_batch(void * vctx, void ** states, int n_states, void ** mel_plans, const float * pcm, int n_samples,
                     const float * mels, int n_len, int n_mel, int n_clips, int n_new, int threads, int * tokens_out, double * seconds) {
    struct whisper_context * ctx = (struct whisper_context *) vctx;
    std::atomic<int> next{0}, err{0};
    g_enc_gate.limit = getenv("DRV_MAX_ENC") ? atoi(getenv("DRV_MAX_ENC")) : 0;
    const auto t0 = std::chrono::steady_clock::now();
    auto work = [&](int w) {
        struct whisper_state * st = (struct whisper_state *) states[w];
        std::vector<float> melbuf;
        for (;;) {
            const int c = next.fetch_add(1);
            if (c >= n_clips || err.load()) break;
            if (pcm) {
                const float * x = pcm + (size_t) c * n_samples;
                if (mel_plans) {
                    if (!g_mel_compute) { err = -12; break; }
                    const int64_t cap = (int64_t) n_mel * ((n_samples + 480000 + 400 - 400) / 160);
                    if ((int64_t) melbuf.size() < cap) melbuf.resize(cap);
                    int nl = 0, nlo = 0;
                    const int e = g_mel_compute(mel_plans[w], x, n_samples, melbuf.data(), cap, &nl, &nlo);
                    if (e) { err = -20 - (e & 0xff); break; }
                    if (whisper_set_mel_with_state(ctx, st, melbuf.data(), nl, n_mel) != 0) { err = -10; break; }
                } else {
                    if (whisper_pcm_to_mel_with_state(ctx, st, x, n_samples, threads) != 0) { err = -11; break; }
                }
            } else {
                if (whisper_set_mel_with_state(ctx, st, mels + (size_t) c * n_len * n_mel, n_len, n_mel) != 0) { err = -10; break; }
            }
            const int e = drv_greedy(ctx, st, n_new, threads, nullptr, tokens_out + (size_t) c * n_new, nullptr, nullptr);
            if (e) { err = e; break; }
        }
    };
    std::vector<std::thread> pool;
    for (int w = 1; w < n_states; ++w) pool.emplace_back(work, w);
    work(0);
    for (auto & t : pool) t.join();
    if (seconds) *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return err.load();
}

const char * drv_system_info(void) { return whisper_print_system_info(); }

}
