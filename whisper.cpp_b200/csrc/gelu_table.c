/* GELU lookup table of the reference CPU backend (ggml/src/ggml-cpu/ggml-cpu.c:3398-3421,
 * ggml/src/ggml-cpu/vec.h:428-457): entry h = f16(gelu_tanh(f32(h))) for every f16 bit pattern.
 * Built on the host with the same expression, libm tanhf and F16C conversions, compiled with the
 * same floating-point options (-O3 -mfma, GNU C mode), so that the table matches the one the CPU
 * backend builds at start-up. */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>

static const float GELU_COEF_A    = 0.044715f;
static const float SQRT_2_OVER_PI = 0.79788456080286535587989211986876f;

static inline float gelu_f32(float x) {
    return 0.5f*x*(1.0f + tanhf(SQRT_2_OVER_PI*x*(1.0f + GELU_COEF_A*x*x)));
}

void b200_build_gelu_table(uint16_t * table) {
    for (int i = 0; i < (1 << 16); ++i) {
        const float f = _cvtsh_ss((uint16_t) i);
        table[i] = _cvtss_sh(gelu_f32(f), 0);
    }
}
