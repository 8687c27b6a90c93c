/*
 * TEST INFRASTRUCTURE ONLY: CPU oracle for the state-space hot path.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may load
 * this library; the shipped CUDA library never does.
 *
 * PARITY UNPINNED for S4/Mamba outputs (see oracle_body.inc): the reference holds no
 * numeric fixture for them and cannot be compiled here; only the primitives are pinned
 * against the reference's two known-answer tests.
 *
 * Build: make -C oracle   ->  oracle/liboracle.so
 * Every function exists as <name>_f32 (the reference's arithmetic) and <name>_f64
 * (shadow copy for error budgeting).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define REAL float
#define SUF f32
#define REAL_IS_DOUBLE 0
#include "oracle_body.inc"
#undef REAL
#undef SUF
#undef REAL_IS_DOUBLE

#define REAL double
#define SUF f64
#define REAL_IS_DOUBLE 1
#include "oracle_body.inc"
#undef REAL
#undef SUF
#undef REAL_IS_DOUBLE

/* Round an f32 to the nearest bf16 (ties to even) and widen it back; NaN stays NaN.
 * Used by the tests to build bf16-exact inputs shared by the oracle and the GPU path. */
void orc_round_bf16(const float *in, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, &in[i], 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) { u |= 0x00400000u; u &= 0xffff0000u; }
        else { u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u; }
        memcpy(&out[i], &u, 4);
    }
}

/* Number of OpenMP threads the parallel loops will use (1 when built without OpenMP). */
#ifdef _OPENMP
#include <omp.h>
int orc_num_threads(void) { return omp_get_max_threads(); }
void orc_set_num_threads(int n) { omp_set_num_threads(n); }
#else
int orc_num_threads(void) { return 1; }
void orc_set_num_threads(int n) { (void)n; }
#endif
