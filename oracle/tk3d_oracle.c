/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the torkit3d hot path (see tk3d_oracle_impl.h).
 *
 * Build (the Makefile beside this file does it):
 *   gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared tk3d_oracle.c -o libtk3d_oracle.so -lm
 *
 * -ffp-contract=off is mandatory: the parity contract is "no fused multiply-add".
 * Pinning: the reference stores no golden vectors; this oracle is pinned against fixtures produced
 * by the reference's own Python brute-force formulations (tests/golden/make_golden.py imports them
 * from the reference checkout) and, on a GPU box, against the reference CUDA extension compiled
 * with -fmad=false (oracle/build_ref.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define T float
#define SUFFIX _f32
#define ORC_T_IS_FLOAT 1
#include "tk3d_oracle_impl.h"
#undef ORC_T_IS_FLOAT
#undef T
#undef SUFFIX

#define T double
#define SUFFIX _f64
#include "tk3d_oracle_impl.h"
#undef T
#undef SUFFIX

int orc_version(void) { return 1; }
