/*
 * CPU restatement of sphericart's harmonics evaluation. TEST INFRASTRUCTURE ONLY
 * (see sph_oracle.h). The body is instantiated once per floating-point type.
 */
#include "sph_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#else
static int omp_get_max_threads(void) { return 1; }
static int omp_get_thread_num(void) { return 0; }
#endif

#define REAL double
#define SUFFIX(name) name##_f64
#define REAL_SQRT sqrt
#include "sph_oracle_body.inc"
#undef REAL
#undef SUFFIX
#undef REAL_SQRT

#define REAL float
#define SUFFIX(name) name##_f32
#define REAL_SQRT sqrtf
#include "sph_oracle_body.inc"
#undef REAL
#undef SUFFIX
#undef REAL_SQRT
