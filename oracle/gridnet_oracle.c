/*
 * TEST INFRASTRUCTURE, not product code: the CPU oracle for the block-local grid
 * update (see gridnet_oracle_impl.inc for what it restates and from where).
 * Built by oracle/Makefile into oracle/libgridnet_oracle.so; exported symbols
 * are gno_<op>_f32 and gno_<op>_f64.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define REAL float
#define SUFFIX f32
#include "gridnet_oracle_impl.inc"
#undef REAL
#undef SUFFIX

#define REAL double
#define SUFFIX f64
#include "gridnet_oracle_impl.inc"
#undef REAL
#undef SUFFIX

#ifdef _OPENMP
#include <omp.h>
int gno_max_threads(void) { return omp_get_max_threads(); }
void gno_set_threads(int n) { omp_set_num_threads(n); }
#else
int gno_max_threads(void) { return 1; }
void gno_set_threads(int n) { (void)n; }
#endif
