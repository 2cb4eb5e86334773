/* TEST INFRASTRUCTURE - CPU oracle for the recurrent-scan hot path.
 *
 * A plain C restatement of the reference algorithms (tsfast v0.5.0): the diagonal scans of
 * tsfast/models/_core/scan.py and scan_backends/{diagonal_c,selective_c}.py, the fused Mamba
 * section of tsfast/models/architectures/mamba/backend_c.py, and the all-pole filter of
 * tsfast/models/architectures/dynonet/allpole_triton.py.  Each function cites the lines it
 * follows in scan_oracle_impl.h.  It exists to check the CUDA kernels and to be timed as the
 * CPU baseline; nothing in the product may link, import or call it.
 *
 * Parity is pinned: tests/golden/ holds inputs and outputs produced by importing the reference
 * itself (script committed beside them), and tests/test_oracle.py checks every function below
 * against them in both precisions.
 *
 * Two instantiations are exported: *_f32 (the arithmetic the reference CPU backends use) and
 * *_f64 (ground truth for tolerance checks).  OpenMP parallelises over independent lanes.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define REAL float
#define ORA(name) oracle_##name##_f32
#define EXP expf
#define LOG1P log1pf
#include "scan_oracle_impl.h"
#undef REAL
#undef ORA
#undef EXP
#undef LOG1P

#define REAL double
#define ORA(name) oracle_##name##_f64
#define EXP exp
#define LOG1P log1p
#include "scan_oracle_impl.h"
#undef REAL
#undef ORA
#undef EXP
#undef LOG1P

#ifdef _OPENMP
#include <omp.h>
int oracle_num_threads(void) { return omp_get_max_threads(); }
void oracle_set_num_threads(int n) { omp_set_num_threads(n); }
#else
int oracle_num_threads(void) { return 1; }
void oracle_set_num_threads(int n) { (void)n; }
#endif
