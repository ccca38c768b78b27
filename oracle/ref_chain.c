/* CPU oracle, C/OpenMP form: restatement of cacti's thunk chains, one loop nest per primitive thunk.
 *
 * TEST INFRASTRUCTURE ONLY: loaded by tests/, by the smoke check and by the CPU-baseline legs of
 * bench.py; never linked into or called from libcacti_b200.so.
 *
 * PARITY UNPINNED: the reference has no tests or golden vectors and cannot be built here (Rust +
 * patched Futhark + 14 unmounted sibling crates), so this file is checked against the numpy
 * restatement (oracle/ref_chain.py) and an fp64 evaluation, not against reference outputs.
 *
 * It also stands in for the reference's CPU backend when a CPU time is reported: the reference
 * runs each primitive as a separate Futhark multicore program over materialised intermediates with
 * one thread per physical core (src/thunk/mod.rs:1843, src/pctx/smp.rs:158-181); here each
 * primitive is one OpenMP parallel loop over materialised intermediates.  Citations are into the
 * reference tree.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <omp.h>

#define PAR _Pragma("omp parallel for schedule(static)")

#define T float
#define NAME(f) f##_f32
#include "ref_chain_body.inc"
#undef T
#undef NAME

#define T _Float16
#define NAME(f) f##_f16
#include "ref_chain_body.inc"
#undef T
#undef NAME

int rc_num_threads(void) { return omp_get_max_threads(); }
void rc_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }
