/* Test infrastructure, not product code.
 *
 * CPU oracle for the five sparse operations of lab-cosmo/mops (forward and VJP, plus the
 * second-order SAP terms): a plain-C restatement of the reference's CPU algorithms, used
 * only by the tests, by the smoke check and as the CPU side of the benchmark. The
 * library under test never links, loads or calls it.
 *
 * Parity status: PINNED. tests/test_oracle.py checks every function here against
 *   (1) golden vectors produced by the reference's own NumPy implementations
 *       (python/mops/src/mops/reference_implementations.py) on the fixture shapes of the
 *       reference's test-suite, committed under tests/golden/, and
 *   (2) the unmodified reference CPU library (oracle/_ref/libmops_ref.so, built from the
 *       reference sources by this directory's Makefile) wherever that library is present.
 *
 * Build: make -C oracle oracle   ->  oracle/_ref/libmops_oracle.so */
#include <stdint.h>
#include <stddef.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define T double
#define FN(name) CAT(name, _f64)
#include "mops_oracle_impl.h"
#undef T
#undef FN

#define T float
#define FN(name) CAT(name, _f32)
#include "mops_oracle_impl.h"
#undef T
#undef FN
