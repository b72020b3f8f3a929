"""TEST INFRASTRUCTURE: CPU oracle for the gated diagonal scan (see naju_oracle.c).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package.  The product package never does.
"""
from .oracle import (build, oracle_fwd, oracle_bwd, oracle_step, oracle_threads,  # noqa: F401
                     make_inputs, rel_l2)
