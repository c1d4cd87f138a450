"""CPU oracle for the KAD-Conv inference hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this directory; it is used by
the tests, by the smoke check and by the CPU-baseline leg of the benchmark as the checker the
CUDA kernels are compared with. It restates, in plain torch CPU ops and a small C file, the
arithmetic of the reference modules (file:line citations are relative to the reference project).

Parity status: pinned. The reference ships no golden vectors or unit tests, so the pin is made
from outputs of the reference's own modules executed on CPU with seeded weights; the generating
script and the resulting fixtures live under tests/golden/.
"""
