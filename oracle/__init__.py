"""CPU restatement of the reference's ops path for the batched decode step. TEST INFRASTRUCTURE ONLY: imported by
tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline / --impl reference legs as the checker, never by
the product package. Each function cites the reference file:line it follows.

Parity status: the reference is Python on MLX, which cannot be imported or installed where this was written, so the
restatement is pinned (a) against the reference's own NumPy fp64 model (volundr-mlx/tests/reference.py, imported at
fixture-generation time; fixtures under tests/golden/) and (b) against the hand values and literal cases held in
the reference's tests (tests/test_volundr.py:53-65, :159-168). Third-party MLX arithmetic whose rounding the
reference's tests do not pin (general-bias dequant, SDPA accumulation order) is "parity unpinned" and defined here."""
