"""CPU oracle for the memorax sequence-mixing path (TEST INFRASTRUCTURE ONLY).

Nothing in the product package imports this directory.  It is used by the
tests, by the smoke check and by the ``cpu_baseline`` / ``--impl reference``
legs of the benchmark, always as the checker or as the timed CPU arm, never
as a fallback for the CUDA kernels.

Parity status: the reference ships no tests or golden vectors and needs JAX,
which cannot be installed in the build image.  The restatement is pinned by
running the reference's own source files (``memoroid.py``, ``lru.py``,
``min_gru.py``, ``linear_attention.py``) under a NumPy stand-in for the few
JAX/Flax symbols they touch (``tests/golden/make_golden.py``); the stand-in's
``associative_scan`` is our own code, so the pin covers the reference's
operators, reset rule, carry handling and read-outs, not XLA's rounding
order.  The gated delta rule has no counterpart in the reference: parity
unpinned for that op (checked against its published recurrence only).
"""
