"""CPU oracle for the message-passing hot path.  TEST INFRASTRUCTURE ONLY.

Plain numpy / torch-CPU restatements of the reference's algorithms, used by
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl
reference`` legs of ``bench.py`` as the checker and the timed CPU baseline.
Nothing under ``fasteq_b200/`` imports this package; the product path has no
CPU fallback.

Pinning: every function here is checked against fixtures produced by running
the e3nn 0.5.6 sources that ship inside the reference's model bundles
(``tests/golden/make_golden.py`` is the generating script, run where the
reference tree is mounted) and against the formula-plus-seed cases of the
reference's own tests (tests/adapters/test_uniform1d_hip_forward.py:48-68,
test/test_eqlinear.py:38-69).  The symmetric-contraction *operator* is pinned by
its path formula; the reference has no test that pins symmetric-contraction
values, so that basis is "parity unpinned" at the reference boundary.
"""
