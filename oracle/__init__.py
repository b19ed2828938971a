"""CPU oracle for the sparse low-bit compressed linear layer.

TEST INFRASTRUCTURE ONLY.  Nothing in the ``cobalt_b200`` package imports this
directory; it is the checker that the parity tests, ``__graft_entry__.smoke()``
and the CPU-baseline legs of ``bench.py`` compare the CUDA path against.

Every function restates one function of the reference implementation
(SDMuhsin/CoBALT) and cites the file and lines it follows.  The restatement is
pinned against the reference itself: ``tests/golden/make_golden.py`` imports the
reference's own Python modules, runs them on seeded inputs and stores the outputs
as fixtures; ``tests/test_oracle_golden.py`` requires this oracle to reproduce
those fixtures bit for bit.
"""
