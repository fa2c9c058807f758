"""CPU oracle for the Helix hot path (test infrastructure, not shipped code).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package.  ``oracle.api`` wraps ``libhelix_oracle.so`` (the C
restatement); ``oracle.ref`` wraps the reference's own host loops when they
have been compiled into ``oracle/_ref``.
"""
