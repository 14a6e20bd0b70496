"""CPU oracle for the int4-AWQ hot path (test infrastructure, never the product path).

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this package.  The library under ``mlir_air_b200`` never does.
"""
