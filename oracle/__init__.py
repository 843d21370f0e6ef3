"""CPU oracle for the svox hot path: test infrastructure, never a product dependency.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package.
"""
