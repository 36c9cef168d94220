"""CPU oracle (test infrastructure only).

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package; the product path never does.
"""
