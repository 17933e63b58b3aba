"""CPU restatement of the reference's algorithms for the hot path: the checker, never the product.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` import this package.
"""
