"""CPU oracle of the 4-bit optimizer-step path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only ``tests/``, the smoke check in
``__graft_entry__.py`` and the CPU-baseline / reference legs of ``bench.py`` may import it, and
only as the checker or as the timed CPU baseline.
"""
