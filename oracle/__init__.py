"""CPU oracles for the SparseConv2D hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only ``tests/``, the smoke check and the
benchmark's CPU-baseline / reference legs import it, as the checker or the timed baseline.
"""
