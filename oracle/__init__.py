"""CPU oracles for the tile-kernel path. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of bench.py may import
this package, and only as the checker. The product (tiledcuda_b200) never imports it and has no CPU
fallback.
"""
