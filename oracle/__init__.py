"""CPU oracle of the static-cache decoder hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this
directory; only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py`` may, and only as the checker or the timed CPU
arm. The product path (``aotolith_b200``) computes on the GPU through the C ABI
and has no CPU substitute.
"""
