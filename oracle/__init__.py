"""CPU oracle for the attention path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: the library in `aotriton_b200/` never
imports it.  Only `tests/`, `__graft_entry__.smoke()` and the CPU-baseline / reference arms
of `bench.py` may use it, and only as the checker or as the thing timed on the host.
"""
