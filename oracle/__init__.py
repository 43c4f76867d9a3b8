"""CPU oracle for the fused-attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the ``tilefusion_b200`` package imports this directory; it is used
by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline and
reference arms of ``bench.py`` as the checker / timed baseline, never as the
product.
"""
