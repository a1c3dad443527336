"""ORACLE: CPU restatement of the reference's algorithm for the tensor-product path.

This package is test infrastructure.  It is imported only by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` (as the checker or the timed CPU baseline), never by ``equitorch_b200``.
The reference is pure Python, so there is nothing to compile: the restatement is plain
PyTorch on CPU, pinned against outputs of the reference itself (``tests/golden``).
"""
