"""CPU oracle for the kernel templates -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this package.  It has two halves:

* :mod:`oracle.scalar` -- ctypes front end of ``cdr_oracle.c``, the plain-C restatement of
  the reference's scalar kernel definitions (numpy arrays in, numpy arrays out);
* :mod:`oracle.reference_path` -- the arithmetic the reference actually executes for a
  compiled graph: PyTorch eager on CPU tensors (``conductor/compiler/gcu_backend.py:89``).
"""
