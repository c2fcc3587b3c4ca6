"""CPU oracle for the generated-kernel path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is imported by the product (``appy_b200``).  It is used
by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` as the checker and as the timed CPU
baseline, never as a fallback for the CUDA path.

Three independent statements of what each annotated loop must compute:

* ``python_loops``  — the loops exactly as the reference runs them on the CPU: the
  example functions with the decorator removed, which is also what ``dry_run``
  executes (appy/dispatcher.py:46-53).  Pure Python; small sizes only.
* ``numpy_oracle``  — float64 NumPy/SciPy vectorised statements, usable at full size.
* ``c_loops``       — the same loops restated in C (``loops.c``, built with gcc into
  ``oracle/_build``), in the loop order and float32 arithmetic of the Python loops;
  this is the timed CPU port.

Pinning: the reference package cannot be imported unmodified in this image (its
dependencies ``ast_comments`` and ``astpass`` are not installed, see
``tests/golden/README.md``).  The oracle is pinned against (a) the known-answer
tests the reference holds for this path (tests/integration/triton/tutorial/*.py and
tests/unit/general/**, which compare with NumPy at ``np.allclose`` defaults), restated
in ``tests/test_reference_behaviour.py``, and (b) golden vectors produced by running
the reference's own Triton code generator on CPU (``TRITON_INTERPRET=1``) with
stand-ins for the two missing packages, committed under ``tests/golden/`` together
with the generating script.
"""
