"""CPU restatement of the BESS sharded KGE training step (TEST INFRASTRUCTURE ONLY).

Nothing in the product package may import this: it is the checker used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.

Pinning status: ``step_oracle`` is pinned against the reference's own torch
model (``tests/python/reference_model.py``) through the fixtures in
``tests/golden/`` and against the known-answer vectors of
``tests/pag/testPag.cpp``.  The paths the reference never tests end to end
(L2 inside the step, DistMult, ComplEx, softmax loss with correction) are a
restatement of the cited source lines only: for those, parity is unpinned.
"""
