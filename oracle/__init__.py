"""CPU oracle for the activation-sparse gated-FFN path.  TEST INFRASTRUCTURE ONLY.

Everything in this package is a CPU restatement (numpy / torch-CPU) of the
reference algorithm.  It exists to check the CUDA path and to provide the timed
CPU baseline; the product package never imports it.

Parity status: the reference ships no golden vectors or known-answer tests for
this path, so the oracle is pinned against outputs of the reference's own torch
implementation (``custom_models/sparse_models.py`` ``SparseMLP`` and
``custom_models/twell_modules/twell.py`` ``packed_to_dense``) generated once by
``tests/golden/make_golden.py`` and committed under ``tests/golden/``.
"""
