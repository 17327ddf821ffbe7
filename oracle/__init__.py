"""CPU oracles for the quantized hot path.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU
arms, never by the shipped package ``nncase_b200``.

* ``oracle.qoracle``     ctypes bindings of the C restatement (``qoracle.c`` -> ``libqoracle.so``)
* ``oracle.ref``         ctypes bindings of the reference's own kernels (``_ref/libnncase_ref.so``)
* ``oracle.quant_params`` numpy restatement of the reference's QuantParam / range math
* ``oracle.attention``   numpy restatement of paged-attention decode (no reference counterpart)
"""
