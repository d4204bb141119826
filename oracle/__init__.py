"""CPU restatement of the reference's arithmetic for the two hot paths — TEST INFRASTRUCTURE.

Nothing in the ``leankv_b200`` package imports this directory. It is used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the CPU-baseline / reference legs of ``bench.py``,
only as the checker or the timed CPU baseline, never as the thing shipped.

Pinning: the reference project has no tests or golden vectors of its own. The functions
here are checked (``tests/test_oracle_golden.py``) against outputs of the reference's own
code, generated in a container where it is importable by ``tests/golden/make_golden.py``
and committed under ``tests/golden/``.

* ``teal``        — leankv/teal/sparse_fns.py and the B=1 path of leankv/teal/patching.py
* ``turboquant``  — leankv/turboquant/{codebook,rotation,quantizer,cache}.py + the attention
                    that HF runs on the cache's dense output
* ``tq_exact``    — C restatement (``tq_exact.c``) of quantize with a fixed summation order,
                    bit-comparable with the CUDA kernels; reports each coordinate's distance
                    to the nearest decision boundary so that near-ties can be counted
* ``pool_layout`` — numpy codec of the 3-bit page layout
"""
