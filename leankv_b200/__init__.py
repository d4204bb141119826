"""leankv_b200: the leankv hot paths (TEAL sparse GEMV, TurboQuant KV cache) on B200.

Sub-modules keep the names and call signatures of the ``leankv`` package they replace:
``teal.patching``, ``teal.sparse_fns``, ``teal.kernels.sparse_gemv``,
``turboquant.quantizer``, ``turboquant.rotation``, ``turboquant.codebook``,
``turboquant.cache``, ``turboquant.paged_cache`` and ``combined``.
"""

__version__ = "0.1.0"
