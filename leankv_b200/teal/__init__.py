"""TEAL activation sparsity on B200 (API of ``leankv.teal``)."""
