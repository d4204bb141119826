"""CUDA sparse kernels (API of ``leankv.teal.kernels``)."""
