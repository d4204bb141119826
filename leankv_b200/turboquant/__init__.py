"""TurboQuant KV-cache quantization on B200 (API of ``leankv.turboquant``)."""
