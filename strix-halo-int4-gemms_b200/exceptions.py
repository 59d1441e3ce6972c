"""Error types raised by the dispatch layer (same names as the reference's exceptions.py:1-6)."""


class KernelError(RuntimeError):
    """Any failure to dispatch a GEMM kernel."""


class KernelNotAvailableError(KernelError):
    """A registry entry exists but the CUDA library cannot run it on this machine."""
