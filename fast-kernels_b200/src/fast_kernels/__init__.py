"""fast_kernels: B200-native (sm_100a) W4A16 decode GEMV behind the fast-kernels op surface."""

__all__ = ["__version__"]

__version__ = "0.1.0"
