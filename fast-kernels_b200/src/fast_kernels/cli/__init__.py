"""The ``fk`` command line (``python -m fast_kernels``)."""
