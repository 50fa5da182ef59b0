"""Kernels of the library and their Python faces."""
