"""Benchmark and profiling drivers (tooling for the measurements under ``profiles/``; not part of the
importable framework). Run from the repository root, e.g. ``python -m benchmarks.kernels``."""
