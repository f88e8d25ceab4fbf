"""Micro-benchmarks of single kernels (run as `python -m monoserve_b200.benchmarks.<name>`)."""
