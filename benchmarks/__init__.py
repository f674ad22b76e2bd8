"""Benchmark and test tooling around the library: seeded synthetic tensors, workload
builders and the timed workloads behind ``bench.py``.  Not part of the product package."""
