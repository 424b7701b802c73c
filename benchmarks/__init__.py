"""flodl_b200-vs-PyTorch training benchmark: the same models, data and optimizer settings in this
framework and in plain PyTorch modules, timed by one harness
(counterpart of benchmarks/src/harness.rs and benchmarks/python/harness.py of the reference)."""
