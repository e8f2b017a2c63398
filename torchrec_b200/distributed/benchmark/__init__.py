"""Benchmarks: kernel micro-benchmarks and module/pipeline benchmarks (cf. ``torchrec/distributed/benchmark/``)."""
