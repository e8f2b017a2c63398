"""Benchmark of managed-collision (zero-collision-hash) embedding lookups: throughput, collision rate and model quality."""
