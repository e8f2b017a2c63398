"""Recommendation metrics: windowed + lifetime states, cross-rank sync, ~30 metrics, throughput."""
