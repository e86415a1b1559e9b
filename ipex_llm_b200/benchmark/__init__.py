"""Benchmark drivers with the reference's schemas: ``all_in_one`` (latency CSV) and ``perplexity``."""
