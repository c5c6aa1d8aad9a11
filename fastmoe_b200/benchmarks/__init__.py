"""Benchmark drivers with the entry points of polkadot21/fastmoe (src/fastmoe/benchmarks)."""
