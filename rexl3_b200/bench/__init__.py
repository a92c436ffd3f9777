"""Benchmarks of the named configurations beyond the headline one (the headline lives in bench.py at the repository root)."""
