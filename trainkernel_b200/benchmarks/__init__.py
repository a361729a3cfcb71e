"""Benchmark harnesses that run through the public API."""
