"""Timing, metrics, profiling and checkpoint helpers."""
