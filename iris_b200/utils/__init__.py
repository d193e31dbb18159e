"""Benchmark timer, result writers, per-tile timestamps, roofline arithmetic."""
