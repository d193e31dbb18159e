"""Shared helpers of the example scripts (argument parsing, timing, matrix printing)."""
