"""Checkers for the tests, the smoke check and the CPU-baseline timing: not product code."""
