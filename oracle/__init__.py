"""Checkers for the NVFP4/MXFP4 hot path.  TEST INFRASTRUCTURE ONLY: imported by tests/,
by the smoke test and by the benchmark's CPU-baseline leg; never by the product package."""
