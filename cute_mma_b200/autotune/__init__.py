"""Autotune: configuration generators, the per-configuration build-and-run sweep, and result analysis."""
