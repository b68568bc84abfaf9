"""Utilities: synthetic workloads, clock sampling, timing helpers."""
