"""Utilities: tensor interop, synthetic data generators, timing and GPU-guard helpers."""
