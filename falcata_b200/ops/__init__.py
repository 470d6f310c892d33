"""Kernel-level entry points (one function per device kernel) used by the numerics tests."""
