"""Whole-engine workloads (scheduler, cache, kernels together) beyond the one-line benchmark."""
