"""Callers of the memory operator inside the reference's global layer, on fused kernels."""
from .global_layer import install_fused_proposals, propose  # noqa: F401
