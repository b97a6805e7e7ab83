"""Operand checks (reference gl_sdm/memory/backends/primitives.py:7-11)."""
import torch


def require_cuda(values):
    if not values.is_cuda or not values.is_contiguous():
        raise ValueError("GL-SDM native kernels require contiguous CUDA tensors")
    if torch.cuda.get_device_capability(values.device) < (10, 0):
        raise ValueError("GL-SDM B200 kernels require SM100")
