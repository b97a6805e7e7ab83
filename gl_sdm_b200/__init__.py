"""B200-native transactional shared-memory operator with the GL-SDM ``gl_sdm.memory`` API.

``gl_sdm_b200.memory`` mirrors the reference package projects/gl-sdm/src/gl_sdm/memory
(state, transactions, routing); ``gl_sdm_b200.install`` registers it under the reference's
module names so the reference's layer stack imports it unchanged. All arithmetic runs in the
sm_100a kernels of ``libglsdm_b200.so`` (C ABI: include/glsdm.h).
"""
from . import _native  # noqa: F401
from . import memory  # noqa: F401

__all__ = ["memory", "_native"]
