"""Names of the reference's native backend seam (gl_sdm/memory/backends), on the CUDA kernels."""
