"""NVLink symmetric-memory communication layer and the kernels fused with it."""
