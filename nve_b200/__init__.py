"""nve_b200: B200 (sm_100a) kernels and call sites for NVE's quantized decode path.

The product is ``nve_b200/lib/libnve_kernels.so`` (C ABI, include/nve_kernels.h).  The Python modules
mirror the reference's Rust call sites over that ABI:
  cuda_kernels  -- src/cuda_kernels.rs wrappers
  gpu_layer     -- src/gpu_layer.rs decode layer and W4A8/W4A16 routing
  decode_graph  -- src/decode_graph.rs static graph capture / replay
"""
__all__ = ["cuda_kernels", "gpu_layer", "decode_graph", "build"]
__version__ = "0.1.0"
