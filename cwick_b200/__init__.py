"""cwick_b200 -- B200 attention engine for the CWICK hot path.

csrc/     CUDA kernels and the C ABI (include/cwk_attn.h) -> libcwk_attn.so
lib.py    ctypes binding (no fallback: raises when the library or a GPU is missing)
ops.py    tensor-level mirror of the C entry points
synth.py  seeded synthetic inputs of the benchmark configurations
"""
__all__ = ["lib", "ops", "synth", "build"]
