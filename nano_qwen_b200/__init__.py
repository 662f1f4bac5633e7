"""B200-native FP8 (e4m3) W8A8 block-scaled linear layers for nano_qwen.

``nano_qwen_b200.layers.linear`` mirrors ``nano_qwen.layers.linear`` (same class
names, constructors, attributes and ``weight_loader`` protocol); the arithmetic
runs in hand-written sm_100a CUDA kernels behind the C ABI of ``libnq_fp8.so``.
"""
__version__ = "0.1.0"
