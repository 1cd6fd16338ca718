"""sam_quantization_b200 — B200-native W8A8 quantized-linear engine for SAM's ViT image encoder.

Drop-in for the quantized-linear path of hchautran/SAM_Quantization: the same Python call
surface (W8A8Linear, the six absmax quantizers, SmoothQuant folding, QuaRot online-Hadamard
wrappers) over hand-written sm_100a CUDA kernels behind a C ABI (include/samq.h).
"""
__version__ = "0.1.0"
