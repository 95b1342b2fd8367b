"""summa_b200: a Blackwell-native (sm_100a) model stack — MAL architectures,
training workflows, inference and generation, MoE dispatch and low-bit weights —
with PyTorch as the framework layer and hand-written CUDA kernels for the hot ops.
"""
__version__ = "0.1.0"
