"""B200-native Mixture-of-Experts training runtime (PyTorch framework layer + sm_100a CUDA kernels)."""

__version__ = "0.1.0"
