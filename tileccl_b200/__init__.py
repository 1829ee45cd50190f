"""tileccl_b200: Blackwell-native (sm_100a) communication/computation overlap.

Fused GEMM -> reduce-scatter and all-gather -> GEMM as single tcgen05/TMEM
kernels that move data over NVLink peer memory, a symmetric heap, the NCCL +
cuBLAS baseline, and the transport / signalling / interference probe suite.
"""
__version__ = "0.1.0"
