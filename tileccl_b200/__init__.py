"""tileccl_b200: Blackwell-native (sm_100a) communication/computation overlap.

Fused GEMM -> reduce-scatter and all-gather -> GEMM as single tcgen05/TMEM kernels that move data
over NVLink peer memory, a symmetric heap, the NCCL + cuBLAS baseline, and the transport /
signalling / interference probe suite.  ``import tileccl_b200`` registers ``torch.ops.tileccl.*``.
"""
__version__ = "0.1.0"


def _register():
    from .ops import torch_ops
    return torch_ops


try:
    _t = _register()
    init, shutdown, symm_empty, heap, check_all = _t.init, _t.shutdown, _t.symm_empty, _t.heap, _t.check_all
except (ImportError, AttributeError, RuntimeError) as _e:
    # torch missing or too old for torch.library (or the op namespace taken): the C++ programs and the ctypes
    # layer still work, the torch.ops layer does not
    import warnings
    warnings.warn(f"tileccl_b200: torch.ops.tileccl is unavailable ({type(_e).__name__}: {_e})")
