"""B200-native NVFP4 quantize + block-scaled FP4 GEMM path.

Submodules mirror the reference's extension modules by name:
``nvfp4`` (fx/src/s4/nvfp4/bindings.cpp), ``nvfp4_linear_cpp``
(fx/src/s4/nvfp4/linear/nvfp4_gemm_kernel.cu) and ``nvfp4_linear_module``
(fx/src/s4/nvfp4/linear/nvfp4_linear_module.py).  Importing them requires the
in-tree CUDA library (see ``build.py``); there is no fallback.
"""
__all__ = ["build", "nvfp4", "nvfp4_linear_cpp", "nvfp4_linear_module"]
