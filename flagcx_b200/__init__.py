"""flagcx_b200 -- a Blackwell-native collective communication framework with the
capabilities of FlagCX.

Layout:
  csrc/                     C++/CUDA library (libflagcx.so): C API, bootstrap, sockets,
                            symmetric windows, sm_100a collective kernels, tuner
  flagcx_b200.capi          ctypes binding of the C API
  flagcx_b200.torch_backend torch.distributed backend "flagcx" (C++ ProcessGroup)
  flagcx_b200.parallel      FSDP / tensor-parallel / expert-parallel engines on top
  flagcx_b200.ops           fused CUDA ops (tcgen05 GEMM+collective, MoE dispatch/combine)
  flagcx_b200.models        Llama-shaped decoder, TP layer, MoE layer
"""
__version__ = "0.1.0"
