"""flagcx_b200 -- a Blackwell-native collective communication framework with the
capabilities of FlagCX.

Layout:
  csrc/                     C++/CUDA library (libflagcx.so): C API, bootstrap, sockets,
                            symmetric windows, sm_100a collective kernels, MoE and
                            tcgen05 GEMM+collective kernels, tuner, trace
  flagcx_b200.capi          ctypes binding of the C API
  flagcx_b200.torch_backend torch.distributed backend "flagcx" (C++ ProcessGroup)
  flagcx_b200.parallel      FSDP, tensor-parallel, expert-parallel and pipeline engines
  flagcx_b200.ops           fused model kernels (RMSNorm, RoPE, SwiGLU, cross-entropy, AdamW)
  flagcx_b200.models        Llama-shaped decoder
  flagcx_b200.tune          offline tuner (python -m flagcx_b200.tune)
"""
__version__ = "0.1.0"
