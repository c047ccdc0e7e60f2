"""torch.distributed backend ``"flagcx"``.

    import flagcx_b200.torch_backend          # registers the backend
    torch.distributed.init_process_group("flagcx", ...)

CUDA tensors run as NVLink kernels of libflagcx, CPU tensors over its socket path.
``comm_of(group)`` returns a ``flagcx_b200.capi.Comm`` on the same communicator for
the parts of the C API torch.distributed has no name for (window registration,
fused collectives, the tuner).
"""
from __future__ import annotations

import importlib.util
import os

import torch
import torch.distributed as dist

from flagcx_b200 import capi
from . import build as _build

_ext = None


def ext():
    """The compiled extension; raises if it has not been built (no silent fallback)."""
    global _ext
    if _ext is None:
        capi.lib()  # libflagcx.so must be resident before the extension resolves its symbols
        path = _build.built_path()
        if path is None:
            if os.environ.get("FLAGCX_TORCH_NO_JIT"):
                raise ImportError("flagcx torch extension is not built; run flagcx_b200.build.build()")
            path = _build.build()
        spec = importlib.util.spec_from_file_location(_build.NAME, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ext = mod
    return _ext


def _create(store, rank, size, timeout):
    return ext().create_backend(store, rank, size, timeout)


def register() -> None:
    if "flagcx" in getattr(dist.Backend, "backend_list", []):
        return
    dist.Backend.register_backend("flagcx", _create, devices=["cpu", "cuda"])


def comm_of(group=None, device=None) -> capi.Comm:
    """Non-owning capi.Comm for the communicator behind a process group."""
    group = group or dist.group.WORLD
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    backend = group._get_backend(device)
    h = ext().comm_handle(backend, device)
    return capi.Comm(capi.C.c_void_p(h), owns=False)


register()
