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


class Options:
    """Backend options, passed as ``pg_options`` to ``init_process_group`` / ``new_group``
    (same fields as the FlagCX torch plugin's ``flagcxBackend::Options``,
    plugin/torch/flagcx/include/backend_flagcx.hpp:104-114 in the FlagCX project).

    enable_tuner   remember every collective's (operation, bytes); ``tune_recorded``
                   then measures exactly those sizes and stores the winners.
    tune_group_idx label of this group in the recorded tune-object file.
    """

    def __init__(self, enable_tuner: bool = False, tune_group_idx: int = 0):
        self.enable_tuner = bool(enable_tuner)
        self.tune_group_idx = int(tune_group_idx)


def _create(dist_backend_opts, pg_options):
    o = pg_options if isinstance(pg_options, Options) else Options(
        enable_tuner=os.environ.get("FLAGCX_TORCH_ENABLE_TUNER", "0") not in ("", "0"))
    return ext().create_backend(dist_backend_opts.store, dist_backend_opts.group_rank, dist_backend_opts.group_size,
                                dist_backend_opts.timeout, o.enable_tuner, o.tune_group_idx)


def register() -> None:
    if "flagcx" in getattr(dist.Backend, "backend_list", []):
        return
    dist.Backend.register_backend("flagcx", _create, extended_api=True, devices=["cpu", "cuda"])


def tune_objects(group=None, device=None):
    """[(operation code, bytes)] of the distinct collectives a group with enable_tuner has run."""
    group = group or dist.group.WORLD
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return list(ext().tune_objects(group._get_backend(device)))


def tune_recorded(group=None, device=None, iters: int = 5, path: str | None = None):
    """Collective.  Measures every recorded (operation, size) with the library's tuner
    (all applicable algorithms and CTA counts, max over ranks), keeps the winners in the
    communicator's table and writes it to `path` or $FLAGCX_TUNE_FILE on rank 0.  Also
    writes the list of tune objects next to it as ``<path>.pid<pid>`` in the layout the
    FlagCX plugin uses ({"<group idx>": {"tune_objects": [{"commOp", "nBytes"}]}}).
    Returns the number of sizes measured."""
    import json
    group = group or dist.group.WORLD
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    backend = group._get_backend(device)
    objs = sorted(ext().tune_objects(backend))
    _, idx = ext().backend_options(backend)
    comm = comm_of(group, device)
    tunable = {capi.OP_ALLREDUCE, capi.OP_ALLGATHER, capi.OP_REDUCESCATTER, capi.OP_ALLTOALL}
    done = 0
    for op, nbytes in objs:
        if op in tunable and nbytes >= 1024:
            comm.tune(op, capi.BFLOAT16, nbytes, nbytes, iters)
            done += 1
    path = path or os.environ.get("FLAGCX_TUNE_FILE")
    if path and dist.get_rank(group) == 0:
        comm.tuner_save(path)
        with open(f"{path}.pid{os.getpid()}", "w") as f:
            json.dump({str(idx): {"tune_objects": [{"commOp": int(o), "nBytes": int(b)} for o, b in objs]}}, f, indent=2)
    return done


def follow_torch_allocator(comm: capi.Comm, device: int | None = None) -> None:
    """For a communicator created through ``flagcx_b200.capi`` (not through
    ``init_process_group``) that is handed torch tensors: before PyTorch's caching
    allocator returns a segment to the driver (``torch.cuda.empty_cache()``, out-of-memory
    retries), the peers unmap it.  Process groups of this backend do this by themselves.
    Call ``unfollow_torch_allocator`` before destroying the communicator."""
    device = torch.cuda.current_device() if device is None else device
    ext().follow_allocator(int(comm.h.value), int(device))


def unfollow_torch_allocator(comm: capi.Comm) -> None:
    ext().unfollow_allocator(int(comm.h.value))


def comm_of(group=None, device=None) -> capi.Comm:
    """Non-owning capi.Comm for the communicator behind a process group."""
    group = group or dist.group.WORLD
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    backend = group._get_backend(device)
    h = ext().comm_handle(backend, device)
    return capi.Comm(capi.C.c_void_p(h), owns=False)


register()
