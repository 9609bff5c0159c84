"""Zero-copy views of the library's device buffers for hosts that use PyTorch (plumbing for tests and the bench).

Work on a view is enqueued on torch's current stream while a step runs on the plan's stream: synchronize (or hand
torch's stream to DpOptimizer.set_stream) between writing a view and stepping.
"""
from __future__ import annotations

from . import _ffi as ffi

_ITEM = {ffi.F32: 4, ffi.BF16: 2, ffi.F16: 2}


def device_view(ptr: int, nbytes: int, dtype, device: int = 0):
    """A torch tensor of `dtype` over `nbytes` bytes of library-owned device memory at `ptr`."""
    import torch

    class _Mem:
        pass

    m = _Mem()
    m.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
    return torch.as_tensor(m, device=f"cuda:{device}").view(dtype)


def torch_dtype(code: int):
    import torch
    return {ffi.F32: torch.float32, ffi.BF16: torch.bfloat16, ffi.F16: torch.float16}[code]


def state_views(opt) -> dict:
    """grads, work (flat space) and master, exp_avg, exp_avg_sq (this rank's local space) of a DpOptimizer."""
    import torch
    p, info = opt.pointers(), opt.info
    out = {
        "grads": device_view(p["grads"], info.padded_total * _ITEM[opt.grad_dtype], torch_dtype(opt.grad_dtype), opt.device),
        "master": device_view(p["master"], info.local_elems * 4, torch.float32, opt.device),
        "exp_avg": device_view(p["exp_avg"], info.local_elems * 4, torch.float32, opt.device),
        "exp_avg_sq": device_view(p["exp_avg_sq"], info.local_elems * 4, torch.float32, opt.device),
    }
    if p["work"] == p["master"]:
        out["work"] = out["master"]
    else:
        out["work"] = device_view(p["work"], info.padded_total * _ITEM[opt.param_dtype], torch_dtype(opt.param_dtype), opt.device)
    return out
