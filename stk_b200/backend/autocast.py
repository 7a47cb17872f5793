"""Autocast behaviour of the custom autograd functions.

Same contract as the reference (stk/backend/autocast.py:19-37): under torch.autocast the forward
casts its floating-point CUDA arguments (not float64) to the autocast dtype and runs with autocast
switched off; the backward always runs with autocast switched off.
"""
import functools

import torch


def _castable(x):
    return (isinstance(x, torch.Tensor) and x.is_cuda and x.is_floating_point()
            and x.dtype is not torch.float64)


def _cast_tree(x, dtype):
    if _castable(x):
        return x.to(dtype)
    if isinstance(x, dict):
        return {k: _cast_tree(v, dtype) for k, v in x.items()}
    if isinstance(x, (list, tuple)) and not isinstance(x, torch.Size):
        return type(x)(_cast_tree(v, dtype) for v in x)
    return x


def custom_fwd(fwd):
    @functools.wraps(fwd)
    def wrapper(*args, **kwargs):
        if not torch.is_autocast_enabled():
            return fwd(*args, **kwargs)
        dtype = torch.get_autocast_dtype("cuda")
        with torch.autocast(device_type="cuda", enabled=False):
            return fwd(*_cast_tree(args, dtype), **_cast_tree(kwargs, dtype))
    return wrapper


def custom_bwd(bwd):
    @functools.wraps(bwd)
    def wrapper(*args, **kwargs):
        with torch.autocast(device_type="cuda", enabled=False):
            return bwd(*args, **kwargs)
    return wrapper
