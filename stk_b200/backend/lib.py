"""ctypes binding of libstk_b200.so (the C ABI declared in include/stk_b200.h).

There is no fallback of any kind: if the library is missing or an entry point reports an
error, the caller gets an exception.
"""
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libstk_b200.so")

STK_F16 = 0
STK_BF16 = 1
STK_F8E4M3 = 2

_c_i64 = ctypes.c_int64
_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p
_c_size = ctypes.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/stk_b200.h
SIGNATURES = {
    "stk_b200_version": (_c_int, []),
    "stk_b200_error_string": (ctypes.c_char_p, [_c_int]),
    "stk_b200_device_status": (_c_int, [ctypes.POINTER(_c_int)]),
    "stk_b200_timeout_site": (_c_int, [ctypes.POINTER(ctypes.c_uint)]),
    "stk_b200_last_tensor_map_error": (_c_int, []),
    "stk_b200_sdd": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64,
                              _c_i64, _c_int, _c_i64, _c_int, _c_i64, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]),
    "stk_b200_dsd": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64,
                              _c_i64, _c_int, _c_int, _c_i64, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr]),
    "stk_b200_dds": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64,
                              _c_i64, _c_int, _c_i64, _c_int, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr]),
    "stk_b200_pair_stats": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr,
                                     _c_ptr]),
    "stk_b200_pair_plan_bytes": (_c_size, [_c_i64]),
    "stk_b200_pair_plan": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_ptr, _c_size, _c_ptr]),
    "stk_b200_row_indices": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr]),
    "stk_b200_transpose_meta_workspace_bytes": (_c_size, [_c_i64, _c_i64]),
    "stk_b200_transpose_meta": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr,
                                         _c_ptr, _c_size, _c_ptr]),
    "stk_b200_transpose_meta_static": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr,
                                                _c_ptr]),
    "stk_b200_block_mask": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr]),
    "stk_b200_mask_to_offsets": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "stk_b200_mask_to_indices": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "stk_b200_gather_blocks": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                        _c_i64, _c_ptr, _c_ptr]),
    "stk_b200_to_dense": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_int, _c_ptr,
                                   _c_i64, _c_ptr]),
    "stk_b200_regroup_blocks": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_ptr]),
    "stk_b200_gather_rows": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_ptr]),
    "stk_b200_scatter_rows": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr]),
    "stk_b200_weighted_sum_rows": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_i64, _c_int,
                                            _c_ptr]),
    "stk_b200_bin_index": (_c_int, [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_i64, _c_ptr,
                                    _c_ptr, _c_ptr]),
    "stk_b200_dmoe_topology": (_c_int, [_c_ptr, _c_int, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                        _c_ptr, _c_ptr, _c_ptr]),
    "stk_b200_copy_bytes": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_ptr]),
    "stk_b200_ep_barrier": (_c_int, [_c_ptr, _c_int, _c_int, _c_i64, _c_i64, _c_ptr]),
    "stk_b200_ep_share_counts": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr]),
    "stk_b200_ep_plan": (_c_int, [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                  _c_ptr]),
    "stk_b200_ep_zero_padding": (_c_int, [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_i64,
                                          _c_i64, _c_ptr]),
    "stk_b200_ep_dispatch": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int,
                                      _c_int, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_ptr]),
    "stk_b200_ep_return": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_i64, _c_i64, _c_ptr]),
}
# every routine that takes or produces int16 block indices has an _i32 twin with the same signature
for _name in ("sdd", "dsd", "dds", "pair_stats", "pair_plan", "row_indices", "transpose_meta",
              "mask_to_indices", "gather_blocks", "to_dense", "dmoe_topology"):
    SIGNATURES[f"stk_b200_{_name}_i32"] = SIGNATURES[f"stk_b200_{_name}"]

_lib = None

# STK_B200_NVTX=1: every call into the library that launches kernels is wrapped in an NVTX range named
# after its entry point (stk_b200_sdd, stk_b200_ep_dispatch, ...), so that a timeline shows which
# product or exchange step a kernel belongs to.  Off by default: a range costs two calls per launch.
NVTX = os.environ.get("STK_B200_NVTX", "0") == "1"
_UNTRACED = ("stk_b200_error_string", "stk_b200_device_status", "stk_b200_timeout_site",
             "stk_b200_last_tensor_map_error")


class _Traced:
    """The loaded library with its launching entry points wrapped in NVTX ranges."""

    def __init__(self, lib):
        self._lib, self._wrapped = lib, {}

    def __getattr__(self, name):
        fn = self._wrapped.get(name)
        if fn is None:
            raw = getattr(self._lib, name)
            if name in _UNTRACED or name.endswith("_bytes"):
                fn = raw
            else:
                def fn(*args, _raw=raw, _name=name):
                    torch.cuda.nvtx.range_push(_name)
                    try:
                        return _raw(*args)
                    finally:
                        torch.cuda.nvtx.range_pop()
            self._wrapped[name] = fn
        return fn


def load():
    """Load the shared library once and attach the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m stk_b200.csrc.build` "
            "(stk_b200 has no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means a stale library
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = _Traced(lib) if NVTX else lib
    return _lib


def error_string(code):
    return load().stk_b200_error_string(code).decode()


def check(code, what):
    """Raise for a non-zero status: ValueError for argument problems, RuntimeError otherwise."""
    if code == 0:
        return
    msg = f"{what}: {error_string(code)} (status {code})"
    if code == -5:
        msg += f", CUresult {load().stk_b200_last_tensor_map_error()}"
    if code in (-1, -2, -3, -4, -9):
        raise ValueError(msg)
    raise RuntimeError(msg)


def device_status():
    """Status word written by kernels that had to give up (0 = none).  Synchronises."""
    out = _c_int(0)
    check(load().stk_b200_device_status(ctypes.byref(out)), "stk_b200_device_status")
    return out.value


def ptr(t):
    """Device pointer of a tensor as a plain int (None -> NULL); ctypes converts it to void*."""
    return None if t is None else t.data_ptr()


def _index(device):
    if isinstance(device, int):
        return device
    if not isinstance(device, torch.device):
        device = torch.device(device)
    return device.index if device.index is not None else torch.cuda.current_device()


def stream_ptr(device):
    """Raw handle of the current stream of `device` (an int; 0 is the legacy default stream)."""
    return torch._C._cuda_getCurrentRawStream(_index(device)) or None


class on_device:
    """Makes `device` current for the duration of a launch, only if it is not current already."""

    __slots__ = ("index", "prev")

    def __init__(self, device):
        self.index = _index(device)
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def entry(name, index_tensor):
    """The entry point `name` for the width of `index_tensor`'s block indices (int16 / int32)."""
    lib = load()
    if index_tensor is not None and index_tensor.dtype == torch.int32:
        return getattr(lib, name + "_i32")
    if index_tensor is not None and index_tensor.dtype != torch.int16:
        raise ValueError(f"block indices are int16 or int32, got {index_tensor.dtype}")
    return getattr(lib, name)


def dtype_code(dtype):
    if dtype == torch.float16:
        return STK_F16
    if dtype == torch.bfloat16:
        return STK_BF16
    if dtype == torch.float8_e4m3fn:
        return STK_F8E4M3
    raise ValueError(f"stk_b200 matmuls support float16, bfloat16 and float8_e4m3fn operands, got {dtype}")
