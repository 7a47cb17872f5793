"""Shared parity criteria."""
import numpy as np
import torch

# 16-bit products with fp32 accumulation, against the dense fp32 path:
#   |out - ref| <= ATOL * RMS(ref) + RTOL * |ref|   for every element.
RTOL = 1e-2
ATOL = 1e-2


def assert_product_close(out, ref, what="", roundings=1):
    """`roundings`: how many independent 16-bit roundings separate `out` from `ref` (a property
    such as linearity compares one rounded result with the sum of two rounded results)."""
    out32, ref32 = out.float().cpu(), ref.float().cpu()
    assert out32.shape == ref32.shape, f"{what}: shape {tuple(out32.shape)} vs {tuple(ref32.shape)}"
    assert not torch.isnan(out32).any(), f"{what}: NaN in output"
    rms = ref32.pow(2).mean().sqrt().item() if ref32.numel() else 0.0
    excess = (out32 - ref32).abs() - roundings * (ATOL * rms + RTOL * ref32.abs())
    worst = excess.max().item() if excess.numel() else -1.0
    assert worst <= 0.0, (f"{what}: {int((excess > 0).sum())} of {excess.numel()} elements outside "
                          f"rtol {RTOL} / atol {ATOL}*RMS (RMS {rms:.3e}, worst excess {worst:.3e})")


def bits(t):
    """Raw bit pattern of a 2- or 4-byte tensor as an unsigned numpy array."""
    t = t.detach().cpu().contiguous()
    if t.element_size() == 2:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.view(torch.int32).numpy().view(np.uint32)
