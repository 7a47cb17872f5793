"""Fits the polynomial of the fused GeLU epilogue (gelu_erf in bsmm_sm100.cuh) and reports its error.

gelu(x) = max(x, 0) - |x| * Phi(-|x|) with Phi(-a) = 2^(-q(a)); q is a least-squares fit on Chebyshev
nodes of [0, 5.8], re-weighted towards the largest residual until the error is level.  The check
evaluates the fp32 Horner form on 2M points of [-8, 8] against the exact x * Phi(x) in fp64.

    python stk_b200/csrc/fit_gelu_poly.py        # needs numpy and scipy
"""
import numpy as np
from scipy.special import erfc, log_ndtr

UPPER, DEGREE = 5.8, 7


def fit(degree=DEGREE, upper=UPPER, nodes=4000, rounds=30):
    a = 0.5 * upper * (1 - np.cos(np.pi * (np.arange(nodes) + 0.5) / nodes))
    target = -log_ndtr(-a) / np.log(2.0)
    weight = np.ones(nodes)
    for _ in range(rounds):
        coeffs = np.polynomial.polynomial.polyfit(a, target, degree, w=weight)
        err = np.polynomial.polynomial.polyval(a, coeffs) - target
        weight *= 1 + 2 * np.abs(err) / np.abs(err).max()
    return coeffs.astype(np.float32), float(np.abs(err).max())


def check(coeffs):
    x = np.linspace(-8, 8, 2000001).astype(np.float32)
    a = np.minimum(np.abs(x), np.float32(8))
    q = np.full_like(a, coeffs[-1])
    for c in coeffs[-2::-1]:
        q = (q * a + c).astype(np.float32)
    h = np.exp2(-q.astype(np.float64)).astype(np.float32)
    out = (np.maximum(x, 0) - a * h).astype(np.float32)
    x64 = x.astype(np.float64)
    ref = x64 * 0.5 * erfc(-x64 / np.sqrt(2.0))
    abs_err = np.abs(out - ref)
    representable = np.abs(ref) > 6e-8          # fp16's smallest subnormal
    rel_err = (abs_err / np.maximum(np.abs(ref), 1e-300))[representable]
    differs = (out.astype(np.float16) != ref.astype(np.float16)).mean()
    return abs_err.max(), rel_err.max(), differs


if __name__ == "__main__":
    coeffs, q_err = fit()
    abs_err, rel_err, differs = check(coeffs)
    print("coefficients, constant term first:", [float(c) for c in coeffs])
    print(f"max |q error| {q_err:.2e}; gelu: max abs error {abs_err:.2e}, max relative error {rel_err:.2e}, "
          f"{100 * differs:.3f} % of fp16 results differ from the correctly rounded one")
