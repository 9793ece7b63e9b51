"""Comparison helpers shared by the GPU parity tests.

``close_elementwise`` is the reference's ``Close`` (kernels/kerneltest/compare.go:31-39) applied to
every element: ``|got - want| <= floor + rel * scale``.  The reference's fixtures are O(1), so its
scale is ``max(|want|, 1)``; gradients are not O(1), so here the unit is stated by the caller as a
fraction of the tensor's largest magnitude: ``floor = floor_frac * max|want|`` and the relative term
uses the element itself, ``rel * |want_i|``.  A tensor therefore has to agree to ``rel`` where it is
large and to ``floor_frac`` of its largest entry where it is near zero.
"""
from __future__ import annotations

import numpy as np


def rel_err(got, want) -> float:
    """Largest difference relative to the largest magnitude of ``want`` (the norm-wise figure logits are held to)."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


def elementwise_excess(got, want, rel: float, floor_frac: float) -> float:
    """max over elements of |got - want| / (floor + rel * |want|): <= 1 means every element is Close."""
    got = np.asarray(got, np.float64).ravel(); want = np.asarray(want, np.float64).ravel()
    unit = max(float(np.max(np.abs(want))) if want.size else 0.0, 1e-30)
    allowed = floor_frac * unit + rel * np.abs(want)
    return float(np.max(np.abs(got - want) / allowed)) if want.size else 0.0


def close_elementwise(got, want, rel: float, floor_frac: float) -> bool:
    return elementwise_excess(got, want, rel, floor_frac) <= 1.0


def error_report(got, want) -> dict:
    """Measured agreement of one tensor: norm-wise error and the smallest floor fraction that makes every element
    Close at rel = 1e-4."""
    got = np.asarray(got, np.float64).ravel(); want = np.asarray(want, np.float64).ravel()
    unit = max(float(np.max(np.abs(want))), 1e-30)
    diff = np.abs(got - want)
    need = np.maximum(diff - 1e-4 * np.abs(want), 0.0) / unit
    return {"normwise": float(diff.max() / unit), "floor_needed": float(need.max()), "unit": unit}


# ---------------------------------------------------------------------------------------------------------------
# Gradient tolerances of the RL step (1e-4 relative), as measured against the float64-accumulating oracle.
# Matrices and tables: every element Close at rel 1e-4 with a floor of 5e-5 of the tensor's largest entry (measured:
# at most 4.1e-5 on the d12 model, 2.8e-5 on the small ones; the reference's own float32-lane products differ from
# its float64-accumulating ones by 1.5e-5 on the same inputs).
GRAD_REL = 1e-4
GRAD_FLOOR = 5e-5
# Scalar parameters are sums over every token of terms of both signs; what bounds their error is the sum of the
# terms' magnitudes, which the parameter's value does not show.  Measured on d12: smear_lambda 6.3e-4 (the
# reference's two backends differ by 7.6e-5 on it), every other scalar <= 2.1e-5.  They are held to 1e-3.
SCALARS = ("resid_lambdas", "x0_lambdas", "smear_gate.weight", "smear_lambda", "backout_lambda")
SCALAR_REL = 1e-3


def assert_gradients_close(gm, om, n_layer=None):
    """Every gradient tensor of the device model ``gm`` against the oracle model ``om``.

    backout_lambda in a model whose tap layer is its last layer (n_layer / 2 == n_layer - 1, i.e. one- and
    two-layer models): the tapped activation is the final activation itself, the gradient of the norm is
    orthogonal to it, and the true value is exactly zero; both sides return rounding noise, which is held to 1e-5
    of the largest gradient entry of the whole model."""
    names = list(gm.names)
    global_unit = max(float(np.max(np.abs(om.grad(n)))) for n in names)
    if n_layer is None:
        n_layer = max((int(n.split(".")[2]) for n in names if n.startswith("transformer.h.")), default=-1) + 1
    bad = []
    for n in names:
        g, w = gm.grad(n), om.grad(n)
        if n == "backout_lambda" and n_layer // 2 == n_layer - 1:
            if float(np.max(np.abs(g - w))) > 1e-5 * global_unit:
                bad.append((n, float(np.max(np.abs(g - w))), global_unit))
        elif n in SCALARS:
            ex = elementwise_excess(g, w, SCALAR_REL, SCALAR_REL * 1e-1)
            if ex > 1.0:
                bad.append((n, ex))
        else:
            ex = elementwise_excess(g, w, GRAD_REL, GRAD_FLOOR)
            if ex > 1.0:
                bad.append((n, ex))
    assert not bad, bad
