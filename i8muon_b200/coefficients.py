"""Newton-Schulz coefficient schedules.

Same tables and selection rules as the reference's ``recommend_coefficients``
(src/i8muon/_coeff.py:6-54; ``coefficients/int8_safe.json`` holds the same five
INT8-safety rows).  Each row (a, b, c) defines X <- (a I + b G + c G^2) X with
G = X X^T.
"""
from __future__ import annotations

import operator

INT8_SAFE = (
    (5.8918421975177555, -16.720493089530553, 11.910583457755012),
    (2.494310935454493, -3.412126511826868, 1.2164669452497787),
    (3.5701187094532, -4.7395286854633145, 1.6544471296026368),
    (2.560082131384165, -3.449401536069734, 1.2608927815298547),
    (3.8985650931142084, -7.180169545826712, 4.424064562981702),
)

_POLAR_EXPRESS_BASE = (
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
    (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
    (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
    (1.875, -1.25, 0.375),
)
_SAFETY = 1.01


def _polar_express_rows():
    """First seven stages carry the 1.01 input safety factor once; the eighth
    (also used for any extra iteration) is left as published."""
    scaled = [(a / _SAFETY, b / _SAFETY ** 3, c / _SAFETY ** 5) for a, b, c in _POLAR_EXPRESS_BASE[:-1]]
    return tuple(scaled) + (_POLAR_EXPRESS_BASE[-1],)


POLAR_EXPRESS = _polar_express_rows()
DEFAULT_COEFFICIENTS = list(INT8_SAFE)


def recommend_coefficients(iters=5, *, method="int8_safe"):
    """Return ``iters`` rows of (a, b, c).

    ``int8_safe`` needs at least five iterations; extra ones repeat the third
    stage (f1, f2, f3, ..., f3, f4, f5).  ``polar_express`` takes a prefix of its
    eight stages and repeats the last, un-scaled stage beyond eight.
    """
    if isinstance(iters, bool):
        raise TypeError("iters must be an integer")
    iters = operator.index(iters)
    if method == "polar_express":
        if iters < 1:
            raise ValueError("Polar Express requires at least one iteration")
        rows = list(POLAR_EXPRESS[:iters])
        rows += [POLAR_EXPRESS[-1]] * (iters - len(rows))
        return rows
    if method != "int8_safe":
        raise ValueError("method must be 'int8_safe' or 'polar_express'")
    if iters < 5:
        raise ValueError("At least five iterations are required for this schedule")
    head, middle, tail = INT8_SAFE[:2], INT8_SAFE[2], INT8_SAFE[3:]
    return list(head) + [middle] * (iters - 4) + list(tail)
