"""B200-native (sm_100a) Newton-Schulz orthogonalisation and Muon optimizer step.

Drop-in names of the reference package (src/i8muon/__init__.py:1-5):
``Muon``, ``muon_step``, ``CutlassNSInt8``, ``recommend_coefficients``; plus ``FusedAdamW``, a
companion for Muon's ``scalar_optimizer`` slot.
"""
from .adamw import FusedAdamW
from .coefficients import recommend_coefficients
from .engine import CutlassNSInt8, check_status
from .optimizer import Muon, muon_step

__all__ = ["Muon", "muon_step", "CutlassNSInt8", "recommend_coefficients", "check_status", "FusedAdamW"]
