"""Muon optimizer family (reference: src/tplr/muon/__init__.py:19-22)."""

from .muon import Muon, SingleDeviceMuonWithAuxAdam, adam_update, apply_momentum, apply_scaling, muon_update
from .newton_schulz import newton_schulz, newton_schulz_triton, zeropower_via_newtonschulz5

__all__ = ["Muon", "SingleDeviceMuonWithAuxAdam", "newton_schulz", "newton_schulz_triton",
           "zeropower_via_newtonschulz5", "muon_update", "adam_update", "apply_momentum", "apply_scaling"]
