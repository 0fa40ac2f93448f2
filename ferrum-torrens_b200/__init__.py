"""B200-native NVFP4 mixture-of-experts layer behind a C-ABI shared library.

The directory name is not a Python identifier; import it with
`importlib.import_module("ferrum-torrens_b200")`.
"""
from .moe import (B200MoE, CachedExperts, ExpertCache, ExpertShapes, MoEDeviceRequest, MoEError, MoEGroup,
                  BANKS, route_lists, run_experts)
from . import _lib, ftw, synth
from .ftw import FtwBanks, FtwIndex

__all__ = ["B200MoE", "CachedExperts", "ExpertCache", "ExpertShapes", "MoEDeviceRequest", "MoEError", "MoEGroup",
           "BANKS", "route_lists", "run_experts", "synth", "_lib", "ftw", "FtwBanks", "FtwIndex"]
