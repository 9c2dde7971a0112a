"""B200-native (sm_100a) Muon hot path: drop-in for the operator interface of nil0x9/flash-muon.

Exports the reference's four names (flash_muon/__init__.py:1-4).  Everything runs through the
C-ABI library ``libflash_muon_b200.so``; importing the package fails if it has not been built.
"""
from .ops import (fast_newtonschulz, matmul_transpose, matmul_transpose_assign,
                  newtonschulz_workspace_bytes)
from .muon import Muon

__all__ = ["matmul_transpose", "matmul_transpose_assign", "fast_newtonschulz", "Muon",
           "newtonschulz_workspace_bytes"]
