"""B200-native fused Mamba-3 SSD scan behind the reference's `ssm` scan entry point.

The arithmetic lives in libm3scan.so (hand-written CUDA for sm_100a, C ABI declared in
include/m3scan.h); this package is the host-side mirror of the reference interface.
"""
from . import ssm
from .ssm import (Discretization, ScanInputs, ScanOutput, SsmConfig, SsmMode, SsmState,
                  StateDynamics, mamba3_scan)

__version__ = "0.1.0"
__all__ = ["ssm", "Discretization", "ScanInputs", "ScanOutput", "SsmConfig", "SsmMode",
           "SsmState", "StateDynamics", "mamba3_scan"]
