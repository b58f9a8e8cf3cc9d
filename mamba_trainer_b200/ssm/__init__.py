"""The `ssm` module of the reference (src/ssm/mod.rs:11-14), scan path only."""
from .config import Discretization, SsmConfig, SsmConfigBuilder, SsmMode, StateDynamics
from .scan import Context, ScanInputs, ScanOutput, SsmState, mamba3_scan, mamba3_step, shift_left, ssd_chunked

__all__ = ["Discretization", "SsmConfig", "SsmConfigBuilder", "SsmMode", "StateDynamics",
           "Context", "ScanInputs", "ScanOutput", "SsmState", "mamba3_scan", "mamba3_step", "shift_left", "ssd_chunked"]
