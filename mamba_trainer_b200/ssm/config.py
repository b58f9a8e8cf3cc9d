"""Configuration of the Mamba-3 state space mixer, as the scan path sees it.

Mirrors src/ssm/config.rs: the enums `Discretization` (:18-42), `StateDynamics`
(:45-56), `SsmMode` (:59-80) and `SsmConfig` with its defaults (:130-155), derived
widths (:163-205), `validate` (:208-246) and builder (:249-348).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field, replace
from typing import Optional

from ..error import ConfigError


class Discretization(enum.IntEnum):
    """How the continuous system becomes a recurrence; values are the C ABI's."""
    Euler = 0
    Trapezoid = 1
    LearnedTrapezoid = 2

    def fixed_lambda(self) -> Optional[float]:
        """The constant lambda when it is not learned (config.rs:30-36)."""
        return {Discretization.Euler: 1.0, Discretization.Trapezoid: 0.5}.get(self)

    def needs_lambda_projection(self) -> bool:
        return self is Discretization.LearnedTrapezoid


class StateDynamics(enum.IntEnum):
    """Real decay, or decay times a rotation of N/2 planes."""
    Real = 0
    Rotational = 1


@dataclass(frozen=True)
class SsmMode:
    """`SsmMode::Siso` is rank 1; `SsmMode::Mimo { rank }` otherwise."""
    mimo_rank: Optional[int] = None

    @staticmethod
    def Siso() -> "SsmMode":
        return SsmMode(None)

    @staticmethod
    def Mimo(rank: int) -> "SsmMode":
        return SsmMode(int(rank))

    def rank(self) -> int:
        return 1 if self.mimo_rank is None else self.mimo_rank


@dataclass
class SsmConfig:
    d_model: int = 768
    n_heads: int = 24
    head_dim: int = 64
    d_state: int = 64
    n_groups: int = 24
    discretization: Discretization = Discretization.LearnedTrapezoid
    dynamics: StateDynamics = StateDynamics.Rotational
    mode: SsmMode = field(default_factory=SsmMode.Siso)
    chunk_size: int = 64
    conv_kernel: Optional[int] = 4
    bc_norm: bool = True
    bc_bias: bool = True
    post_gate_norm: bool = False
    skip_connection: bool = True
    dt_min: float = 0.001
    dt_max: float = 0.1
    dt_init_floor: float = 1e-4
    a_init_min: float = 1.0
    a_init_max: float = 16.0
    bias: bool = False

    @staticmethod
    def builder() -> "SsmConfigBuilder":
        return SsmConfigBuilder()

    def d_inner(self) -> int:
        return self.n_heads * self.head_dim * self.mode.rank()

    def bc_width(self) -> int:
        return self.n_groups * self.d_state * self.mode.rank()

    def theta_width(self) -> int:
        return 0 if self.dynamics is StateDynamics.Real else self.n_heads * self.d_state // 2

    def lambda_width(self) -> int:
        return self.n_heads if self.discretization.needs_lambda_projection() else 0

    def in_proj_width(self) -> int:
        return (2 * self.d_inner() + 2 * self.bc_width() + self.n_heads
                + self.lambda_width() + self.theta_width())

    def validate(self) -> None:
        if min(self.d_model, self.n_heads, self.head_dim, self.d_state) <= 0:
            raise ConfigError("SSM dimensions must all be positive")
        if self.n_groups <= 0 or self.n_heads % self.n_groups:
            raise ConfigError(f"n_heads ({self.n_heads}) must be a multiple of n_groups ({self.n_groups})")
        if self.dynamics is StateDynamics.Rotational and self.d_state % 2:
            raise ConfigError("rotational dynamics pair up state dimensions, so d_state must be "
                              f"even, got {self.d_state}")
        if self.chunk_size <= 0:
            raise ConfigError("chunk_size must be positive")
        if self.mode.rank() <= 0:
            raise ConfigError("MIMO rank must be positive")
        if self.dt_min <= 0.0 or self.dt_max <= self.dt_min:
            raise ConfigError(f"expected 0 < dt_min < dt_max, got {self.dt_min} and {self.dt_max}")
        if self.a_init_min <= 0.0 or self.a_init_max < self.a_init_min:
            raise ConfigError("expected 0 < a_init_min <= a_init_max")
        if self.conv_kernel is not None and self.conv_kernel < 2:
            raise ConfigError("conv_kernel must be at least 2; use None to disable")


class SsmConfigBuilder:
    """Chained setters, then `build()` validates (config.rs:249-348)."""

    _FIELDS = ("d_model", "n_heads", "head_dim", "d_state", "n_groups", "discretization",
               "dynamics", "mode", "chunk_size", "conv_kernel", "bc_norm", "bc_bias",
               "post_gate_norm", "skip_connection", "bias")

    def __init__(self):
        self._config = SsmConfig()

    def __getattr__(self, name):
        if name in SsmConfigBuilder._FIELDS:
            def setter(value):
                self._config = replace(self._config, **{name: value})
                return self
            return setter
        raise AttributeError(name)

    def dt_range(self, lo: float, hi: float) -> "SsmConfigBuilder":
        self._config = replace(self._config, dt_min=lo, dt_max=hi)
        return self

    def a_init_range(self, lo: float, hi: float) -> "SsmConfigBuilder":
        self._config = replace(self._config, a_init_min=lo, a_init_max=hi)
        return self

    def expand(self, expansion: float) -> "SsmConfigBuilder":
        c = self._config
        inner = int(c.d_model * expansion)
        per_head = max(1, c.head_dim * c.mode.rank())
        heads = max(1, inner // per_head)
        self._config = replace(c, n_heads=heads, n_groups=heads)
        return self

    def build(self) -> SsmConfig:
        self._config.validate()
        return self._config
