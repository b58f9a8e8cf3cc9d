"""Host-side logic of the mixer-side mirrors: widths, validation and error mapping (no GPU)."""
import pytest
import torch

from mamba_trainer_b200.error import ConfigError, ShapeError, UnsupportedError
from mamba_trainer_b200.nn import CausalConv1d, MixerCore, MixerShape, causal_conv1d
from mamba_trainer_b200.ssm import Discretization


def test_widths_follow_the_reference_config():
    """src/ssm/config.rs:165-200: d_inner = heads * head_dim * rank, bc = groups * d_state * rank, the
    projection is z | x | B | C | dt | lambda | theta."""
    s = MixerShape(heads=12, head_dim=64, d_state=128, rank=2, groups=4)
    assert s.d_inner == 12 * 64 * 2 and s.bc_width == 4 * 128 * 2
    assert s.lambda_width == 12 and s.theta_width == 12 * 128 // 2
    assert s.conv_channels == s.d_inner + 2 * s.bc_width
    assert s.in_proj_width == 2 * s.d_inner + 2 * s.bc_width + 12 + 12 + 768
    plain = MixerShape(heads=4, head_dim=8, d_state=16, learned_lambda=False, rotational=False)
    assert plain.n_groups == 4 and plain.lambda_width == 0 and plain.theta_width == 0
    assert plain.in_proj_width == 2 * 32 + 2 * 64 + 4


def test_mixer_core_rejects_inconsistent_configurations():
    with pytest.raises(ConfigError):
        MixerCore(MixerShape(heads=6, head_dim=4, d_state=8, groups=4))               # heads % groups
    with pytest.raises(ConfigError):
        MixerCore(MixerShape(heads=2, head_dim=4, d_state=7, rotational=True))        # odd d_state with rotation
    with pytest.raises(ConfigError):
        MixerCore(MixerShape(heads=3, head_dim=4, d_state=8), bidirectional=True)     # mamba3.rs:107-108
    with pytest.raises(ConfigError):
        MixerCore(MixerShape(heads=2, head_dim=4, d_state=8, learned_lambda=False),
                  discretization=Discretization.LearnedTrapezoid)
    with pytest.raises(ConfigError):
        MixerCore(MixerShape(heads=2, head_dim=4, d_state=8), bidirectional=True, post_gate_norm=True)   # mamba3.rs:175-179
    assert MixerCore(MixerShape(heads=2, head_dim=4, d_state=8, rank=2), post_gate_norm=True).post_norm_w.shape == (16,)
    core = MixerCore(MixerShape(heads=2, head_dim=4, d_state=8))
    assert core.post_norm_w is None
    assert core.conv_w.shape == (4, 2 * 4 + 2 * 2 * 8) and core.norm_w.shape == (8,)
    with pytest.raises(ShapeError):
        core(torch.zeros(1, 3, core.shape.in_proj_width + 1))
    with pytest.raises(UnsupportedError):
        core(torch.zeros(1, 3, core.shape.in_proj_width, dtype=torch.float16))


def test_conv_validates_before_touching_the_device():
    w = torch.zeros(4, 6)
    with pytest.raises(ShapeError):
        causal_conv1d(torch.zeros(2, 6), w)                       # rank (conv.rs:178-187)
    with pytest.raises(ShapeError):
        causal_conv1d(torch.zeros(1, 5, 7), w)                    # channel count
    with pytest.raises(UnsupportedError):
        causal_conv1d(torch.zeros(1, 5, 6), torch.zeros(9, 6))    # more taps than the kernels serve
    with pytest.raises(ShapeError):
        causal_conv1d(torch.zeros(1, 5, 6), w, history=torch.zeros(1, 2, 6))
    conv = CausalConv1d(6, 4)
    assert conv.empty_history(3).shape == (3, 3, 6) and conv.weight.shape == (4, 6)
