"""The stretch of the Mamba-3 mixer between its input and output projections, as seven launches.

Mirrors Mamba3Mixer::project + mamba3_scan + finish of the reference (src/models/mamba3.rs:340-461,
:475-484, :540-556; one direction or bidirectional, with or without post_gate_norm): the projection's output
[batch, seq, width] is cut into z | x B C | dt | lambda | theta WITHOUT copies (the kernels read
column bands of it and the backward pass writes the bands of one gradient buffer), then

    convolution + SiLU over x|B|C  ->  B/C bias + RMS norm + layout  ->  softplus / sigmoid
    ->  scan  ->  y * silu(z)        (rms_norm(y) * gain * silu(z) with post_gate_norm)

Every step runs in libm3scan; the node's backward calls the matching adjoints in reverse order.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _ffi
from ..error import ConfigError, ShapeError, UnsupportedError
from ..ssm.config import Discretization
from ..ssm.scan import Context, ScanInputs, SsmState, _DTYPES, _Saved, mamba3_scan, mamba3_step


def _p(t: Optional[torch.Tensor], offset: int = 0):
    """Device address of element `offset` of t (None -> NULL)."""
    return C.c_void_p(t.data_ptr() + offset * t.element_size()) if t is not None else None


@dataclass(frozen=True)
class MixerShape:
    """The widths of SsmConfig (src/ssm/config.rs:165-200)."""
    heads: int
    head_dim: int
    d_state: int
    rank: int = 1
    groups: Optional[int] = None
    learned_lambda: bool = True
    rotational: bool = True

    @property
    def n_groups(self) -> int:
        return self.groups or self.heads

    @property
    def d_inner(self) -> int:
        return self.heads * self.head_dim * self.rank

    @property
    def bc_width(self) -> int:
        return self.n_groups * self.d_state * self.rank

    @property
    def lambda_width(self) -> int:
        return self.heads if self.learned_lambda else 0

    @property
    def theta_width(self) -> int:
        return self.heads * self.d_state // 2 if self.rotational else 0

    @property
    def conv_channels(self) -> int:
        return self.d_inner + 2 * self.bc_width

    @property
    def in_proj_width(self) -> int:
        return 2 * self.d_inner + 2 * self.bc_width + self.heads + self.lambda_width + self.theta_width


@dataclass
class MixerCache:
    """What a layer carries from one window to the next (MixerCache, src/models/mamba3.rs:62-80): the
    convolution's last K-1 inputs and the scan's state."""
    conv: torch.Tensor      # [batch, K-1, conv_channels]
    ssm: SsmState


class _MixerCore(torch.autograd.Function):
    @staticmethod
    def forward(fctx, o, proj, conv_w, conv_b, dt_bias, a_log, d_skip, b_bias, c_bias, norm_w, post_w):
        s: MixerShape = o["shape"]
        ctx = Context.for_device(proj.device)
        lib, hd = ctx.lib, ctx.handle
        B, T, W = proj.shape
        el, dt_code = proj.dtype, _DTYPES[proj.dtype]
        H, P, N, R, G = s.heads, s.head_dim, s.d_state, s.rank, s.n_groups
        di, bc = s.d_inner, s.bc_width
        off_x, off_dt = di, 2 * di + 2 * bc
        off_lam, off_th = off_dt + H, off_dt + H + s.lambda_width
        dev = proj.device
        new = lambda *shape: torch.empty(shape, device=dev, dtype=el)
        # 1. convolution + SiLU over x | B C, cut into two dense results
        x, bcr = new(B, T, H, P, R), new(B, T, 2 * bc)
        K = conv_w.shape[0]
        cdesc = _ffi.ConvDesc(batch=B, seq=T, channels=di + 2 * bc, kernel_size=K, dtype=dt_code, activation=1,
                              x_stride=W, y_stride=di, x=_p(proj, off_x), history=None, weight=_p(conv_w),
                              bias=_p(conv_b), split=di, y2_stride=2 * bc, y2=_p(bcr), dy2=None)
        if o["reverse_heads"]:
            # direction-major bands (mamba3.rs:352-370): the second half of x, of B and of C belongs to
            # the heads that walk right to left; their convolution runs right to left as well
            cdesc.n_reversed = 3
            for i, (lo, hi) in enumerate(((di // 2, di), (di + bc // 2, di + bc), (di + bc + bc // 2, di + 2 * bc))):
                cdesc.reversed_lo[i], cdesc.reversed_hi[i] = lo, hi
        ctx.check(lib.m3_conv_forward(hd, C.byref(cdesc), _p(x), None))
        # 2. B / C: groups -> heads, bias, RMS norm, rank last
        b, c = new(B, T, H, N, R), new(B, T, H, N, R)
        bdesc = _ffi.BcDesc(batch=B, seq=T, heads=H, groups=G, d_state=N, rank=R, dtype=dt_code,
                            has_norm=1 if o["norm"] else 0, eps=float(o["eps"]), raw_stride=2 * bc,
                            b_raw=_p(bcr), c_raw=_p(bcr, bc), b_bias=_p(b_bias), c_bias=_p(c_bias),
                            norm_weight=_p(norm_w))
        ctx.check(lib.m3_bc_forward(hd, C.byref(bdesc), _p(b), _p(c)))
        # 3. dt, lambda
        dt = new(B, T, H)
        lam = new(B, T, H) if s.learned_lambda else None
        adesc = _ffi.ActDesc(batch=B, seq=T, heads=H, dtype=dt_code, stride=W, dt_raw=_p(proj, off_dt),
                             lambda_raw=_p(proj, off_lam) if s.learned_lambda else None, dt_bias=_p(dt_bias))
        ctx.check(lib.m3_dt_lambda_forward(hd, C.byref(adesc), _p(dt), _p(lam)))
        # 4. scan (theta is read in place: a band of the projection is not dense, so it is copied once)
        theta = proj[..., off_th:off_th + s.theta_width].reshape(B, T, H, N // 2).contiguous() if s.rotational else None
        y = new(B, T, H, P, R)
        sdesc = _ffi.ScanDesc(batch=B, seq=T, heads=H, head_dim=P, d_state=N, rank=R, chunk=int(o["chunk"]),
                              dtype=dt_code, discretization=int(o["disc"]), dynamics=1 if s.rotational else 0,
                              want_state=0, path=int(o["path"]), reverse_heads=int(o["reverse_heads"]),
                              x=_p(x), b=_p(b), c=_p(c), dt=_p(dt), lambda_=_p(lam), theta=_p(theta),
                              a_log=_p(a_log), d_skip=_p(d_skip))
        sout = _ffi.ScanOut(y=_p(y))
        track = any(fctx.needs_input_grad)
        saved = C.c_void_p()
        ctx.check(lib.m3_scan_forward(hd, C.byref(sdesc), C.byref(sout), C.byref(saved) if track else None))
        # 5. gate
        out = new(B, T, di)
        if o["post_norm"]:
            gdesc = _ffi.GateNormDesc(batch=B, seq=T, channels=di, dtype=dt_code, z_stride=W, y=_p(y), z=_p(proj),
                                      weight=_p(post_w), eps=float(o["eps"]))
            ctx.check(lib.m3_gate_norm_forward(hd, C.byref(gdesc), _p(out)))
        else:
            gdesc = _ffi.GateDesc(batch=B, seq=T, channels=di, dtype=dt_code, z_stride=W, y=_p(y), z=_p(proj))
            ctx.check(lib.m3_gate_forward(hd, C.byref(gdesc), _p(out)))
        if track:
            fctx.o, fctx.m3 = o, ctx
            fctx.saved = _Saved(ctx, saved)
            fctx.descs = (cdesc, bdesc, adesc, sdesc, gdesc)
            fctx.keep = (proj, conv_w, conv_b, dt_bias, a_log, d_skip, b_bias, c_bias, norm_w, x, bcr, b, c, dt, lam, theta, y, post_w)
        return out

    @staticmethod
    def backward(fctx, dout):
        o, ctx = fctx.o, fctx.m3
        s: MixerShape = o["shape"]
        lib, hd = ctx.lib, ctx.handle
        ctx.bind_current_stream()
        cdesc, bdesc, adesc, sdesc, gdesc = fctx.descs
        proj, conv_w, conv_b, dt_bias, a_log, d_skip, b_bias, c_bias, norm_w, x, bcr, b, c, dt, lam, theta, y, post_w = fctx.keep
        B, T, W = proj.shape
        H, P, N, R = s.heads, s.head_dim, s.d_state, s.rank
        di, bc = s.d_inner, s.bc_width
        off_x, off_dt = di, 2 * di + 2 * bc
        off_lam, off_th = off_dt + H, off_dt + H + s.lambda_width
        dev, el = proj.device, proj.dtype
        new = lambda *shape: torch.empty(shape, device=dev, dtype=el)
        f32 = lambda *shape: torch.empty(shape, device=dev, dtype=torch.float32)
        dproj = new(B, T, W)            # every band is written exactly once below
        dout = dout.contiguous()
        # 5'. gate: dy (dense) and dz (band 0 of dproj)
        dy = new(B, T, H, P, R)
        dpost = None
        if o["post_norm"]:
            dpost = f32(di) if post_w is not None else None
            ctx.check(lib.m3_gate_norm_backward(hd, C.byref(gdesc), _p(dout), _p(dy), _p(dproj), _p(dpost)))
        else:
            ctx.check(lib.m3_gate_backward(hd, C.byref(gdesc), _p(dout), _p(dy), _p(dproj)))
        # 4'. scan
        dx, db, dc, ddt = new(B, T, H, P, R), new(B, T, H, N, R), new(B, T, H, N, R), new(B, T, H)
        dlam = new(B, T, H) if s.learned_lambda else None
        dtheta = new(B, T, H, N // 2) if s.rotational else None
        da_log, dd_skip = f32(H), (f32(H) if d_skip is not None else None)
        grads = _ffi.ScanGrads(dx=_p(dx), db=_p(db), dc=_p(dc), ddt=_p(ddt), dlambda=_p(dlam), dtheta=_p(dtheta),
                               da_log=_p(da_log), dd_skip=_p(dd_skip))
        mask = _ffi.GRAD_X | _ffi.GRAD_B | _ffi.GRAD_C | _ffi.GRAD_DT | _ffi.GRAD_A_LOG
        mask |= _ffi.GRAD_LAMBDA if s.learned_lambda else 0
        mask |= _ffi.GRAD_THETA if s.rotational else 0
        mask |= _ffi.GRAD_D_SKIP if d_skip is not None else 0
        bin_ = _ffi.ScanBwdIn(dy=_p(dy))
        ctx.check(lib.m3_scan_backward(hd, fctx.saved.handle, C.byref(bin_), mask, C.byref(grads)))
        if s.rotational:
            dproj[..., off_th:off_th + s.theta_width].copy_(dtheta.reshape(B, T, s.theta_width))
        # 3'. dt, lambda -> their bands of dproj
        ddt_bias = f32(H)
        ctx.check(lib.m3_dt_lambda_backward(hd, C.byref(adesc), _p(ddt), _p(dlam), _p(dproj, off_dt),
                                            _p(dproj, off_lam) if s.learned_lambda else None, _p(ddt_bias)))
        # 2'. B / C -> gradient of the convolution's second result
        dbcr = new(B, T, 2 * bc)
        db_bias = f32(H, N) if b_bias is not None else None
        dc_bias = f32(H, N) if c_bias is not None else None
        dnorm = f32(N) if (norm_w is not None and o["norm"]) else None
        ctx.check(lib.m3_bc_backward(hd, C.byref(bdesc), _p(db), _p(dc), _p(dbcr), _p(dbcr, bc), _p(db_bias),
                                     _p(dc_bias), _p(dnorm)))
        # 1'. convolution -> the x|B|C band of dproj
        K = conv_w.shape[0]
        dconv_w = f32(K, di + 2 * bc)
        dconv_b = f32(di + 2 * bc) if conv_b is not None else None
        cdesc.dy2 = _p(dbcr)
        ctx.check(lib.m3_conv_backward(hd, C.byref(cdesc), _p(dx), _p(dproj, off_x), _p(dconv_w), _p(dconv_b), None))
        return (None, dproj, dconv_w, dconv_b, ddt_bias, da_log, dd_skip, db_bias, dc_bias, dnorm, dpost)


class MixerCore(torch.nn.Module):
    """Parameters and forward of the mixer between its projections (src/models/mamba3.rs:140-270 for
    the parameters; float32 masters, activations float32 or bfloat16)."""

    def __init__(self, shape: MixerShape, conv_kernel: int = 4, chunk: int = 64, conv_bias: bool = True,
                 bc_bias: bool = True, bc_norm: bool = True, norm_gain: bool = True, d_skip: bool = True,
                 eps: float = 1e-5, discretization: Optional[Discretization] = None, bidirectional: bool = False,
                 post_gate_norm: bool = False, device=None):
        super().__init__()
        if shape.heads % shape.n_groups:
            raise ConfigError(f"heads {shape.heads} not a multiple of groups {shape.n_groups}")
        if shape.rotational and shape.d_state % 2:
            raise ConfigError("rotational dynamics require an even d_state")
        if bidirectional and (shape.heads % 2 or shape.n_groups % 2):
            raise ConfigError("a bidirectional mixer needs even heads and groups")      # mamba3.rs:107-108
        if bidirectional and post_gate_norm:                                            # mamba3.rs:175-179
            raise ConfigError("post_gate_norm would normalise across both directions at once; use bc_norm with a "
                              "bidirectional mixer")
        self.shape, self.chunk, self.eps, self.use_norm = shape, chunk, eps, bc_norm
        self.bidirectional = bidirectional
        self.disc = Discretization(discretization) if discretization is not None else (
            Discretization.LearnedTrapezoid if shape.learned_lambda else Discretization.Euler)
        if shape.learned_lambda != self.disc.needs_lambda_projection():
            raise ConfigError("learned_lambda and the discretization disagree")
        par = lambda t: torch.nn.Parameter(t.to(device) if device is not None else t)
        Cc, H, N = shape.conv_channels, shape.heads, shape.d_state
        self.conv_w = par((torch.rand(conv_kernel, Cc) * 2 - 1) / conv_kernel ** 0.5)
        self.conv_b = par(torch.zeros(Cc)) if conv_bias else None
        self.dt_bias = par(torch.log(torch.expm1(torch.exp(torch.empty(H).uniform_(-6.9, -2.3)))))  # softplus^-1
        self.a_log = par(torch.empty(H).uniform_(0.0, 2.77))
        self.d_skip = par(torch.ones(H)) if d_skip else None
        self.b_bias = par(torch.zeros(H, N)) if bc_bias else None
        self.c_bias = par(torch.zeros(H, N)) if bc_bias else None
        self.norm_w = par(torch.ones(N)) if (bc_norm and norm_gain) else None
        # RmsNormConfig::new(d_inner) (mamba3.rs:245-247): a gain of ones over the scan's flattened output
        self.post_gate_norm = post_gate_norm
        self.post_norm_w = par(torch.ones(shape.d_inner)) if post_gate_norm else None

    def empty_cache(self, batch: int, device, dtype=torch.float32) -> MixerCache:
        s = self.shape
        return MixerCache(torch.zeros((batch, self.conv_w.shape[0] - 1, s.conv_channels), device=device, dtype=dtype),
                          SsmState.zeros(batch, s.heads, s.head_dim, s.d_state, s.rotational, device))

    @torch.no_grad()
    def forward_cached(self, proj: torch.Tensor, cache: Optional[MixerCache] = None):
        """Inference with a carried state (Mamba3Mixer::apply_with_state, src/models/mamba3.rs:486-560):
        a prefill window or a single decoding step.  Returns (gated output, new MixerCache).  A window
        of one position runs the decode kernel (mamba3_step), longer ones the scan."""
        s = self.shape
        if proj.dim() != 3 or proj.shape[2] != s.in_proj_width:
            raise ShapeError(f"expected [batch, seq, {s.in_proj_width}], got {tuple(proj.shape)}")
        if self.bidirectional:
            raise UnsupportedError("a bidirectional mixer has no causal state to carry")   # mamba3.rs:494-499
        proj = proj.contiguous()
        ctx = Context.for_device(proj.device)
        lib, hd = ctx.lib, ctx.handle
        B, T, W = proj.shape
        el, code, dev = proj.dtype, _DTYPES[proj.dtype], proj.device
        H, P, N, R, G = s.heads, s.head_dim, s.d_state, s.rank, s.n_groups
        di, bc = s.d_inner, s.bc_width
        off_dt = 2 * di + 2 * bc
        off_lam, off_th = off_dt + H, off_dt + H + s.lambda_width
        if cache is None:
            cache = self.empty_cache(B, dev, el)
        f = lambda t: None if t is None else t.detach().to(torch.float32).contiguous()
        conv_w, conv_b, dt_bias = f(self.conv_w), f(self.conv_b), f(self.dt_bias)
        b_bias, c_bias, norm_w = f(self.b_bias), f(self.c_bias), f(self.norm_w)
        new = lambda *shape: torch.empty(shape, device=dev, dtype=el)
        K = conv_w.shape[0]
        hist = cache.conv.to(el).contiguous()
        x, bcr, new_hist = new(B, T, H, P, R), new(B, T, 2 * bc), new(B, K - 1, di + 2 * bc)
        cdesc = _ffi.ConvDesc(batch=B, seq=T, channels=di + 2 * bc, kernel_size=K, dtype=code, activation=1,
                              x_stride=W, y_stride=di, x=_p(proj, di), history=_p(hist), weight=_p(conv_w),
                              bias=_p(conv_b), split=di, y2_stride=2 * bc, y2=_p(bcr), dy2=None)
        ctx.check(lib.m3_conv_forward(hd, C.byref(cdesc), _p(x), _p(new_hist)))
        b, c = new(B, T, H, N, R), new(B, T, H, N, R)
        bdesc = _ffi.BcDesc(batch=B, seq=T, heads=H, groups=G, d_state=N, rank=R, dtype=code,
                            has_norm=1 if self.use_norm else 0, eps=float(self.eps), raw_stride=2 * bc,
                            b_raw=_p(bcr), c_raw=_p(bcr, bc), b_bias=_p(b_bias), c_bias=_p(c_bias), norm_weight=_p(norm_w))
        ctx.check(lib.m3_bc_forward(hd, C.byref(bdesc), _p(b), _p(c)))
        dt = new(B, T, H)
        lam = new(B, T, H) if s.learned_lambda else None
        adesc = _ffi.ActDesc(batch=B, seq=T, heads=H, dtype=code, stride=W, dt_raw=_p(proj, off_dt),
                             lambda_raw=_p(proj, off_lam) if s.learned_lambda else None, dt_bias=_p(dt_bias))
        ctx.check(lib.m3_dt_lambda_forward(hd, C.byref(adesc), _p(dt), _p(lam)))
        theta = proj[..., off_th:off_th + s.theta_width].reshape(B, T, H, N // 2).contiguous() if s.rotational else None
        if T == 1:
            y, ssm = mamba3_step(x[:, 0], b[:, 0], c[:, 0], dt[:, 0], lam[:, 0] if lam is not None else None,
                                 self.a_log, theta[:, 0] if theta is not None else None, self.d_skip, cache.ssm,
                                 self.disc)
            y = y.unsqueeze(1)
        else:
            inp = ScanInputs.new(x, b, c, dt, self.a_log.detach(), lam).with_chunk_size(self.chunk)
            inp = inp.with_discretization(self.disc).with_state(cache.ssm).with_state_output(True)
            if theta is not None:
                inp = inp.with_theta(theta)
            if self.d_skip is not None:
                inp = inp.with_skip(self.d_skip.detach())
            res = mamba3_scan(inp)
            y, ssm = res.y, res.state
        y = y.contiguous()
        out = new(B, T, di)
        if self.post_gate_norm:
            post_w = f(self.post_norm_w)
            gdesc = _ffi.GateNormDesc(batch=B, seq=T, channels=di, dtype=code, z_stride=W, y=_p(y), z=_p(proj),
                                      weight=_p(post_w), eps=float(self.eps))
            ctx.check(lib.m3_gate_norm_forward(hd, C.byref(gdesc), _p(out)))
        else:
            gdesc = _ffi.GateDesc(batch=B, seq=T, channels=di, dtype=code, z_stride=W, y=_p(y), z=_p(proj))
            ctx.check(lib.m3_gate_forward(hd, C.byref(gdesc), _p(out)))
        return out, MixerCache(new_hist, ssm)

    def forward(self, proj: torch.Tensor, path: int = _ffi.PATH_AUTO) -> torch.Tensor:
        """proj: the input projection's output [batch, seq, in_proj_width]; returns the gated scan
        output [batch, seq, d_inner], the input of the output projection."""
        s = self.shape
        if proj.dim() != 3 or proj.shape[2] != s.in_proj_width:
            raise ShapeError(f"expected [batch, seq, {s.in_proj_width}], got {tuple(proj.shape)}")
        if proj.dtype not in _DTYPES:
            raise UnsupportedError(f"element type {proj.dtype}: float32 and bfloat16 are served")
        # Bidirectional (mamba3.rs:97-112): every piece of the projection is direction-major; the second
        # half of the heads walks right to left inside the convolution and the scan, and nothing is
        # reversed in memory.
        if proj.shape[1] == 0:                      # nothing to scan (scan.rs:134-144)
            return proj.new_zeros((proj.shape[0], 0, s.d_inner)) + 0.0 * proj.sum()
        o = {"shape": s, "chunk": self.chunk, "eps": self.eps, "norm": self.use_norm, "disc": int(self.disc),
             "path": path, "reverse_heads": s.heads // 2 if self.bidirectional else 0,
             "post_norm": self.post_gate_norm}
        f = lambda t: None if t is None else t.to(torch.float32).contiguous()
        return _MixerCore.apply(o, proj.contiguous(), f(self.conv_w), f(self.conv_b), f(self.dt_bias), f(self.a_log),
                                f(self.d_skip), f(self.b_bias), f(self.c_bias), f(self.norm_w), f(self.post_norm_w))
