"""The Mamba selective scan, as a mixer with a fixed-size state per request.

Per step: the input projection gives a token's [x | z]; one kernel runs the causal convolution with SiLU over x, reading the
taps before a row's first token from the request's state, and one moves the row's last ``conv_taps`` - 1 inputs into the state
(the convolution kernels of the Mamba-2 mixer, which take any channel range); a projection of the convolved x gives
[dt | B | C]; the step projection gives W_dt dt as 32-bit sums; one kernel walks every (row, channel) through its tokens,
dt = softplus(W_dt dt + bias), S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = sum_n S[c, n] C_n + D_c x_c, multiplies
by SiLU(z) and rounds once; then the output projection. A = -exp(A_log) is formed once at load. Decays, steps, the state
and y are 32-bit.

A request's slot holds [S: inner x state | the convolution's last inputs] as one float32 vector; the executor zeroes it when
the request's first token arrives. The kernels read the step's device tables only, so steps are captured; the padding rows
of a captured step work on the scratch slot.
"""
from __future__ import annotations

import torch

from ..config.spec import Mamba1Spec
from .base import CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear


class Mamba1(Mixer):
    state_capturable = True

    def __init__(self, spec: Mamba1Spec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.inner, s.state, s.dt_rank, s.conv_taps) <= 0:
            raise ValueError("mamba1: every size must be positive")
        if s.state > 256:
            raise ValueError(f"mamba1: a state of {s.state} numbers a channel is beyond 256, the most the scan kernel keeps in registers")
        if s.conv_taps > 16:
            raise ValueError(f"mamba1: {s.conv_taps} taps are beyond 16, the most the convolution kernel serves")
        self.spec = s
        self.rt = runtime
        self.conv_offset = s.inner * s.state                       # where the convolution's inputs start in a slot
        self.state_size = self.conv_offset + (s.conv_taps - 1) * s.inner
        self.proj_in = Linear(runtime, 2 * s.inner, s.hidden)
        self.proj_x = Linear(runtime, s.dt_rank + 2 * s.state, s.inner)
        self.proj_dt = Linear(runtime, s.inner, s.dt_rank)
        self.out = Linear(runtime, s.hidden, s.inner)
        self.conv = self.conv_bias = self.dt_bias = self.a = self.d = None

    @classmethod
    def parameters(cls, spec: Mamba1Spec):
        s = spec
        v = lambda *shape, init=None: ParamDecl(shape=shape, role="vector", init=init)
        # the random-weights mode draws rates and steps with which a state lives for hundreds of tokens
        return {"in": ParamDecl(shape=(2 * s.inner, s.hidden)), "conv": v(s.inner, s.conv_taps, init=("normal", 0.0, 0.4)),
                "conv_bias": v(s.inner, init=("normal", 0.0, 0.1)), "x": ParamDecl(shape=(s.dt_rank + 2 * s.state, s.inner)),
                "dt": ParamDecl(shape=(s.inner, s.dt_rank)), "dt_bias": v(s.inner, init=("normal", -2.0, 0.5)),
                "A_log": v(s.inner, s.state, init=("uniform", -2.0, 1.0)), "D": v(s.inner), "out": ParamDecl(shape=(s.hidden, s.inner))}

    def load(self, params):
        f = lambda name: params[name].float().contiguous()
        self.proj_in.load(params["in"])
        self.proj_x.load(params["x"])
        self.proj_dt.load(params["dt"])
        self.out.load(params["out"])
        self.conv, self.conv_bias, self.dt_bias, self.d = f("conv"), f("conv_bias"), f("dt_bias"), f("D")
        self.a = (-torch.exp(f("A_log"))).contiguous()             # [inner, state]

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.state_size,), state_dtype=torch.float32)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("mamba1: a run cannot read another run's state")
        slots = batch.groups[cache.group].state_slots
        xz = self.proj_in(x)                                                                 # [T, x | z]
        xc = k.mamba2_conv(xz, 0, s.inner, self.conv, self.conv_bias, cache.state, self.conv_offset, batch.token_row, batch.q_indptr, slots)
        k.mamba2_conv_state(xz, 0, s.inner, s.conv_taps, cache.state, self.conv_offset, batch.q_indptr, slots)
        dbc = self.proj_x(xc)                                                                # [T, dt | B | C]
        dt = self.proj_dt(dbc[:, : s.dt_rank], out_dtype=torch.float32)                      # W_dt dt as 32-bit sums, [T, inner]
        g = k.mamba1_scan(xc, dt, dbc, xz, self.dt_bias, self.a, self.d, cache.state, batch.q_indptr, slots, s.inner, s.state, s.dt_rank)
        return self.out(g)


register_mixer("mamba1", Mamba1)
