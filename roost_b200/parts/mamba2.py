"""The Mamba-2 recurrence, as a mixer with a fixed-size state per request.

Per step: the input projection gives a token's [z | x | B | C | dt]; one kernel runs the causal convolution with SiLU
over [x | B | C], reading the taps before a row's first token from the request's state; one kernel moves the row's last
``conv_taps`` - 1 inputs into the state; one kernel walks every (row, head) through its tokens,
S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x with dt = softplus(dt + dt_bias), the state S (``state`` x
``head_dim``, 32-bit) read from and written back to the request's slot; one kernel multiplies y by SiLU(z), divides each
of ``norm_groups`` equal parts by its root mean square and applies the weight; then the output projection. Everything
that enters the recurrence besides the projection and the convolution's output is 32-bit.

A request's slot holds [S of every head | the convolution's last inputs] as one float32 vector; the executor zeroes it
when the request's first token arrives. The kernels read the step's device tables only, so steps are captured; the
padding rows of a captured step work on the scratch slot.
"""
from __future__ import annotations

import torch

from ..config.spec import Mamba2Spec
from .base import CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear


class Mamba2(Mixer):
    state_capturable = True

    def __init__(self, spec: Mamba2Spec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.head_dim, s.state, s.groups, s.conv_taps, s.norm_groups) <= 0:
            raise ValueError("mamba2: every size must be positive")
        if s.num_heads % s.groups:
            raise ValueError(f"mamba2: {s.num_heads} heads are not a multiple of {s.groups} groups")
        self.inner = s.num_heads * s.head_dim
        if self.inner % s.norm_groups:
            raise ValueError(f"mamba2: {self.inner} inner values do not divide into {s.norm_groups} norm groups")
        if s.state > 256:
            raise ValueError(f"mamba2: a state of {s.state} rows is beyond 256, the largest the scan kernel keeps in registers")
        if s.head_dim > 128:
            raise ValueError(f"mamba2: heads of {s.head_dim} values are beyond 128, the most a block of the scan kernel holds")
        if s.conv_taps > 16:
            raise ValueError(f"mamba2: {s.conv_taps} taps are beyond 16, the most the convolution kernel serves")
        self.spec = s
        self.rt = runtime
        self.channels = self.inner + 2 * s.groups * s.state          # what the convolution runs over: [x | B | C]
        self.width_in = 2 * self.inner + 2 * s.groups * s.state + s.num_heads
        self.conv_offset = s.num_heads * s.state * s.head_dim        # where the convolution's inputs start in a slot
        self.state_size = self.conv_offset + (s.conv_taps - 1) * self.channels
        self.proj_in = Linear(runtime, self.width_in, s.hidden)
        self.out = Linear(runtime, s.hidden, self.inner)
        self.conv = self.conv_bias = self.dt_bias = self.a_log = self.d = self.norm = None

    @classmethod
    def parameters(cls, spec: Mamba2Spec):
        s = spec
        inner = s.num_heads * s.head_dim
        channels = inner + 2 * s.groups * s.state
        v = lambda *shape, init=None: ParamDecl(shape=shape, role="vector", init=init)
        # the random-weights mode draws rates and steps with which a state lives for hundreds of tokens
        return {"in": ParamDecl(shape=(2 * inner + 2 * s.groups * s.state + s.num_heads, s.hidden)),
                "conv": v(channels, s.conv_taps, init=("normal", 0.0, 0.4)), "conv_bias": v(channels, init=("normal", 0.0, 0.1)),
                "dt_bias": v(s.num_heads, init=("normal", -1.0, 0.5)), "A_log": v(s.num_heads, init=("uniform", -3.0, -0.5)),
                "D": v(s.num_heads), "norm": v(inner), "out": ParamDecl(shape=(s.hidden, inner))}

    def load(self, params):
        f = lambda name: params[name].float().contiguous()
        self.proj_in.load(params["in"])
        self.out.load(params["out"])
        self.conv, self.conv_bias, self.dt_bias, self.a_log, self.d, self.norm = (f("conv"), f("conv_bias"), f("dt_bias"), f("A_log"),
                                                                                  f("D"), f("norm"))

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.state_size,), state_dtype=torch.float32)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("mamba2: a run cannot read another run's state")
        slots = batch.groups[cache.group].state_slots
        u = self.proj_in(x)                                                                  # [T, z | x | B | C | dt]
        xbc = k.mamba2_conv(u, self.inner, self.channels, self.conv, self.conv_bias, cache.state, self.conv_offset, batch.token_row,
                            batch.q_indptr, slots)
        k.mamba2_conv_state(u, self.inner, self.channels, s.conv_taps, cache.state, self.conv_offset, batch.q_indptr, slots)
        y = k.mamba2_scan(xbc, u, self.inner + self.channels, self.dt_bias, self.a_log, self.d, cache.state, batch.q_indptr, slots,
                          s.num_heads, s.head_dim, s.state, s.groups)
        g = k.gated_group_norm(y, u, self.norm, s.norm_groups, s.eps, self.rt.dtype)
        return self.out(g)


register_mixer("mamba2", Mamba2)
