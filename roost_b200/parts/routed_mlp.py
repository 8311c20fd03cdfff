"""A feed-forward routed over small gated experts, with a shared expert beside them.

Router logits are a 32-bit product; a token's scores are their sigmoid; the ``top`` largest choose its experts (ties to
the lower index) and are the experts' weights as they are. The weight multiplies the expert's input: the token's row,
times the score, rounded once to the activation dtype, is what the chosen expert is given, and the experts' outputs are
summed; the shared expert sees the token's row itself.

Per step, all on the device (nothing is read back, so steps are captured): the router product; one kernel that scores,
chooses, counts the rows of every expert and sorts the (token, choice) pairs by expert; a gather that scales; two
products over the sorted rows in which a tile of rows meets the one expert it belongs to (gate and up with
SiLU(gate) * up applied to the sums, then down), or for the few rows of a decode step two products that stream each
row's expert once; and a kernel that sums a token's expert outputs and the shared expert's in 32-bit.
"""
from __future__ import annotations

import torch

from ..config.spec import GatedMlpSpec, RoutedMlpSpec
from .base import FeedForward, ParamDecl, Runtime, register_feed_forward
from .linear import Linear
from .mlp import GatedMlp


class RoutedMlp(FeedForward):
    def __init__(self, spec: RoutedMlpSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.experts, s.top, s.expert_intermediate) <= 0 or s.shared_intermediate < 0:
            raise ValueError("routed_mlp: hidden, experts, top and the experts' size must be positive")
        if s.top > s.experts:
            raise ValueError(f"routed_mlp: top {s.top} is more than the {s.experts} experts")
        if s.experts > 1024 or s.top > 32:
            raise ValueError("routed_mlp: more than 1024 experts or a top beyond 32 is more than the routing kernel serves")
        for what, got, built in (("activation", s.activation, "silu"), ("score", s.score, "sigmoid"), ("weight_on", s.weight_on, "input")):
            if got != built:
                raise ValueError(f"routed_mlp: {what} '{got}' has no kernel (built: {built})")
        if s.renormalize:
            raise ValueError("routed_mlp: renormalised weights have no kernel")
        self.spec = s
        self.rt = runtime
        self.router: torch.Tensor | None = None
        # steps of many tokens in bfloat16 take the router's logits from the library product with a float32 output (the same
        # 32-bit sums of bfloat16 products, on the tensor cores); fewer tokens and float32 run a warp a (token, expert)
        self.router_product = Linear(runtime, s.experts, s.hidden)
        self.router_product_min_rows = 256
        self.gate = self.up = self.down = None       # [experts, ff, hidden], [experts, ff, hidden], [experts, hidden, ff]
        # bfloat16 with an expert size that is a multiple of 128: gate and up are kept as one tensor with an expert's rows
        # interleaved in blocks of 128, the layout in which the tcgen05 product of steps of many rows applies SiLU(gate) * up
        # to its accumulator; the products of fewer rows read the same tensor
        self.gate_up: torch.Tensor | None = None
        self.interleave = 128 if (not runtime.full_precision and s.expert_intermediate % 128 == 0 and s.hidden % 8 == 0
                                  and hasattr(runtime.kernels, "_moe_gemm_tcgen05")) else 0
        self.shared = (GatedMlp(GatedMlpSpec(hidden=s.hidden, intermediate=s.shared_intermediate, activation=s.activation), runtime)
                       if s.shared_intermediate else None)

    @classmethod
    def parameters(cls, spec: RoutedMlpSpec):
        s = spec
        E, F, H = s.experts, s.expert_intermediate, s.hidden
        p = {"router": ParamDecl(shape=(E, H)), "gate": ParamDecl(shape=(E * F, H), row_splits=(F,) * E),
             "up": ParamDecl(shape=(E * F, H), row_splits=(F,) * E), "down": ParamDecl(shape=(E * H, F), row_splits=(H,) * E)}
        if s.shared_intermediate:
            S = s.shared_intermediate
            p.update({"shared_gate_up": ParamDecl(shape=(2 * S, H), row_splits=(S, S)), "shared_down": ParamDecl(shape=(H, S))})
        return p

    def load(self, params):
        s, dt = self.spec, self.rt.dtype
        E, F, H = s.experts, s.expert_intermediate, s.hidden
        self.router = params["router"].to(dt).contiguous()
        self.router_product.weight = self.router
        self.gate = params["gate"].to(dt).reshape(E, F, H).contiguous()
        self.up = params["up"].to(dt).reshape(E, F, H).contiguous()
        self.down = params["down"].to(dt).reshape(E, H, F).contiguous()
        if self.interleave:
            b = self.interleave
            self.gate_up = torch.stack([self.gate.reshape(E, F // b, b, H), self.up.reshape(E, F // b, b, H)], dim=2).reshape(E, 2 * F, H).contiguous()
            self.gate = self.up = None
        if self.shared is not None:
            self.shared.load({"gate_up": params["shared_gate_up"], "down": params["shared_down"]})

    def __call__(self, x, batch=None):
        s, k = self.spec, self.rt.kernels
        if not self.rt.full_precision and x.shape[0] >= self.router_product_min_rows and x.is_contiguous():
            logits = self.router_product(x, out_dtype=torch.float32)
        else:
            logits = k.moe_router_logits(x, self.router)                        # 32-bit sums, whatever the activation dtype
        route = k.moe_route(logits, s.top)
        xs = k.moe_gather_scale(x, route)                                       # [T * top, hidden]: score * row, sorted by expert
        act = (k.moe_expert_gate_up(xs, self.gate, self.up, route, self.gate_up) if self.gate_up is not None
               else k.moe_expert_gate_up(xs, self.gate, self.up, route))       # [T * top, ff]
        ys = k.moe_expert_down(act, self.down, route)                           # [T * top, hidden]
        shared = self.shared(x, batch) if self.shared is not None else None
        return k.moe_combine(ys, route, shared)


register_feed_forward("routed_mlp", RoutedMlp)
