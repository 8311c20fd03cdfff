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

A second form of routing (``score`` "softmax", ``weight_on`` "output"): the scores are the softmax of the router's logits over
the experts and the identity experts; a stored correction is added for the choice only; the weights are the chosen scores
times a constant and multiply the experts' outputs; an identity expert has no weights and gives its input back; the shared
expert's output is multiplied by the sigmoid of one more product a token, whose row rides along as the last row of the
router's matrix. The experts' gate function and its limit are the spec's (``GatedMlpSpec``).
"""
from __future__ import annotations

import torch

from ..config.spec import GatedMlpSpec, RoutedMlpSpec
from .base import FeedForward, ParamDecl, Runtime, register_feed_forward
from .linear import Linear
from .mlp import GATE_FUNCTIONS, GatedMlp


class RoutedMlp(FeedForward):
    def __init__(self, spec: RoutedMlpSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.experts, s.top, s.expert_intermediate) <= 0 or s.shared_intermediate < 0:
            raise ValueError("routed_mlp: hidden, experts, top and the experts' size must be positive")
        if s.top > s.experts + max(s.identity_experts, 0):
            raise ValueError(f"routed_mlp: top {s.top} is more than the {s.experts} experts and {s.identity_experts} identity experts")
        if s.experts > 1024 or s.top > 32:
            raise ValueError("routed_mlp: more than 1024 experts or a top beyond 32 is more than the routing kernel serves")
        if s.activation not in GATE_FUNCTIONS:
            raise ValueError(f"routed_mlp: activation '{s.activation}' has no kernel (built: {', '.join(GATE_FUNCTIONS)})")
        if (s.score, s.weight_on) not in (("sigmoid", "input"), ("softmax", "output")):
            raise ValueError(f"routed_mlp: score '{s.score}' with the weight on the {s.weight_on} has no kernel "
                             "(built: sigmoid scores on the input, softmax scores on the output)")
        if s.renormalize:
            raise ValueError("routed_mlp: renormalised weights have no kernel")
        self.legacy = s.score == "sigmoid"
        if self.legacy and (s.correction or s.identity_experts or s.shared_gate or s.route_scale != 1.0):
            raise ValueError("routed_mlp: a correction, identity experts, a scale or a gated shared expert need softmax scores on the output")
        if s.identity_experts < 0 or s.top > s.experts + s.identity_experts:
            raise ValueError("routed_mlp: top is more than the experts and identity experts together")
        if s.shared_gate and not s.shared_intermediate:
            raise ValueError("routed_mlp: a shared gate needs a shared expert")
        self.routed = s.experts + s.identity_experts            # router outputs that take part in the choice
        self.columns = self.routed + (1 if s.shared_gate else 0)  # rows of the router's matrix: the shared gate's row is the last
        self.correction: torch.Tensor | None = None
        self.spec = s
        self.rt = runtime
        self.router: torch.Tensor | None = None
        # steps of many tokens in bfloat16 take the router's logits from the library product with a float32 output (the same
        # 32-bit sums of bfloat16 products, on the tensor cores); fewer tokens and float32 run a warp a (token, expert)
        self.router_product = Linear(runtime, self.columns, s.hidden)
        self.router_product_min_rows = 256
        self.gate = self.up = self.down = None       # [experts, ff, hidden], [experts, ff, hidden], [experts, hidden, ff]
        # bfloat16 with an expert size that is a multiple of 128: gate and up are kept as one tensor with an expert's rows
        # interleaved in blocks of 128, the layout in which the tcgen05 product of steps of many rows applies SiLU(gate) * up
        # to its accumulator; the products of fewer rows read the same tensor
        self.gate_up: torch.Tensor | None = None
        self.interleave = 128 if (not runtime.full_precision and s.expert_intermediate % 128 == 0 and s.hidden % 8 == 0
                                  and hasattr(runtime.kernels, "_moe_gemm_tcgen05")) else 0
        self.shared = (GatedMlp(GatedMlpSpec(hidden=s.hidden, intermediate=s.shared_intermediate, activation=s.activation,
                                             limit=s.shared_limit), runtime) if s.shared_intermediate else None)

    @classmethod
    def parameters(cls, spec: RoutedMlpSpec):
        s = spec
        E, F, H = s.experts, s.expert_intermediate, s.hidden
        p = {"router": ParamDecl(shape=(E + s.identity_experts, H)), "gate": ParamDecl(shape=(E * F, H), row_splits=(F,) * E),
             "up": ParamDecl(shape=(E * F, H), row_splits=(F,) * E), "down": ParamDecl(shape=(E * H, F), row_splits=(H,) * E)}
        if s.shared_intermediate:
            S = s.shared_intermediate
            p.update({"shared_gate_up": ParamDecl(shape=(2 * S, H), row_splits=(S, S)), "shared_down": ParamDecl(shape=(H, S))})
        if s.shared_gate:
            p["shared_gate"] = ParamDecl(shape=(1, H))
        if s.correction:
            p["correction"] = ParamDecl(shape=(E + s.identity_experts,), role="vector", init=("normal", 0.0, 0.02))
        return p

    def load(self, params):
        s, dt = self.spec, self.rt.dtype
        E, F, H = s.experts, s.expert_intermediate, s.hidden
        self.router = params["router"].to(dt)
        if s.shared_gate:
            self.router = torch.cat([self.router, params["shared_gate"].to(dt)], dim=0)
        self.router = self.router.contiguous()
        if s.correction:
            self.correction = params["correction"].float().contiguous()
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
        if self.legacy:
            route = k.moe_route(logits, s.top)
            xs = k.moe_gather_scale(x, route)                                   # [T * top, hidden]: score * row, sorted by expert
            act = (k.moe_expert_gate_up(xs, self.gate, self.up, route, self.gate_up) if self.gate_up is not None
                   else k.moe_expert_gate_up(xs, self.gate, self.up, route))   # [T * top, ff]
            ys = k.moe_expert_down(act, self.down, route)                       # [T * top, hidden]
            shared = self.shared(x, batch) if self.shared is not None else None
            return k.moe_combine(ys, route, shared)
        route = k.moe_route(logits, s.top, score="softmax", correction=self.correction, scale=float(s.route_scale), routed=self.routed,
                            real=s.experts)
        xs = k.moe_gather_scale(x, route, scale=False)                          # [T * top, hidden]: the rows, sorted by expert
        fn = dict(activation=s.activation, limit=float(s.limit))
        act = (k.moe_expert_gate_up(xs, self.gate, self.up, route, self.gate_up, **fn) if self.gate_up is not None
               else k.moe_expert_gate_up(xs, self.gate, self.up, route, **fn))
        ys = k.moe_expert_down(act, self.down, route)
        shared = self.shared(x, batch) if self.shared is not None else None
        return k.moe_combine_weighted(ys, route, x, shared, logits if s.shared_gate else None)


register_feed_forward("routed_mlp", RoutedMlp)
