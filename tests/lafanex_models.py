"""Small Lafanex models for the tests: configurations that differ in every size and option, weights drawn so that faults
show, and a recorder of the engine's routing decisions.

Weights: matrices N(0, std) scaled by their fan-in; norm weights around zero (the design adds one); the streams' read weights
around 1/S, mix matrices near the identity, write weights around one; output projections small beside the residual, so that
a layer's rounding error is not doubled by the next one; the scan's A_log and dt bias so that a state lives for
hundreds of tokens (a lost or misplaced state changes every later logit); router rows that spread the scores; a correction
large enough to change choices. ``sharpen`` makes one query token of the first layer score one key token far above all
others, so that whether that key is seen decides the output.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from roost_b200.weights.safetensors_io import write_safetensors
from tests.plain import lafanex_plain as P


def attention(heads=4, kv_heads=2, dim=8, vdim=6, rot=4, base=300.0, scale=0.5):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "rot": {"base": base, "dims": rot}}}


def mamba(inner=12, state=5, dt_rank=3, conv=3):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=3, ff=12, limit=2.0, scale=1.7, shared=20, shared_limit=1.5):
    f = {"kind": "moe", "router": {"experts": experts, "top": top, "identity": identity, "scale": scale}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        f["shared"] = {"ff": shared, "limit": shared_limit}
    return f


def config(layers, width=40, vocab=97, eps=1e-5, streams=3, loop=None):
    c = {"architecture": "Lafanex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}
    if streams is not None:
        c["streams"] = streams
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# Configurations. None uses the sizes of anyone's released model; they differ from one another in every size.
MIXED = config([(attention(), dense()), (mamba(), moe()), (attention(heads=3, kv_heads=1, dim=6, vdim=9, rot=6, scale=0.7), moe(experts=4, identity=0, top=1, ff=16, shared=0)),
                (mamba(inner=20, state=9, dt_rank=2, conv=4), None)], loop=(1, 3, 2))
# values that many models make equal or 1 differ here, and the other way round: one stream with learned weights, as many
# key/value heads as query heads, keys and values of one size (the cache of two planes), a rotation narrower than the head,
# two taps, a step projection of rank one, a top of one among identity experts, no shared expert, a scan first, no loop
ODD = config([(mamba(inner=9, state=17, dt_rank=1, conv=2), moe(experts=3, identity=3, top=1, ff=10, limit=0.8, scale=1.0, shared=0)),
              (attention(heads=3, kv_heads=3, dim=10, vdim=10, rot=4, base=50.0, scale=0.3), None),
              (attention(heads=6, kv_heads=2, dim=4, vdim=7, rot=2, base=50.0, scale=1.1), dense(ff=31)),
              (mamba(inner=16, state=16, dt_rank=5, conv=5), dense(ff=18))], width=36, vocab=61, eps=1e-6, streams=1)
# sizes of whole vectors (multiples of 8 and 64), heads the tensor-core attention kernels serve, a loop of one layer run thrice
WIDE = config([(attention(heads=4, kv_heads=2, dim=64, vdim=64, rot=32, base=10000.0, scale=0.125), moe(experts=6, identity=1, top=2, ff=128, shared=64)),
               (mamba(inner=128, state=16, dt_rank=8, conv=4), dense(ff=128)),
               (attention(heads=4, kv_heads=1, dim=32, vdim=48, rot=32, base=10000.0, scale=0.2), dense(ff=64))],
              width=128, vocab=200, streams=2, loop=(0, 1, 3))
# no streams at all: one residual and plain sums
PLAIN = config([(attention(heads=2, kv_heads=1, dim=8, vdim=4, rot=8), dense(ff=20)), (mamba(inner=10, state=4, dt_rank=2, conv=4), moe(experts=4, identity=1, top=2, ff=8, shared=12))],
               width=24, vocab=50, streams=None, loop=(0, 2, 2))
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "plain": PLAIN}


def tensor_shapes(cfg) -> dict:
    W, S = cfg["width"], cfg.get("streams")
    shapes = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm2"] = (W,)
        if S:
            for q in ("hc1.", "hc2."):
                shapes.update({p + q + "in": (S,), p + q + "out": (S,), p + q + "mix": (S, S)})
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W), p + "mix.o": (W, H * dv)})
        else:
            inner, N, R = m["inner"], m["state"], m["dt_rank"]
            shapes.update({p + "mix.in": (2 * inner, W), p + "mix.conv": (inner, m["conv"]), p + "mix.conv.b": (inner,), p + "mix.x": (R + 2 * N, inner),
                           p + "mix.dt": (inner, R), p + "mix.dt.b": (inner,), p + "mix.A_log": (inner, N), p + "mix.D": (inner,), p + "mix.o": (W, inner)})
        f = layer["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            shapes.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        else:
            routed = f["router"]["experts"] + f["router"].get("identity", 0)
            shapes.update({p + "mlp.router": (routed, W), p + "mlp.correction": (routed,)})
            names = [f"e{e}" for e in range(f["router"]["experts"])]
            sizes = [f["expert"]["ff"]] * len(names)
            if f.get("shared"):
                names.append("shared")
                sizes.append(f["shared"]["ff"])
                shapes[p + "mlp.shared.sg"] = (1, W)
            for n, ff in zip(names, sizes):
                shapes.update({f"{p}mlp.{n}.gate": (ff, W), f"{p}mlp.{n}.up": (ff, W), f"{p}mlp.{n}.down": (W, ff)})
    return shapes


def draw_tensors(cfg, seed: int, std: float = 0.25) -> dict:
    g = torch.Generator().manual_seed(seed)
    S = cfg.get("streams") or 1
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g)
        if name.endswith("hc1.in") or name.endswith("hc2.in"):
            t = (1.0 + 0.3 * r) / S
        elif name.endswith(".mix") and "hc" in name:
            t = torch.eye(S) + 0.15 * r
        elif name.endswith(".out") and "hc" in name:
            t = 1.0 + 0.2 * r
        elif "norm" in name:
            t = 0.1 * r
        elif name.endswith("A_log"):
            t = -2.0 + 2.5 * torch.rand(shape, generator=g)
        elif name.endswith("dt.b"):
            t = -2.0 + 0.5 * r
        elif name.endswith("conv.b"):
            t = 0.1 * r
        elif name.endswith(".D"):
            t = 1.0 + 0.3 * r
        elif name.endswith("mix.conv"):
            t = 0.5 * r
        elif name.endswith("router"):
            t = 0.5 * r
        elif name.endswith("correction"):
            t = 0.05 * r
        elif name == "embed":
            t = r
        elif name.endswith(".o") or name.endswith(".down"):
            t = 0.25 * std * r * (32.0 / max(shape[-1], 1)) ** 0.5      # branches smaller than the residual: rounding does not compound from layer to layer
        else:
            t = std * r * (32.0 / max(shape[-1], 1)) ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out


def sharpen(cfg, tensors: dict, key_token: int, query_token: int) -> None:
    """Changes layer 0's query weights (an attention whose rotation is narrower than its heads, run first) so that
    ``query_token``'s queries point along ``key_token``'s keys in the elements the rotation leaves alone: unit-norm queries
    and keys then meet with nearly the largest score there is, wherever the two tokens stand. The first layer's input depends
    on the token alone, so both are known from the weights."""
    layer = cfg["layers"][0]
    m = layer["mixer"]
    assert layer["type"] == "attention" and m["rot"]["dims"] < m["dim"] and P.layer_order(cfg)[0] == 0
    w = {k: v.double() for k, v in tensors.items()}
    S = cfg.get("streams")
    read = float(w["l0.hc1.in"].sum()) if S else 1.0
    x = P.offset_norm(read * w["embed"][[key_token, query_token]], w["l0.norm1"], cfg["norm"]["eps"])
    H, G, d, rot = m["heads"], m["kv_heads"], m["dim"], m["rot"]["dims"]
    keys = (x[0] @ w["l0.mix.k"].T).reshape(G, d)
    q = w["l0.mix.q"].reshape(H, d, -1).clone()
    xq = x[1]
    for h in range(H):
        k = keys[h // (H // G)].clone()
        k[:rot] = 0.0
        q[h] = q[h] * 0.05 + torch.outer(k / k.norm(), xq) * (8.0 / float(xq @ xq))
    tensors["l0.mix.q"] = q.reshape(w["l0.mix.q"].shape).to(torch.bfloat16)
    # ... and the key token's value is large, so that seeing it moves the layer's output by much
    g = torch.Generator().manual_seed(key_token)
    direction = torch.randn(w["l0.mix.v"].shape[0], generator=g, dtype=torch.float64)
    tensors["l0.mix.v"] = (w["l0.mix.v"] + torch.outer(20.0 * direction / direction.norm(), x[0]) / float(x[0] @ x[0])).to(torch.bfloat16)


def write_model(model_dir, cfg, tensors) -> Path:
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(model_dir / "model.safetensors", tensors, metadata={"format": "pt"})
    return model_dir


def plain_weights(tensors: dict) -> dict:
    """The stored bfloat16 values in float64."""
    return {k: v.double() for k, v in tensors.items()}


class RouteRecorder:
    """Wraps a kernel library's ``moe_route`` and keeps, per call, the experts every token was given (in the order of the
    token's choices). A bfloat16 engine and a float64 plain implementation may order two nearly equal scores differently;
    the tests hand the engine's choices to the plain implementation and check separately that each choice was within a
    rounding of the best."""

    def __init__(self, kernels):
        self.kernels = kernels
        self.calls = []
        self._orig = kernels.moe_route

    def __enter__(self):
        def wrapped(logits, top, **kw):
            route = self._orig(logits, top, **kw)
            experts = torch.as_tensor(route.expert).to(torch.int64).cpu()[route.inverse.cpu().long()].reshape(-1, top)
            self.calls.append(experts)
            return route
        self.kernels.moe_route = wrapped
        return self

    def __exit__(self, *exc):
        del self.kernels.moe_route


def routed_runs(cfg) -> list:
    """The layer runs (indices into the order layers run in, a looped layer once a pass) that have routed experts."""
    return [run for run, i in enumerate(P.layer_order(cfg)) if cfg["layers"][i]["mlp"] is not None and cfg["layers"][i]["mlp"]["kind"] == "moe"]
