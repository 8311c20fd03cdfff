"""Small Vamatar models for the tests: configurations that differ in every size and option, weights drawn so that
faults show, and a recorder of the engine's routing decisions.

Weights: matrices N(0, std); norm weights 1 + N(0, 0.1), biases N(0, 0.1); the recurrence's A_log in [-3, -0.5] and
dt_bias around -1 so that a state lives for hundreds of tokens (a lost or misplaced state changes every later logit);
router rows of a size that spreads the scores without saturating the sigmoid. ``sharpen`` makes one query token of the first layer score one key token
far above all others, so that whether that key is inside the window decides the output.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from roost_b200.weights.safetensors_io import write_safetensors
from tests.plain import vamatar_plain as P


def latent(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=10, window=9, base=300.0, dims=None, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": dims or rot_dim}, "scale": scale or 1.0 / math.sqrt(dim + rot_dim)}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def mamba(heads=4, vdim=6, state=5, groups=2, conv=3, norm_groups=2):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=12, shared=20):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def config(layers, width=40, vocab=97, eps=1e-5, scale=0.7, cap=9.0):
    c = {"architecture": "Vamatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


# Configurations. None uses the sizes of anyone's released model; they differ from one another in every size.
MIXED = config([(latent(), dense()), (mamba(), moe()), (latent(window=14, kv_from=0), moe(experts=4, top=1, ff=16, shared=0)),
                (mamba(heads=2, vdim=12, state=9, groups=1, conv=4, norm_groups=1), None)])
# values that many models make equal or 1 differ here: top 3, one group, one norm group, taps 2, rot.dims below rot_dim, no
# window in the reading layer's owner, no cap, no shared expert, a first layer that is a recurrence
ODD = config([(mamba(heads=3, vdim=10, state=7, groups=3, conv=2, norm_groups=3), moe(experts=7, top=3, ff=10, shared=0)),
              (latent(heads=2, dim=6, rot_dim=8, vdim=9, kv_rank=12, window=None, dims=4, base=50.0), None),
              (latent(heads=5, dim=4, rot_dim=8, vdim=3, kv_rank=12, window=6, dims=4, base=50.0, kv_from=1), dense(ff=31)),
              (mamba(heads=1, vdim=16, state=16, groups=1, conv=5, norm_groups=1), dense(ff=18))], width=36, vocab=61, eps=1e-6,
             scale=1.0, cap=None)
# sizes of whole vectors (multiples of 8 and 64): the paths that load 16 bytes at a time
WIDE = config([(latent(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=48, window=40, base=10000.0), moe(experts=6, top=2, ff=64, shared=64)),
               (mamba(heads=4, vdim=32, state=64, groups=2, conv=4, norm_groups=2), dense(ff=128)),
               (latent(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=48, window=24, base=10000.0, kv_from=0), dense(ff=64))],
              width=128, vocab=200, eps=1e-5, scale=0.5, cap=20.0)
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE}


def tensor_shapes(cfg) -> dict:
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "final.norm": (W,), "final.norm.b": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (W,)
        if layer["type"] == "latent_attention":
            H = m["heads"]
            shapes.update({p + "mix.q": (H * (m["dim"] + m["rot_dim"]), W), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                           p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.o": (W, H * m["vdim"])})
            if "kv_from" not in m:
                shapes.update({p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W), p + "mix.dkv.norm": (m["kv_rank"],)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            shapes.update({p + "mix.in": (2 * inner + 2 * gn + m["heads"], W), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                           p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (m["heads"],), p + "mix.A_log": (m["heads"],),
                           p + "mix.D": (m["heads"],), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        f = layer["mlp"]
        if f is None:
            continue
        shapes[p + "norm2"] = shapes[p + "norm2.b"] = (W,)
        if f["kind"] == "dense":
            shapes.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        else:
            shapes[p + "mlp.router"] = (f["router"]["experts"], W)
            names = [f"e{e}" for e in range(f["router"]["experts"])]
            sizes = [f["expert"]["ff"]] * len(names)
            if f.get("shared"):
                names.append("shared")
                sizes.append(f["shared"]["ff"])
            for n, ff in zip(names, sizes):
                shapes.update({f"{p}mlp.{n}.gate": (ff, W), f"{p}mlp.{n}.up": (ff, W), f"{p}mlp.{n}.down": (W, ff)})
    return shapes


def draw_tensors(cfg, seed: int, std: float = 0.25) -> dict:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g)
        if name.endswith(".b"):
            t = 0.1 * r
        elif "norm" in name:
            t = 1.0 + 0.1 * r
        elif name.endswith("A_log"):
            t = -3.0 + 2.5 * torch.rand(shape, generator=g)
        elif name.endswith("dt_bias"):
            t = -1.0 + 0.5 * r
        elif name.endswith(".D"):
            t = 1.0 + 0.3 * r
        elif name.endswith("mix.conv"):
            t = 0.5 * r
        elif name.endswith("router"):
            t = 0.5 * r
        elif name == "embed":
            t = r
        else:
            t = std * r * (32.0 / max(shape[-1], 1)) ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out


def sharpen(cfg, tensors: dict, key_token: int, query_token: int, strength: float = 40.0) -> None:
    """Changes layer 0's query weights (a latent attention that makes its own latent) so that ``query_token`` scores
    ``key_token`` by about ``strength`` above every other key, in every head: the first layer's input depends on the token
    alone, so the plain key of ``key_token`` and the normed input of ``query_token`` are known from the weights."""
    layer = cfg["layers"][0]
    m = layer["mixer"]
    assert layer["type"] == "latent_attention" and "kv_from" not in m
    w = {k: v.double() for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = P.layer_norm(w["embed"][[key_token, query_token]] * cfg["embedding"]["scale"], w["l0.norm1"], w["l0.norm1.b"], eps)
    c, _ = P.latent_kv(x[:1], w, "l0.mix.", m, eps, [0])
    keys = (c @ w["l0.mix.uk"].T).reshape(m["heads"], m["dim"])                 # the key token's plain key, per head
    q = w["l0.mix.q"].reshape(m["heads"], m["dim"] + m["rot_dim"], -1).clone()
    xq = x[1]
    for h in range(m["heads"]):
        gain = strength / (m["scale"] * float(keys[h] @ keys[h]) * float(xq @ xq))
        q[h, : m["dim"]] += gain * torch.outer(keys[h], xq)
    tensors["l0.mix.q"] = q.reshape(w["l0.mix.q"].shape).to(torch.bfloat16)


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
        def wrapped(logits, top):
            route = self._orig(logits, top)
            experts = torch.as_tensor(route.expert).to(torch.int64).cpu()[route.inverse.cpu().long()].reshape(-1, top)
            self.calls.append(experts)
            return route
        self.kernels.moe_route = wrapped
        return self

    def __exit__(self, *exc):
        del self.kernels.moe_route


def routed_layers(cfg) -> list:
    return [i for i, layer in enumerate(cfg["layers"]) if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe"]
