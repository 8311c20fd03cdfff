"""The Lafanex decoder written plainly: one function a mechanism, float64, whole sequences, no cache, no batching. It
shares nothing with the package; the tests compare the engine with it.

A model: token embedding; ``streams`` copies of the residual (hyper-connections); layers in the order the configuration
gives, a range of which runs several times with the same weights; a final norm; logits against the embedding table.
A layer: x <- x + mixer(norm1(x)), x <- x + ff(norm2(x)), each sum replaced by the hyper-connection's read, mix and write.
Mixers: causal attention with grouped heads, a rotation of interleaved pairs, unit-root-mean-square queries and keys and
one added to the softmax's denominator; the Mamba selective scan. Feed-forwards: a gated one with the tanh form of
GELU; routed experts with softmax scores, a correction that only the choice sees, identity experts and a gated shared
expert.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ small functions
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, dim]: elements (2i, 2i+1), i < dims/2, turned by the angle position * base^(-2i/dims); the rest pass."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def sink_attention(h, w, p, m, eps, positions=None):
    """h [T, width] -> [T, width]. p: the tensors' prefix ('l0.mix.')."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T)) if positions is None else positions
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = unit_rms(rotate_pairs(q, positions, m["rot"]["dims"], m["rot"]["base"]), eps)
    k = unit_rms(rotate_pairs(k, positions, m["rot"]["dims"], m["rot"]["base"]), eps)
    out = torch.zeros(T, H, dv, dtype=F64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        e = torch.where(causal, torch.exp(s), torch.zeros_like(s))
        weights = e / (1.0 + e.sum(-1, keepdim=True))        # the sink: a key of score 0 that has no value
        out[:, head] = weights @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def mamba1(h, w, p, m):
    """The selective scan from an empty state and zeros before the sequence's start."""
    T = h.shape[0]
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=F64), x])
    conv = torch.stack([(padded[t : t + taps] * w[p + "conv"].T).sum(0) for t in range(T)]) + w[p + "conv.b"]
    x = silu(conv)
    dbc = x @ w[p + "x"].T
    dt = softplus(dbc[:, :R] @ w[p + "dt"].T + w[p + "dt.b"])              # [T, inner]
    B, C = dbc[:, R : R + N], dbc[:, R + N :]
    A = -torch.exp(w[p + "A_log"])                                            # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routed_ff(h, w, p, f, forced=None, slack=0.0):
    """``forced`` [T, top]: the experts to use instead of choosing (each is checked to lie within ``slack`` of the
    ``top``-th best choice score)."""
    r = f["router"]
    E, top, I = r["experts"], r["top"], r.get("identity", 0)
    z = h @ w[p + "router"].T
    s = torch.softmax(z, dim=-1)                       # over the experts and the identity experts
    choice = s + w[p + "correction"]
    if forced is None:
        chosen = torch.topk(choice, top, dim=-1).indices
    else:
        chosen = torch.as_tensor(forced).long()
        kth = torch.topk(choice, top, dim=-1).values[:, -1:]
        assert bool((choice.gather(1, chosen) >= kth - slack).all()), "a forced expert is not near the best choices"
        assert all(len(set(row.tolist())) == top for row in chosen), "a forced choice names an expert twice"
    out = torch.zeros_like(h)
    outputs = {e: clamped_expert(h, w, f"{p}e{e}.", f["expert"]["limit"]) for e in range(E)}
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            weight = s[t, e] * r["scale"]
            out[t] += weight * (outputs[e][t] if e < E else h[t])      # an identity expert gives its input back
    if f.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)                 # [T, 1]
        out = out + gate * clamped_expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------ the model
def layer_order(cfg) -> list:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def hyper_sublayer(streams, w, p, eps, norm_w, fn):
    """streams [S, T, width]: read u = sum_s in[s] x_s, y = fn(norm(u)), then every stream at once from the old ones:
    x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,stw->tw", w[p + "in"], streams)
    y = fn(offset_norm(u, norm_w, eps))
    return torch.einsum("sr,stw->rtw", w[p + "mix"], streams) + w[p + "out"][:, None, None] * y[None]


def plain_sublayer(x, eps, norm_w, fn):
    return x + fn(offset_norm(x, norm_w, eps))


def forward(cfg, w, ids, forced=None, slack=0.0, layer_outputs=None):
    """Logits [T, vocab] of the sequence ``ids`` (float64). ``forced``: {layer run index: [T, top] experts}.
    ``layer_outputs``: a list that receives the residual (the sum of the streams) after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids).long()]
    S = cfg.get("streams")
    streams = torch.stack([x] * S) if S else None
    for run, i in enumerate(layer_order(cfg)):
        layer, p = cfg["layers"][i], f"l{i}."
        m = layer["mixer"]
        mixer = ((lambda h: sink_attention(h, w, p + "mix.", m, eps)) if layer["type"] == "attention"
                 else (lambda h: mamba1(h, w, p + "mix.", m)))
        f = layer.get("mlp")
        ff = None
        if f is not None:
            ff = ((lambda h: dense_ff(h, w, p + "mlp.")) if f["kind"] == "dense"
                  else (lambda h: routed_ff(h, w, p + "mlp.", f, None if forced is None else forced.get(run), slack)))
        if S:
            streams = hyper_sublayer(streams, w, p + "hc1.", eps, w[p + "norm1"], mixer)
            if ff is not None:
                streams = hyper_sublayer(streams, w, p + "hc2.", eps, w[p + "norm2"], ff)
            x = streams.sum(0)
        else:
            x = plain_sublayer(x, eps, w[p + "norm1"], mixer)
            if ff is not None:
                x = plain_sublayer(x, eps, w[p + "norm2"], ff)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T
