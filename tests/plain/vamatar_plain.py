"""Plain, slow implementation of the Vamatar decoder: whole sequences, no cache, no pages, one function a mechanism.

Vamatar is a pre-norm decoder whose layers mix tokens either by a latent attention (keys and values are made per head
from one small latent vector a token, plus one rotated key part that all heads share; a sliding window; a layer may
read the latent of an earlier layer instead of making its own) or by a Mamba-2 recurrence (a short causal convolution,
then a state of N x P numbers a head that decays and takes in an outer product at every token), and whose feed-forward
is a gated one, dense or routed over small experts with a shared expert beside them. Norms are layer norms with bias,
the embedding is scaled and the logits are capped by a tanh.

Nothing here is shared with the product path under ``roost_b200/``: the tests compare the two. All arithmetic is
float64; weights are taken as given (the caller rounds matrices to bfloat16 first when the engine under test does).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from .qwen3_plain import read_safetensors

F64 = torch.float64


def load_model_dir(model_dir) -> tuple[dict, dict]:
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in read_safetensors(model_dir / "model.safetensors").items()}
    return cfg, w


# ---------------------------------------------------------------------------------------------- small functions
def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * w + b with var the mean squared deviation."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight + bias


def unit_rms(x, eps):
    """x over its root mean square, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_half_pairs(x, positions, base, dims):
    """Element i < dims/2 of the last axis is paired with element i + dims/2; the pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims). Elements from ``dims`` on pass unchanged.
    x: [T, ..., n]; positions: T integers."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    a = torch.as_tensor(positions, dtype=F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---------------------------------------------------------------------------------------------- latent attention
def latent_kv(h, w, prefix, m, eps, positions):
    """The latent c [T, kv_rank] (unit-rms times a weight) and the shared rotated key part [T, rot_dim] of a layer that
    makes its own."""
    r = m["kv_rank"]
    d = h @ w[prefix + "dkv"].T
    c = unit_rms(d[:, :r], eps) * w[prefix + "dkv.norm"]
    kr = rotate_half_pairs(d[:, r:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, w, prefix, m, eps, positions, kv):
    """kv = (c, kr) of this layer or of the layer it reads. Per head: key = [W_uk c | kr], value = W_uv c,
    query = [q_plain | rotated q_rot]; score = q . k * scale over the keys j with 0 <= i - j < window."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kv
    q = (h @ w[prefix + "q"].T).reshape(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_half_pairs(q[..., dn:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ w[prefix + "uk"].T).reshape(T, H, dn)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for hd in range(H):
            s = (kn[lo : i + 1, hd] @ qn[i, hd] + kr[lo : i + 1] @ qr[i, hd]) * m["scale"]
            p = torch.softmax(s, 0)
            out[i, hd] = p @ v[lo : i + 1, hd]
    return out.reshape(T, H * dv) @ w[prefix + "o"].T


# ---------------------------------------------------------------------------------------------- mamba-2
def causal_conv(x, weight, bias):
    """out[t, c] = b[c] + sum_k w[c, k] x[t - (taps - 1) + k, c], zeros before the start (the last tap is the token's own)."""
    T, taps = x.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x])
    out = bias.expand(T, -1).clone()
    for k in range(taps):
        out = out + padded[k : k + T] * weight[:, k]
    return out


def mamba2(h, w, prefix, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ w[prefix + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner : 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N :]
    xbc = silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner : inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N :].reshape(T, G, N)
    dt = softplus(dt + w[prefix + "dt_bias"])                       # [T, H]
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]) * dt)         # [T, H]
    per_group = H // G
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        for hd in range(H):
            g = hd // per_group
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w[prefix + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"]
    return y @ w[prefix + "o"].T


# ---------------------------------------------------------------------------------------------- feed-forwards
def gated_ff(x, w, prefix):
    return (silu(x @ w[prefix + "gate"].T) * (x @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def routed_ff(x, w, prefix, f, round_input=None, forced=None, slack=0.0):
    """Scores sigmoid(W_router x); the ``top`` largest choose the experts; each chosen expert is given score * x and the
    outputs are summed; a shared expert, when the layer has one, sees x itself. ``round_input``: what the engine under
    test does to an expert's scaled input (rounding to bfloat16), None for nothing. ``forced`` [T, top]: the experts an
    engine chose; they are used instead of this function's own choice after a check that each one's router logit is
    within ``slack`` of the ``top``-th largest (an engine in lower precision may order near-equal scores differently)."""
    E, top = f["router"]["experts"], f["router"]["top"]
    z = x @ w[prefix + "router"].T
    s = torch.sigmoid(z)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        if forced is not None:
            mine, order = order, [int(e) for e in forced[t]]
            assert len(set(order)) == top, f"token {t}: the engine chose {order}"
            for e in order:
                assert float(z[t, e]) >= float(z[t, mine[-1]]) - slack, f"token {t}: the engine chose expert {e}, logit {float(z[t, e])}, but the {top}-th largest is {float(z[t, mine[-1]])}"
        for e in order:
            xin = (s[t, e] * x[t])[None, :]
            if round_input is not None:
                xin = round_input(xin)
            out[t] += gated_ff(xin, w, f"{prefix}e{e}.")[0]
    if f.get("shared"):
        out = out + gated_ff(x, w, prefix + "shared.")
    return out


# ---------------------------------------------------------------------------------------------- the model
def forward(cfg, w, ids, return_layers: bool = False, round_input=None, forced=None, slack=0.0):
    """Logits [T, vocab] of one sequence at positions 0..T-1 (and the stream after every layer when asked). ``forced``:
    {layer index: [T, top] experts} for routed layers whose choices are given (see ``routed_ff``)."""
    eps = cfg["norm"]["eps"]
    positions = list(range(len(ids)))
    h = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept, layers = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        x = layer_norm(h, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(x, w, p + "mix.", m, eps, positions)
                src = i
            h = h + latent_attention(x, w, p + "mix.", m, eps, positions, kept[src])
        elif layer["type"] == "mamba2":
            h = h + mamba2(x, w, p + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: no mixer '{layer['type']}'")
        f = layer.get("mlp")
        if f is not None:
            x = layer_norm(h, w[p + "norm2"], w[p + "norm2.b"], eps)
            if f["kind"] == "dense":
                h = h + gated_ff(x, w, p + "mlp.")
            elif f["kind"] == "moe":
                h = h + routed_ff(x, w, p + "mlp.", f, round_input, None if forced is None else forced.get(i), slack)
            else:
                raise ValueError(f"layer {i}: no feed-forward '{f['kind']}'")
        layers.append(h)
    x = layer_norm(h, w["final.norm"], w["final.norm.b"], eps)
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if return_layers else logits
