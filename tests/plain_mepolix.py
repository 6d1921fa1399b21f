"""Plain, slow implementation of the Mepolix decoder, used only as the tests' oracle.

Whole sequences on the CPU, no cache: attention sees the whole prefix, recurrences walk the
sequence token by token from a zero state.  One function per mechanism; nothing is shared
with the product package (config.json is parsed here, weights are read with the `safetensors`
package).  The default element type is float64, which bounds how much of a difference between
the engine and this file is rounding.

The model, in this file's notation (h: a sublayer's input, the residual stream itself):

    x_0 = E[token]
    per layer:   x <- x + LN_1(mixer(x));   x <- x + LN_2(ff(x))   (the second only with a feed-forward)
    logits = c * tanh(W_head LN_f(x) / c)

LN is a layer norm with a gain and no bias.  Two mixers exist: "delta" (a gated delta-rule
memory) and "parallel" (softmax attention with a sink beside a gated linear recurrence,
summed with two fixed factors).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------- small pieces

def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w, var the mean squared deviation."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], w [C, taps]: y_t = sum_j w[:, taps-1-j] * x_{t-j}, zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        shifted = torch.zeros_like(x)
        if j < T:
            shifted[j:] = x[:T - j]
        y = y + shifted * w[:, taps - 1 - j]
    return y if b is None else y + b


# --------------------------------------------------------------------------- rotation

def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """Per pair i < dims/2: the frequency and the factor on cos and sin."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]; the first rot.dims entries of each head turn, pair (i, i + dims/2); the angle is formed in
    float32 as the product of the position and the float32 frequency."""
    dims = int(rot["dims"])
    f, m = yarn_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    angle = (positions.to(torch.float32)[:, None] * f.to(torch.float32)[None, :]).to(x.dtype)     # [T, dims/2]
    c, s = (torch.cos(angle) * m)[:, None, :], (torch.sin(angle) * m)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- attention with a sink

def sink_attention(h, w, p, m, eps, positions):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].t()).view(T, H, d)
    k = (h @ w[p + "k"].t()).view(T, G, d)
    v = (h @ w[p + "v"].t()).view(T, G, dv)
    q = rotate(rms_norm(q, w[p + "q.norm"], eps), positions, m["rot"])
    k = rotate(rms_norm(k, w[p + "k.norm"], eps), positions, m["rot"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    causal = positions[:, None] >= positions[None, :]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].t()) * m["scale"]
        s = s.masked_fill(~causal, float("-inf"))
        sink = w[p + "sink"][head]
        mx = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        out[:, head] = (e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - mx))) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


# --------------------------------------------------------------------------- gated linear recurrence

def gated_recurrence(h, w, p, m):
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].t() + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].t() + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
    log_a = -8.0 * r * F.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(W, dtype=h.dtype)
    out = torch.zeros(T, W, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w[p + "o"].t()


def parallel_mixer(h, w, p, m, eps, positions):
    left = sink_attention(h, w, p + "left.", m["left"], eps, positions)
    right = gated_recurrence(h, w, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


# --------------------------------------------------------------------------- gated delta rule

def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].t(), w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].t(), w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].t(), w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].t())                                            # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(h @ w[p + "a"].t() + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].t()).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.t() @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.t() @ q[t, g]
    out = rms_norm(out, w[p + "norm"], eps) * gate
    return out.reshape(T, H * dv) @ w[p + "o"].t()


# --------------------------------------------------------------------------- feed-forward, model

def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and, on request, the residual stream after every layer run)."""
    dtype = w["embed"].dtype
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    positions = torch.arange(len(tokens))
    streams: List[torch.Tensor] = []
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % layer.get("weights_of", i)
        if layer["type"] == "delta":
            y = delta_mixer(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(x, w, p + "mix.", layer["mixer"], eps, positions)
        else:
            raise ValueError("unknown layer type " + str(layer["type"]))
        x = x + layer_norm(y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(dense_ff(x, w, p + "mlp."), w[p + "norm2"], eps)
        streams.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].t()
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    logits = logits.to(dtype)
    return (logits, torch.stack(streams)) if return_layers else logits
