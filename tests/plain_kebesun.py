"""Plain, slow implementation of the Kebesun decoder, used only as the tests' oracle.

Whole sequences on the CPU, no cache: attention sees the whole prefix through an explicit mask,
the recurrence walks the sequence token by token from a zero state.  One function per
mechanism; nothing is shared with the product package (config.json is parsed here, weights are
read with the `safetensors` package).  The default element type is float64, which bounds how
much of a difference between the engine and this file is rounding.

The model, in this file's notation (N: RMS norm with gain 1 + w; s1, s2: per-channel factors):

    e = E[token];  x = e
    a run of layers [start, stop) is walked `times` times with the same weights; before each walk
        x <- W_in [x ; e]
    per layer:   h = N(x);   x <- x + s1 * mixer(h) + s2 * ff(h)          (ff may be absent)
    logits = W_head N_f(x)

Three mixers: "attention" (grouped-query softmax attention over a sliding window that also keeps
the first tokens, rotate-half rotation with linearly stretched positions), "gla" (a matrix memory
per head with a decay per key channel) and "latent_attention" (keys and values expanded from a
normed low-rank latent, plus one rotated key part shared by the heads; YaRN-stretched rotation).
Two feed-forwards: dense SwiGLU, and a mixture of SwiGLU experts chosen by the largest router
logits and weighted by the softmax over the chosen logits.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------- small pieces

def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def swiglu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.t()) * (h @ up.t())) @ down.t()


# --------------------------------------------------------------------------- rotation

def frequencies(rot: dict):
    """Per pair i < dims/2: the frequency, and the factor on cos and sin.  scaling {factor}: every frequency divided by
    the factor.  scaling {factor, original, fast, slow}: YaRN."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])
    if "original" not in sc:
        return f / factor, 1.0
    original = float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]; the first rot.dims entries of each head turn, entry i with entry i + dims/2.  The angle is the
    float32 product of the position and the float32 frequency."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    f, m = frequencies(rot)
    angle = (positions.to(torch.float32)[:, None] * f.to(torch.float32)[None, :]).to(x.dtype)
    c, s = (torch.cos(angle) * m)[:, None, :], (torch.sin(angle) * m)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- masks and softmax attention

def visible(T: int, window: Optional[int] = None, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and (i - j < window or j < keep_first); no window: all j <= i."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m = m & ((i - j < window) | (j < keep_first))
    return m


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def window_attention(h, w, p, m, positions):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[p + "q"].t()).view(T, H, d), positions, m.get("rot"))
    k = rotate((h @ w[p + "k"].t()).view(T, G, d), positions, m.get("rot"))
    v = (h @ w[p + "v"].t()).view(T, G, dv)
    mask = m.get("mask") or {}
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T, mask.get("size"), int(mask.get("keep_first", 0))))
    return o.reshape(T, H * dv) @ w[p + "o"].t()


def latent_attention(h, w, p, m, eps, positions):
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].t()).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, m["rot"])
    down = h @ w[p + "dkv"].t()
    c = norm_plain(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, rank:], positions, m["rot"])                   # one head, shared
    k_plain = (c @ w[p + "uk"].t()).view(T, H, d)
    v = (c @ w[p + "uv"].t()).view(T, H, dv)
    qq = torch.cat([q_plain, q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, r)], dim=-1)
    o = softmax_attention(qq, kk, v, float(m["scale"]), visible(T))
    return o.reshape(T, H * dv) @ w[p + "o"].t()


# --------------------------------------------------------------------------- gated linear attention

def gla(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + "q"].t()).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].t()).view(T, H, d)
    v = (h @ w[p + "v"].t()).view(T, H, dv)
    z = (h @ w[p + "a1"].t()) @ w[p + "a2"].t() + w[p + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = norm_plain(o, w[p + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].t())) @ w[p + "o"].t()


# --------------------------------------------------------------------------- feed-forwards

def dense_ff(h, w, p):
    return swiglu(h, w[p + "gate"], w[p + "up"], w[p + "down"])


def route(h, w, p, top: int):
    """Chosen experts [T, top] and their weights: softmax over the chosen logits only."""
    z = h @ w[p + "router"].t() + w[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, w, p, mlp):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    idx, wt = route(h, w, p, top)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel():
                q = p + f"e{e}."
                out[rows] += wt[rows, j, None] * swiglu(h[rows], w[q + "gate"], w[q + "up"], w[q + "down"])
    return out


# --------------------------------------------------------------------------- the model

def layer(x, w, i, spec, eps, positions):
    p = f"l{i}."
    h = norm_one_plus(x, w[p + "norm1"], eps)
    m = spec["mixer"]
    if spec["type"] == "attention":
        y = window_attention(h, w, p + "mix.", m, positions)
    elif spec["type"] == "gla":
        y = gla(h, w, p + "mix.", m, eps)
    elif spec["type"] == "latent_attention":
        y = latent_attention(h, w, p + "mix.", m, eps, positions)
    else:
        raise ValueError(spec["type"])
    x = x + w[p + "ls1"] * y
    mlp = spec.get("mlp")
    if mlp is not None:
        f = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
        x = x + w[p + "ls2"] * f
    return x


def order_of_runs(cfg: dict) -> List[List[int]]:
    """The passes: each a list of layer numbers; a pass that belongs to the repeated run is marked by the caller."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [list(range(n))]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return [list(range(a))] + [list(range(a, b)) for _ in range(times)] + [list(range(b, n))]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, stream_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token."""
    dtype = w["embed"].dtype
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    eps = float(cfg["norm"]["eps"])
    e = w["embed"][tokens]
    x = e
    loop = cfg.get("loop")
    passes = order_of_runs(cfg)
    for k, run in enumerate(passes):
        looped = bool(loop) and 1 <= k <= int(loop["times"])
        if looped and run:
            x = torch.cat([x, e], dim=-1) @ w["loop.in"].t()
        for i in run:
            x = layer(x, w, i, cfg["layers"][i], eps, positions)
            if stream_out is not None:
                stream_out.append(x.clone())
    return norm_one_plus(x, w["final.norm"], eps).to(dtype) @ w["head"].t()
