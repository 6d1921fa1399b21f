"""Shared by the Mepolix tests: small configurations of their own (sizes chosen so that nothing that could be equal is
equal: key and value head sizes, rotated and whole head size, kv heads > 1, taps that differ between mixers, widths that
are no multiple of 32), model folders with random weights in which some tensors are set by hand so that what they do
shows, and the comparison with the plain implementation."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Optional, Sequence

import torch

import helpers
import mini_llama_cpp_release_b200 as ml
import plain_mepolix as pm
from mini_llama_cpp_release_b200.config import ModelConfig


def rot(dims, base=10000.0, scaling=None):
    return {"dims": dims, "base": base, "scaling": scaling}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}

# mixed: both types, with and without a feed-forward, a layer that runs another's weights again, a partial stretched
# rotation, value heads narrower than key heads, two kv heads, taps 4 / 2 / 3
MIXED = {
    "architecture": "Mepolix", "vocab": 300, "width": 72, "logit_softcap": 12.0, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 112},
         "mixer": parallel({"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.21, "rot": rot(16, 5000.0, YARN)},
                           {"width": 96, "blocks": 3, "conv": 4}, 1.3, 0.8)},
        {"type": "delta", "mlp": None, "mixer": delta(4, 2, 16, 24, 2)},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 112}, "weights_of": 0,
         "mixer": parallel({"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.21, "rot": rot(16, 5000.0, YARN)},
                           {"width": 96, "blocks": 3, "conv": 4}, 1.3, 0.8)},
        {"type": "delta", "mlp": {"kind": "dense", "ff": 80}, "mixer": delta(3, 3, 40, 20, 3)},
    ],
}

# wide heads: head size 64 on both sides of the attention (the tcgen05 prompt kernel), one head per kv head, the whole
# head rotated without stretching, a delta rule with 128-entry keys, one tap (no convolution state), one gate block
WIDE = {
    "architecture": "Mepolix", "vocab": 257, "width": 128, "logit_softcap": 30.0, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "delta", "mlp": {"kind": "dense", "ff": 144}, "mixer": delta(2, 1, 128, 64, 1)},
        {"type": "parallel", "mlp": None,
         "mixer": parallel({"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "rot": rot(64, 1e6)},
                           {"width": 64, "blocks": 1, "conv": 2}, 0.7, 1.1)},
    ],
}

# value heads wider than key heads, sixteen query heads on one kv head, no soft cap
TALL = {
    "architecture": "Mepolix", "vocab": 128, "width": 48, "logit_softcap": None, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 64},
         "mixer": parallel({"heads": 16, "kv_heads": 1, "dim": 16, "vdim": 48, "scale": 0.3, "rot": rot(8, 100.0, {**YARN, "factor": 2.0})},
                           {"width": 40, "blocks": 5, "conv": 3}, 1.0, 1.0)},
    ],
}

ONLY_DELTA = {"architecture": "Mepolix", "vocab": 200, "width": 64, "logit_softcap": 20.0, "norm": {"eps": 1e-5},
              "layers": [{"type": "delta", "mlp": None, "mixer": delta(6, 2, 24, 40, 4)}]}
ONLY_PARALLEL = {"architecture": "Mepolix", "vocab": 200, "width": 64, "logit_softcap": 20.0, "norm": {"eps": 1e-5},
                 "layers": [{"type": "parallel", "mlp": None,
                             "mixer": parallel({"heads": 6, "kv_heads": 3, "dim": 48, "vdim": 32, "scale": 0.17, "rot": rot(24, 300.0, YARN)},
                                               {"width": 72, "blocks": 2, "conv": 5}, 0.9, 1.4)}]}

# sizes the fast paths do not take: a width that is no multiple of 8 (the library's product), 200-entry keys (one token a
# round), value heads of 36 (no 16-byte copies), nine taps (the plain convolution), a head that is not rotated at all,
# value heads wider than key heads, gate blocks of 20, one tap, a delta layer that runs another's weights again
ODD_A = {
    "architecture": "Mepolix", "vocab": 77, "width": 100, "logit_softcap": 8.0, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "delta", "mlp": {"kind": "dense", "ff": 36}, "mixer": delta(2, 1, 200, 36, 9)},
        {"type": "parallel", "mlp": None,
         "mixer": parallel({"heads": 3, "kv_heads": 3, "dim": 24, "vdim": 40, "scale": 0.4, "rot": rot(0, 10000.0)},
                           {"width": 60, "blocks": 3, "conv": 1}, 0.5, 2.0)},
        {"type": "delta", "mlp": {"kind": "dense", "ff": 36}, "mixer": delta(2, 1, 200, 36, 9), "weights_of": 0},
    ],
}
# two attention layers of different shapes (two cache groups; one with 128-entry value heads on 64-entry keys), eight
# delta heads of 8 x 8, eight taps, no soft cap
ODD_B = {
    "architecture": "Mepolix", "vocab": 150, "width": 64, "logit_softcap": None, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 48},
         "mixer": parallel({"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25, "rot": rot(16, 777.0)},
                           {"width": 128, "blocks": 4, "conv": 2}, 1.0, 1.0)},
        {"type": "delta", "mlp": None, "mixer": delta(8, 8, 8, 8, 2)},
        {"type": "parallel", "mlp": None,
         "mixer": parallel({"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 128, "scale": 0.11, "rot": rot(32, 1e5, YARN)},
                           {"width": 32, "blocks": 1, "conv": 8}, -0.8, 0.6)},
    ],
}

CONFIGS = {"mixed": MIXED, "wide": WIDE, "tall": TALL, "delta": ONLY_DELTA, "parallel": ONLY_PARALLEL, "odd_a": ODD_A, "odd_b": ODD_B}


def shape_weights(weights: Dict[str, torch.Tensor], seed: int) -> None:
    """Random weights hide some faults: a sink near zero counts like one more key, decays near one half forget within a few
    tokens.  Sinks are spread out (so that a softmax without them is far off), the delta rule's and the recurrence's
    decays are moved close to one (so that tokens hundreds of places back still count), and biases are made large enough
    to matter."""
    g = torch.Generator().manual_seed(seed)
    for name, t in weights.items():
        if name.endswith(".sink"):
            t.copy_(torch.randn(t.shape, generator=g) * 1.5 + 1.0)
        elif name.endswith(".A_log"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5 - 3.0)
        elif name.endswith(".dt_bias"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)
        elif name.endswith(".lam"):
            t.copy_(torch.randn(t.shape, generator=g) * 1.0 - 4.0)
        elif name.endswith(".b") and t.dim() <= 2 and not name.endswith("mix.b"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.3)
        elif name.endswith(".conv"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)


@functools.lru_cache(maxsize=None)
def folder_of(name: str, seed: int = 1, std: float = 0.08, sink_mean: Optional[float] = None) -> str:
    """`sink_mean`: the sinks are drawn around this value instead (about the logarithm of the number of keys makes the sink
    weigh as much as all keys together, so that it still shows in a long sequence)."""
    from safetensors.torch import load_file, save_file
    folder = os.path.join(helpers.tmp_root(), f"mepolix_{name}_{seed}_{std}_{sink_mean}")
    ml.write_random_model(ModelConfig.from_dict(CONFIGS[name]), folder, seed, torch.bfloat16, std=std)
    path = os.path.join(folder, "model.safetensors")
    weights = {k: v.float() for k, v in load_file(path).items()}
    shape_weights(weights, seed)
    if sink_mean is not None:
        for k, t in weights.items():
            if k.endswith(".sink"):
                t.copy_(sink_mean + 0.5 * torch.randn(t.shape, generator=torch.Generator().manual_seed(seed + 7)))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, path)
    return folder


@functools.lru_cache(maxsize=None)
def oracle(folder: str):
    return pm.read_config(folder), pm.read_weights(folder, torch.float64)


def oracle_logits(folder: str, tokens: Sequence[int]) -> torch.Tensor:
    cfg, w = oracle(folder)
    return pm.forward(cfg, w, tokens).float()


TOL = {"float32": 1e-4, "bfloat16": 6e-2}
# Over hundreds of rows the 16-bit engine's error has a long tail: rounding the branches' inputs to bfloat16 in the plain
# implementation alone moves single rows of these small models by a tenth of their largest logit, at a mean of a
# hundredth.  Long comparisons therefore bound the mean and, more loosely, the worst row.
TOL_MANY = {"float32": (1e-4, 1e-4), "bfloat16": (3e-2, 0.3)}


def check(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str, many: bool = False) -> None:
    assert got.shape == want.shape, (what, got.shape, want.shape)
    errs = [helpers.rel_err(got[i], want[i]) for i in range(got.shape[0])]
    if many:
        mean_tol, max_tol = TOL_MANY[dtype]
        assert sum(errs) / len(errs) <= mean_tol and max(errs) <= max_tol, f"{what}: mean {sum(errs) / len(errs):.3e}, worst {max(errs):.3e}"
    else:
        assert max(errs) <= TOL[dtype], f"{what}: {max(errs):.3e}"
