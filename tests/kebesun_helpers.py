"""Shared by the Kebesun tests: small configurations of their own (sizes chosen so that nothing that could be equal is
equal: key, rotated and value sizes, heads and kv heads, windows that are no multiple of a page, kept first tokens below
and above a page, experts that are no power of two, `top` equal to one and to all), model folders with random weights in
which some tensors are set by hand so that what they do shows, and the comparison with the plain implementation."""
from __future__ import annotations

import functools
import os
from typing import Dict, Optional, Sequence

import torch

import helpers
import mini_llama_cpp_release_b200 as ml
import plain_kebesun as pk
from mini_llama_cpp_release_b200.config import ModelConfig

YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}


def attention(heads, kv_heads, dim, vdim, scale, rot=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if mask is not None:
        m["mask"] = mask
    return m


def gla(heads, dim, vdim, tau, decay_rank=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    if decay_rank:
        m["decay_rank"] = decay_rank
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"dims": rot_dim, "base": base, "scaling": scaling}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, eps, layers, loop=None):
    d = {"architecture": "Kebesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# all three mixers and all three feed-forwards; the middle two layers walked three times; a partial rotation with linear
# stretching; a window of 40 that keeps three first tokens; value heads narrower than key heads; a layer without a window
MIXED = model(300, 96, 1e-5, [
    {"type": "attention", "mlp": dense(112),
     "mixer": attention(6, 3, 32, 16, 0.2, {"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0}}, {"size": 40, "keep_first": 3})},
    {"type": "gla", "mlp": moe(48, 5, 2), "mixer": gla(3, 24, 40, 8.0, 6)},
    {"type": "latent_attention", "mlp": None, "mixer": latent(3, 24, 8, 20, 40, 0.17, 3000.0, YARN)},
    {"type": "attention", "mlp": moe(32, 4, 4),
     "mixer": attention(4, 1, 16, 16, 0.25, {"dims": 16, "base": 100.0, "scaling": None})},
], loop=(1, 3, 3))

# head size 64 and latent rows of 128 (the tensor-core attention kernels), a window of 70 that keeps 65 first tokens (more
# than a page), keys of 128 in the linear attention, the first layer alone walked twice
WIDE = model(257, 128, 2e-6, [
    {"type": "latent_attention", "mlp": dense(144), "mixer": latent(2, 64, 48, 40, 80, 0.1, 40000.0, {**YARN, "factor": 3.0})},
    {"type": "attention", "mlp": moe(64, 6, 3),
     "mixer": attention(4, 4, 64, 64, 0.11, {"dims": 64, "base": 1e6, "scaling": {"factor": 2.5}}, {"size": 70, "keep_first": 65})},
    {"type": "gla", "mlp": None, "mixer": gla(2, 128, 64, 32.0)},
], loop=(0, 1, 2))

# sizes the fast paths do not take: a width that is no multiple of 8, keys of 200, value heads of 36, a window of one token,
# more kept first tokens than the window is wide, no rotation at all, one expert of 33 chosen, tau of one, no repeated run
ODD = model(77, 100, 1e-5, [
    {"type": "gla", "mlp": moe(20, 33, 1), "mixer": gla(2, 200, 36, 1.0, 3)},
    {"type": "attention", "mlp": None, "mixer": attention(3, 3, 24, 40, 0.4, None, {"size": 1, "keep_first": 0})},
    {"type": "attention", "mlp": dense(36), "mixer": attention(2, 1, 16, 8, 0.3, {"dims": 8, "base": 50.0}, {"size": 5, "keep_first": 9})},
    {"type": "latent_attention", "mlp": None, "mixer": latent(5, 12, 6, 10, 30, 0.3)},
])

ONLY_ATTENTION = model(200, 64, 1e-5, [
    {"type": "attention", "mlp": None,
     "mixer": attention(6, 2, 48, 32, 0.17, {"dims": 24, "base": 300.0, "scaling": {"factor": 1.5}}, {"size": 33, "keep_first": 2})}])
ONLY_GLA = model(200, 64, 1e-5, [{"type": "gla", "mlp": None, "mixer": gla(5, 40, 24, 4.0, 8)}])
ONLY_LATENT = model(200, 64, 1e-5, [{"type": "latent_attention", "mlp": None, "mixer": latent(6, 20, 12, 28, 50, 0.21, 700.0, YARN)}])
ONLY_MOE = model(200, 64, 1e-5, [{"type": "gla", "mlp": moe(40, 7, 3), "mixer": gla(1, 8, 8, 2.0, 2)}])
LOOPED = model(200, 48, 1e-5, [{"type": "gla", "mlp": dense(40), "mixer": gla(2, 16, 24, 4.0, 4)},
                               {"type": "attention", "mlp": None, "mixer": attention(2, 2, 16, 16, 0.25, {"dims": 16, "base": 1e4})}],
               loop=(0, 2, 4))

# a latent of 280 with 24 rotated entries: cached rows of 304, above what the tensor-core attention kernels take
BIG_LATENT = model(120, 64, 1e-5, [{"type": "latent_attention", "mlp": None, "mixer": latent(2, 24, 24, 16, 280, 0.2, 900.0)}])

CONFIGS = {"big_latent": BIG_LATENT, "mixed": MIXED, "wide": WIDE, "odd": ODD, "attention": ONLY_ATTENTION, "gla": ONLY_GLA, "latent": ONLY_LATENT,
           "moe": ONLY_MOE, "looped": LOOPED}


def shape_weights(weights: Dict[str, torch.Tensor], seed: int, peaked: float = 1.0) -> None:
    """Random weights hide some faults.  The decays' biases are moved up (slow decays: tokens hundreds of places back still
    count), routers are made decisive (so that the chosen experts do not hang on the last bit), the per-channel factors of
    the branches are spread out, and with `peaked` the attention's queries are scaled so that single keys decide rows."""
    g = torch.Generator().manual_seed(seed)
    for name, t in weights.items():
        if name.endswith(".a2.b"):
            t.copy_(torch.randn(t.shape, generator=g) * 1.0 + 3.0)
        elif name.endswith(".router"):
            t.mul_(12.0)
        elif name.endswith(".router.b"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)
        elif name.endswith((".ls1", ".ls2")):
            t.copy_(torch.rand(t.shape, generator=g) * 1.5 + 0.25)
        elif name.endswith("mix.q") and peaked != 1.0:
            t.mul_(peaked)


@functools.lru_cache(maxsize=None)
def folder_of(name: str, seed: int = 1, std: float = 0.08, peaked: float = 1.0) -> str:
    from safetensors.torch import load_file, save_file
    folder = os.path.join(helpers.tmp_root(), f"kebesun_{name}_{seed}_{std}_{peaked}")
    ml.write_random_model(ModelConfig.from_dict(CONFIGS[name]), folder, seed, torch.bfloat16, std=std)
    path = os.path.join(folder, "model.safetensors")
    weights = {k: v.float() for k, v in load_file(path).items()}
    shape_weights(weights, seed, peaked)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, path)
    return folder


@functools.lru_cache(maxsize=None)
def oracle(folder: str):
    return pk.read_config(folder), pk.read_weights(folder, torch.float64)


def oracle_logits(folder: str, tokens: Sequence[int]) -> torch.Tensor:
    cfg, w = oracle(folder)
    return pk.forward(cfg, w, tokens).float()


TOL = {"float32": 1e-4, "bfloat16": 8e-2}       # the mixed model runs eight layers, each with two branches rounded to 16 bits
TOL_MANY = {"float32": (1e-4, 1e-4), "bfloat16": (3e-2, 0.3)}
# In the 16-bit engine a router's choice can differ from the plain implementation's where two logits lie within the
# rounding of the branch's input; such a token then takes another expert and its row is off by a visible amount, as it
# would be in any 16-bit evaluation.  The 16-bit comparison therefore lets a few rows in a hundred pass the bound on single
# rows (the mean over all rows stays bounded); the 32-bit comparison, whose routers see the same numbers as the plain
# implementation to six digits, lets none.
ROWS_OFF = {"float32": 0.0, "bfloat16": 0.04}


def check(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str, many: bool = False) -> None:
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert bool(torch.isfinite(got).all()), what
    errs = sorted(helpers.rel_err(got[i], want[i]) for i in range(got.shape[0]))
    spared = int(ROWS_OFF[dtype] * len(errs)) + (1 if dtype == "bfloat16" and len(errs) >= 10 else 0)
    kept = errs[:len(errs) - spared] if spared else errs
    if many:
        mean_tol, max_tol = TOL_MANY[dtype]
        mean = sum(kept) / len(kept)                   # of the rows that are held to the bound: a spared row can be off by its whole size
        assert mean <= mean_tol and kept[-1] <= max_tol, f"{what}: mean {mean:.3e}, worst {errs[-1]:.3e}, worst kept {kept[-1]:.3e}"
    else:
        assert kept[-1] <= TOL[dtype], f"{what}: worst {errs[-1]:.3e}, worst kept {kept[-1]:.3e}"
