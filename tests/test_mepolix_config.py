"""Mepolix on the CPU: its config.json is read and checked, the model specification has the schedule and the tensors the
layers' list asks for, the stretched frequencies are the plain implementation's, and the plain implementation's pieces
agree with textbook forms of themselves."""
import copy
import math

import numpy as np
import pytest
import torch

import mepolix_helpers as mh
import plain_mepolix as pm
from mini_llama_cpp_release_b200.config import ConfigError, ModelConfig, build_model_spec
from mini_llama_cpp_release_b200.engine.model import build_parts
from mini_llama_cpp_release_b200.parts.rotary import stretched_frequencies
from mini_llama_cpp_release_b200.weights.loader import expected_tensors


def test_config_is_read_by_its_own_class_and_round_trips():
    cfg = ModelConfig.from_dict(mh.MIXED)
    assert type(cfg).__name__ == "MepolixConfig" and cfg.architecture == "Mepolix"
    assert cfg.vocab_size == 300 and cfg.hidden_size == 72 and cfg.norm_eps == 1e-5 and cfg.logit_softcap == 12.0
    assert ModelConfig.from_dict(cfg.to_dict()) == cfg
    assert ModelConfig.from_dict(mh.TALL).logit_softcap is None


def test_a_layer_that_uses_anothers_weights_is_a_second_run_of_it():
    spec = build_model_spec(ModelConfig.from_dict(mh.MIXED))
    assert [l.name for l in spec.layers] == ["l0.", "l1.", "l3."]
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 2]
    assert all(e.reads_cache_of is None for e in spec.schedule)          # a cache and state of its own


def test_tensors_follow_the_layers_list():
    parts = build_parts(build_model_spec(ModelConfig.from_dict(mh.MIXED))).all_parts()
    t = {k: tuple(v.shape) for k, v in expected_tensors(parts).items()}
    assert t["embed"] == (300, 72) and t["head"] == (300, 72) and t["final.norm"] == (72,)
    assert t["l0.mix.left.q"] == (4 * 32, 72) and t["l0.mix.left.k"] == (2 * 32, 72) and t["l0.mix.left.v"] == (2 * 16, 72)
    assert t["l0.mix.left.o"] == (72, 4 * 16) and t["l0.mix.left.sink"] == (4,) and t["l0.mix.left.q.norm"] == (32,)
    assert t["l0.mix.right.ra"] == (3, 32, 32) and t["l0.mix.right.ri.b"] == (3, 32) and t["l0.mix.right.conv"] == (96, 4)
    assert t["l0.mix.right.lam"] == (96,) and t["l0.mix.right.y.b"] == (96,) and t["l0.mix.right.o"] == (72, 96)
    assert t["l0.mlp.gate"] == (112, 72) and t["l0.mlp.down"] == (72, 112) and t["l0.norm2"] == (72,)
    assert t["l1.mix.q"] == (2 * 16, 72) and t["l1.mix.v"] == (4 * 24, 72) and t["l1.mix.v.conv"] == (96, 2)
    assert t["l1.mix.b"] == (4, 72) and t["l1.mix.A_log"] == (4,) and t["l1.mix.norm"] == (24,) and t["l1.mix.o"] == (72, 96)
    assert "l1.norm2" not in t and "l1.mlp.gate" not in t                 # no feed-forward there
    assert not any(k.startswith("l2.") for k in t)                        # layer 2 has no tensors of its own
    assert t["l3.mix.q.conv"] == (3 * 40, 3) and t["l3.mlp.up"] == (80, 72)


@pytest.mark.parametrize("change, key", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][2].update(weights_of=1), "another type"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "dense"),
])
def test_bad_configurations_are_refused_with_the_key(change, key):
    raw = copy.deepcopy(mh.MIXED)
    change(raw)
    with pytest.raises(ConfigError) as e:
        build_model_spec(ModelConfig.from_dict(raw))
    assert key in str(e.value)


@pytest.mark.parametrize("dims, base, scaling", [(16, 5000.0, mh.YARN), (64, 1e6, None), (8, 100.0, {**mh.YARN, "factor": 2.0}),
                                                 (96, 250000.0, {"factor": 3.0, "original": 512, "fast": 24.0, "slow": 0.5})])
def test_stretched_frequencies_are_the_plain_ones(dims, base, scaling):
    f, m = stretched_frequencies(dims, base, scaling)
    want_f, want_m = pm.yarn_frequencies(dims, base, scaling)
    assert f.dtype == np.float32 and np.array_equal(f, want_f.to(torch.float32).numpy()) and m == pytest.approx(want_m)
    if scaling is None:
        assert m == 1.0 and f[0] == 1.0
    else:
        plain = np.power(base, -2.0 * np.arange(dims // 2) / dims)
        assert np.all(f <= plain.astype(np.float32)) and np.all(f >= (plain / scaling["factor"]).astype(np.float32) * 0.999999)


def test_plain_pieces_against_textbook_forms():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 12, generator=g, dtype=torch.float64)
    w = torch.randn(12, generator=g, dtype=torch.float64)
    assert torch.allclose(pm.layer_norm(x, w, 1e-5), torch.nn.functional.layer_norm(x, (12,), w, None, 1e-5))
    assert torch.allclose(pm.gelu_tanh(x), torch.nn.functional.gelu(x, approximate="tanh"))
    cw = torch.randn(12, 3, generator=g, dtype=torch.float64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(x.t()[None], (2, 0)), cw[:, None, :], groups=12)[0].t()
    assert torch.allclose(pm.causal_conv(x, cw), want)
    # a rotation keeps a pair's length (times the factor) and turns by position x frequency
    r = pm.rotate(torch.ones(4, 1, 8, dtype=torch.float64), torch.arange(4), {"dims": 4, "base": 10.0, "scaling": None})
    assert torch.allclose(r[..., 4:], torch.ones(4, 1, 4, dtype=torch.float64))
    assert torch.allclose(r[..., 0] ** 2 + r[..., 2] ** 2, torch.full((4, 1), 2.0, dtype=torch.float64))
    assert math.isclose(float(r[1, 0, 0]), math.cos(1.0) - math.sin(1.0), rel_tol=1e-6)


def test_inspect_and_random_weights_on_the_command_line(tmp_path):
    """Random weights of the design are written without a GPU, and `inspect` reads them back: the schedule with its
    second run, the cache of the attention runs and the state of every run."""
    import subprocess
    import sys
    import os
    import mini_llama_cpp_release_b200 as ml
    folder = ml.write_random_model(ModelConfig.from_dict(mh.MIXED), str(tmp_path / "m"), seed=3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "mini_llama_cpp_release_b200", "inspect", folder], capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "architecture: Mepolix -> 3 layers, 4 runs per step" in p.stdout
    assert "l0.mix.left.sink" in p.stdout and "PROBLEM" not in p.stdout
    # two attention runs of 2 kv heads x 32 entries (keys and values), in bfloat16
    assert f"cache per token per sequence: {2 * 2 * 2 * 32 * 2} B in bfloat16" in p.stdout
    # parallel: 96 channels x 4 taps; delta: 4 x 16 x 24 + 1 x (32 + 32 + 96); delta: 3 x 40 x 20 + 2 x (120 + 120 + 60)
    want = 4 * (2 * 96 * 4 + (4 * 16 * 24 + 160) + (3 * 40 * 20 + 2 * 300))
    assert f"state per sequence: {want} B in 4 of 4 runs" in p.stdout
