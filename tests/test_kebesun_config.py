"""Kebesun without a GPU: its configuration, the order in which its layers run, what each run asks of the cache, the
cache's bookkeeping of a window that keeps first tokens, and the plain implementation's mechanisms against each other."""
import copy

import pytest
import torch

import kebesun_helpers as kh
import plain_kebesun as pk
from mini_llama_cpp_release_b200.cache.paged import SlotBook, plan_groups
from mini_llama_cpp_release_b200.config import ModelConfig
from mini_llama_cpp_release_b200.config.model_config import ConfigError
from mini_llama_cpp_release_b200.config.registry import build_model_spec
from mini_llama_cpp_release_b200.engine.model import build_parts
from mini_llama_cpp_release_b200.parts.base import CacheNeed
from mini_llama_cpp_release_b200.parts.rotary import stretched_frequencies


def test_config_round_trip_and_checks():
    cfg = ModelConfig.from_dict(kh.MIXED)
    assert cfg.architecture == "Kebesun" and cfg.vocab_size == 300 and cfg.hidden_size == 96 and cfg.loop == (1, 3, 3)
    assert ModelConfig.from_dict(cfg.to_dict()) == cfg
    for path, value in [(("layers", 0, "type"), "conv"), (("loop", "stop"), 9), (("loop", "times"), 0),
                        (("layers", 1, "mlp", "kind"), "sparse")]:
        bad = copy.deepcopy(kh.MIXED)
        d = bad
        for key in path[:-1]:
            d = d[key]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            ModelConfig.from_dict(bad)


def test_the_repeated_run_is_walked_with_a_mixing_step_before_each_walk():
    spec = build_model_spec(ModelConfig.from_dict(kh.MIXED))
    mix = len(kh.MIXED["layers"])
    assert [e.layer for e in spec.schedule] == [0, mix, 1, 2, mix, 1, 2, mix, 1, 2, 3]
    assert spec.layers[mix].block.kind == "stream_mix"
    plain = build_model_spec(ModelConfig.from_dict(kh.ODD))
    assert [e.layer for e in plain.schedule] == [0, 1, 2, 3] and len(plain.layers) == 4
    assert pk.order_of_runs(kh.MIXED) == [[0], [1, 2], [1, 2], [1, 2], [3]]
    empty = build_model_spec(ModelConfig.from_dict({**kh.ODD, "loop": {"start": 2, "stop": 2, "times": 5}}))
    assert [e.layer for e in empty.schedule] == [0, 1, 2, 3] and empty.layers[4].block.kind == "stream_mix"    # its tensor is still read


def test_what_the_runs_ask_of_the_cache():
    spec = build_model_spec(ModelConfig.from_dict(kh.MIXED))
    parts = build_parts(spec)
    needs = [getattr(parts.blocks[e.layer], "mixer", None) for e in spec.schedule]
    needs = [m.cache_need() if m is not None else None for m in needs]
    assert needs[0] == CacheNeed("window", 3, 32, 40, 3) and needs[1] is None and needs[2] is None
    assert needs[3] == CacheNeed("all", 1, 48, None, 0, True)                      # ceil16(40 + 8), values inside the key rows
    groups, where = plan_groups(needs, [None] * len(needs))
    assert len(groups) == 3 and where[3] != where[6] and where[3][0] == where[6][0]   # every walk has an entry of its own
    states = [getattr(parts.blocks[e.layer], "mixer", None) for e in spec.schedule]
    assert [s.state_spec().shape if s is not None and s.state_spec() else None for s in states][2] == (3 * 24 * 40,)
    names = {t.name for p in parts.all_parts() for t in p.all_tensors()}
    assert {"embed", "head", "final.norm", "loop.in", "l0.norm1", "l0.ls1", "l0.ls2", "l2.ls1", "l1.mix.a2.b", "l1.mlp.e4.down",
            "l1.mlp.router.b", "l2.mix.dkv.norm", "l2.mix.uk"} <= names and "l2.ls2" not in names


def test_a_window_that_keeps_first_tokens_keeps_their_pages():
    need = CacheNeed("window", 1, 16, window=70, keep_first=65)
    book = SlotBook(plan_groups([need], [None])[0], max_tokens=1024, max_seqs=4)
    s = book.acquire()
    book.reserve(s, 400)
    book.commit(s, 400)
    pages = book.page_lists[s][0]
    assert pages[0] >= 0 and pages[1] >= 0 and pages[2:5] == [-1, -1, -1] and all(p >= 0 for p in pages[5:])
    for _ in range(200):
        book.reserve(s, 1)
        book.commit(s, 1)
    pages = book.page_lists[s][0]
    assert pages[0] >= 0 and pages[1] >= 0 and all(p == -1 for p in pages[2:8]) and pages[8] >= 0
    book.check()
    book.release(s)
    book.check()
    assert book.pages[0].n_held == 0


def test_linear_and_yarn_stretching_of_the_rotation():
    f, m = stretched_frequencies(16, 5000.0, {"factor": 4.0})
    want, _ = pk.frequencies({"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0}})
    assert m == 1.0 and torch.allclose(torch.from_numpy(f).double(), want, rtol=1e-6)
    assert torch.allclose(want * 4.0, pk.frequencies({"dims": 16, "base": 5000.0})[0])
    f, m = stretched_frequencies(8, 3000.0, kh.YARN)
    want, wm = pk.frequencies({"dims": 8, "base": 3000.0, "scaling": kh.YARN})
    assert abs(m - wm) < 1e-12 and torch.allclose(torch.from_numpy(f).double(), want, rtol=1e-6)


def test_plain_mask_and_routing():
    m = pk.visible(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4 and m[3].tolist() == [True] * 4 + [False] * 8
    assert pk.visible(5).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()
    g = torch.Generator().manual_seed(0)
    h = torch.randn(9, 6, generator=g, dtype=torch.float64)
    w = {"r.router": torch.randn(5, 6, generator=g, dtype=torch.float64), "r.router.b": torch.randn(5, generator=g, dtype=torch.float64)}
    idx, wt = pk.route(h, w, "r.", 2)
    z = h @ w["r.router"].t() + w["r.router.b"]
    assert torch.equal(idx[:, 0], z.argmax(dim=-1)) and torch.allclose(wt.sum(dim=-1), torch.ones(9, dtype=torch.float64))
    assert torch.allclose(wt[:, 0] / wt[:, 1], torch.exp(z.gather(1, idx)[:, 0] - z.gather(1, idx)[:, 1]))


def test_plain_latent_attention_equals_attention_on_the_cached_rows():
    """The form the engine computes (key expansion on the query's side, value expansion behind the sum) against the plain
    form (keys and values expanded per head)."""
    g = torch.Generator().manual_seed(1)
    T, H, d, r, dv, rank, width = 11, 3, 6, 4, 5, 7, 10
    m = {"heads": H, "dim": d, "rot_dim": r, "vdim": dv, "kv_rank": rank, "scale": 0.3, "rot": {"dims": r, "base": 100.0}}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"q": rnd(H * (d + r), width), "dkv": rnd(rank + r, width), "dkv.norm": rnd(rank), "uk": rnd(H * d, rank),
         "uv": rnd(H * dv, rank), "o": rnd(width, H * dv)}
    h = rnd(T, width)
    pos = torch.arange(T)
    want = pk.latent_attention(h, w, "", m, 1e-5, pos)
    q = (h @ w["q"].t()).view(T, H, d + r)
    down = h @ w["dkv"].t()
    c = pk.norm_plain(down[:, :rank], w["dkv.norm"], 1e-5)
    rows = torch.cat([c, pk.rotate(down[:, None, rank:], pos, m["rot"])[:, 0]], dim=-1)                     # what is cached
    q2 = torch.cat([torch.einsum("thd,hdr->thr", q[..., :d], w["uk"].view(H, d, rank)), pk.rotate(q[..., d:], pos, m["rot"])], dim=-1)
    o = pk.softmax_attention(q2, rows[:, None, :], c[:, None, :], 0.3, pk.visible(T))                          # one shared head
    got = torch.einsum("thr,hvr->thv", o, w["uv"].view(H, dv, rank)).reshape(T, H * dv) @ w["o"].t()
    assert torch.allclose(got, want, atol=1e-10)
