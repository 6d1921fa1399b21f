"""Kebesun through the engine against the plain implementation: each mechanism alone, whole models, whole prompts
against token-by-token decoding, portions down to two tokens, unequal batches against each request alone, slots and
pages that are used again, keys far back, at page borders and just inside and outside the window and the kept first
tokens, long decoding, greedy generation through `LLM.generate`; and the new kernels on their own against plain torch."""
import os

import pytest
import torch

import helpers
import kebesun_helpers as kh
import plain_kebesun as pk
from helpers import random_tokens
from kebesun_helpers import check, folder_of, oracle_logits
from mini_llama_cpp_release_b200 import kernels
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.engine.batch import SequenceChunk
from test_mepolix_gpu import run_in_portions, step_of

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def vocab_of(name):
    return kh.CONFIGS[name]["vocab"]


# ------------------------------------------------------------------ whole prompts

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, n", [("attention", 150), ("gla", 70), ("latent", 70), ("big_latent", 90), ("moe", 70), ("looped", 70),
                                     ("mixed", 150), ("wide", 200), ("odd", 90)])
def test_whole_prompt_against_plain(name, n, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    tokens = random_tokens(n, vocab_of(name), 11)
    check(run_in_portions(ctx, tokens, [n]), oracle_logits(folder, tokens), dtype, f"{name} whole prompt", many=n > 100)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(dtype):
    for name in ("mixed", "wide", "odd"):
        folder = folder_of(name)
        ctx = helpers.engine(folder, dtype).context
        for n in (1, 2, 3, 5):
            tokens = random_tokens(n, vocab_of(name), 20 + n)
            check(run_in_portions(ctx, tokens, [n]), oracle_logits(folder, tokens), dtype, f"{name} first {n}")
            check(run_in_portions(ctx, tokens, list(range(1, n + 1))), oracle_logits(folder, tokens), dtype, f"{name} first {n}, one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide", "odd"])
def test_token_by_token_decoding_equals_the_whole_prompt(name, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    n = 100
    tokens = random_tokens(n, vocab_of(name), 31)
    want = oracle_logits(folder, tokens)
    check(run_in_portions(ctx, tokens, [20] + list(range(21, n + 1))), want, dtype, f"{name} decoded", many=True)
    if dtype == "float32":
        whole = run_in_portions(ctx, tokens, [n])
        stepped = run_in_portions(ctx, tokens, list(range(1, n + 1)))
        check(stepped, whole, dtype, f"{name} stepped against whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_portions_of_several_sizes_down_to_two_tokens(name, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    n = 140
    tokens = random_tokens(n, vocab_of(name), 41)
    want = oracle_logits(folder, tokens)
    for cuts in ([2, 4, 7, 64, 65, 66, 128, 130, n], [63, 64, 129, n], [1, 3, 100, n]):
        check(run_in_portions(ctx, tokens, cuts), want, dtype, f"{name} portions {cuts}", many=True)
    ctx.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_far_back_and_at_page_borders_in_prompts_and_in_decoding(dtype):
    """A prompt over eleven pages, then short portions (few rows against many keys), then single tokens, every token
    against the plain implementation.  The decays are slow, so the state still holds the first tokens at the end; the
    windows have long left the first pages, which were given back but for the pages of the kept first tokens."""
    for name in ("mixed", "wide"):
        folder = folder_of(name)
        ctx = helpers.engine(folder, dtype).context
        n = 730
        tokens = random_tokens(n, vocab_of(name), 51)
        want = oracle_logits(folder, tokens)
        cuts = [640, 641, 660, 704, 705] + list(range(706, n + 1))
        check(run_in_portions(ctx, tokens, cuts), want, dtype, f"{name} long", many=True)
        ctx.cache.check()


@pytest.mark.parametrize("name", ["attention", "latent", "mixed"])
def test_single_keys_decide_the_logits(name):
    """The query matrices are six times larger, so the softmax of most rows is a choice of one or two keys, wherever among
    the visible ones they lie: a far key among hundreds, the window's oldest key, a kept first token.  A kernel that lost
    one of them, or saw the key just outside the window or just behind the kept ones, would miss whole rows."""
    folder = folder_of(name, seed=5, peaked=6.0)
    n = 400
    tokens = random_tokens(n, vocab_of(name), 61)
    cfg, w = kh.oracle(folder)
    want = pk.forward(cfg, w, tokens).float()
    if name == "attention":
        # the plain attention is as peaked as claimed, and its favourite keys include the edges
        m = cfg["layers"][0]["mixer"]
        h = pk.norm_one_plus(w["embed"][torch.as_tensor(tokens)], w["l0.norm1"], cfg["norm"]["eps"])
        pos = torch.arange(n)
        q = pk.rotate((h @ w["l0.mix.q"].t()).view(n, m["heads"], m["dim"]), pos, m["rot"])
        k = pk.rotate((h @ w["l0.mix.k"].t()).view(n, m["kv_heads"], m["dim"]), pos, m["rot"])
        size, keep = m["mask"]["size"], m["mask"]["keep_first"]
        best = []
        for head in range(m["heads"]):
            s = (q[:, head] @ k[:, head // (m["heads"] // m["kv_heads"])].t()) * m["scale"]
            p = torch.softmax(s.masked_fill(~pk.visible(n, size, keep), float("-inf")), dim=-1)
            best.append(torch.stack([p.max(dim=-1).values, p.argmax(dim=-1).double()]))
        best = torch.stack(best)                                  # [heads, 2, n]
        assert float((best[:, 0, 100:] > 0.5).double().mean()) > 0.4
        dist = pos[None, 100:] - best[:, 1, 100:].long()
        assert int((dist == size - 1).sum()) > 0 and int((best[:, 1, 100:] < keep).sum()) > 0
    # through the eight layer runs of the mixed model the sharp softmaxes multiply the 16-bit engine's rounding beyond what
    # a comparison can bound; the one-layer models run in both types
    for dtype in (DTYPES if name != "mixed" else ["float32"]):
        ctx = helpers.engine(folder, dtype).context
        check(run_in_portions(ctx, tokens, [n]), want, dtype, f"{name} peaked, whole", many=True)
        check(run_in_portions(ctx, tokens, [300] + list(range(301, n + 1))), want, dtype, f"{name} peaked, decoded", many=True)


# ------------------------------------------------------------------ batches, slots, pages

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    lens = [1, 66, 130, 17, 2]
    prompts = [random_tokens(n + 6, vocab_of(name), 70 + i) for i, n in enumerate(lens)]
    slots = [ctx.acquire() for _ in prompts]
    got = [[] for _ in prompts]
    logits = ctx.forward_batch(MiniBatch([SequenceChunk(s, p[:n], list(range(n))) for s, p, n in zip(slots, prompts, lens)]))
    row = 0
    for i, n in enumerate(lens):
        got[i].append(logits[row:row + n].float().cpu())
        row += n
    live = list(range(len(prompts)))
    for step in range(6):                               # the shorter-lived requests leave one by one
        live = [i for i in live if step < 6 - i or i == 0]
        logits = ctx.forward_batch(MiniBatch.decode([slots[i] for i in live], [prompts[i][lens[i] + step] for i in live]))
        for r, i in enumerate(live):
            got[i].append(logits[r:r + 1].float().cpu())
    for s in slots:
        ctx.release(s)
    for i, p in enumerate(prompts):
        mine = torch.cat(got[i])
        check(mine, oracle_logits(folder, p)[:mine.shape[0]], dtype, f"{name} request {i} in a batch", many=mine.shape[0] > 32)
        if dtype == "float32":
            alone = run_in_portions(ctx, p[:mine.shape[0]], [lens[i]] + list(range(lens[i] + 1, mine.shape[0] + 1)))
            check(mine, alone, dtype, f"{name} request {i}: batch against alone")
    ctx.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_that_are_used_again_start_from_nothing(dtype):
    folder = folder_of("mixed")
    ctx = helpers.engine(folder, dtype).context
    a = random_tokens(200, vocab_of("mixed"), 81)
    b = random_tokens(90, vocab_of("mixed"), 82)
    s = ctx.acquire()
    ctx.forward_batch(MiniBatch.from_tokens(s, a))
    ctx.release(s)
    s2 = ctx.acquire()
    assert s2 == s                                       # the slot, its pages and its state rows are the ones a used
    got = ctx.forward_batch(MiniBatch([SequenceChunk(s2, b[:60], list(range(60)))])).float().cpu()
    rest = torch.cat([ctx.forward_batch(MiniBatch.single(s2, t)).float().cpu() for t in b[60:]])
    ctx.release(s2)
    check(torch.cat([got, rest]), oracle_logits(folder, b), dtype, "a slot used again")


def test_the_window_gives_pages_back_but_for_the_kept_first_tokens():
    folder = folder_of("wide")
    ctx = helpers.engine(folder, "float32").context
    cache = ctx.cache
    g = next(i for i, layout in enumerate(cache.groups) if layout.need.kind == "window")
    need = cache.groups[g].need
    assert (need.window, need.keep_first) == (70, 65)
    s = ctx.acquire()
    ctx.forward_batch(MiniBatch.from_tokens(s, random_tokens(400, vocab_of("wide"), 83)))
    pages = cache.page_lists[s][g]
    # 65 kept tokens: pages 0 and 1 stay; the window of 70 before position 400 starts in page 5
    assert pages[0] >= 0 and pages[1] >= 0 and pages[2:5] == [-1, -1, -1] and all(p >= 0 for p in pages[5:])
    ctx.release(s)
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_larger_than_a_step_is_cut_and_changes_nothing(dtype):
    import mini_llama_cpp_release_b200 as ml
    folder = folder_of("mixed")
    llm = ml.load(folder, dtype=dtype, max_tokens=1024, max_batch_tokens=50)
    prompts = [random_tokens(n, vocab_of("mixed"), 90 + n) for n in (70, 45, 120)]
    slots = [llm.context.acquire() for _ in prompts]
    logits = llm.context.forward_batch(MiniBatch([SequenceChunk(s, p, [0, len(p) // 2, len(p) - 1]) for s, p in zip(slots, prompts)]))
    for i, p in enumerate(prompts):
        want = oracle_logits(folder, p)[[0, len(p) // 2, len(p) - 1]]
        check(logits[3 * i:3 * i + 3].float().cpu(), want, dtype, f"cut batch, request {i}")


# ------------------------------------------------------------------ generation

def confident_greedy(folder, prompt, n, margin=2e-4):
    cfg, w = kh.oracle(folder)
    ids, sure = list(prompt), 0
    undecided = False
    for _ in range(n):
        row = pk.forward(cfg, w, ids)[-1]
        top = torch.topk(row, 2).values
        if not undecided and float(top[0] - top[1]) > margin:
            sure += 1
        else:
            undecided = True
        ids.append(int(torch.argmax(row)))
    return ids[len(prompt):], sure


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_greedy_generation_through_generate_matches_plain(name):
    folder = folder_of(name)
    llm = helpers.engine(folder, "float32")
    prompts = [random_tokens(n, vocab_of(name), 100 + n) for n in (5, 1, 33, 70)]
    out = llm.generate(prompts, n_predict=24, stop_token_ids=[])
    total = 0
    for p, got in zip(prompts, out):
        want, sure = confident_greedy(folder, p, 24)
        assert len(got) == 24 and got[:sure] == want[:sure], (got, want, sure)
        total += sure
    assert total >= 48, total
    llm.context.cache.check()
    assert llm.context.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_the_captured_step(dtype):
    """150 generated tokens (the decode runner's graph; state carried by the graph's kernels from replay to replay; a page
    border crossed twice; the window of 40 passes over decoded tokens), each step's logits against the plain
    implementation run on the ids the engine chose."""
    folder = folder_of("mixed")
    llm = helpers.engine(folder, dtype)
    prompts = [random_tokens(50, vocab_of("mixed"), 121), random_tokens(3, vocab_of("mixed"), 122)]
    seen = []
    out = llm.generate(prompts, n_predict=150, stop_token_ids=[],
                       on_step=lambda live, chosen, logits: seen.append((list(live), logits.float().cpu().clone())))
    assert llm.context.use_graphs
    refs = [oracle_logits(folder, p + o) for p, o in zip(prompts, out)]
    for i in range(len(prompts)):
        got = torch.stack([logits[live.index(i)] for live, logits in seen if i in live])
        assert got.shape[0] == 150
        check(got, refs[i][len(prompts[i]) - 1:len(prompts[i]) - 1 + 150], dtype, f"generated tokens of request {i}", many=True)


# ------------------------------------------------------------------ the kernels on their own

@pytest.mark.parametrize("n, E, top", [(50, 5, 2), (1, 4, 4), (300, 33, 1), (17, 200, 7)])
def test_routing_plan_products_and_sum_against_plain_torch(n, E, top):
    g = torch.Generator().manual_seed(n + E)
    K, N, tile = 40, 24, 64
    logits = torch.randn(n, E, generator=g).cuda()
    bias = torch.randn(E, generator=g).cuda()
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
    kernels.moe_route(logits, bias, top, ids, wts)
    val, idx = torch.topk(logits + bias, top, dim=-1)
    assert torch.equal(ids.long(), idx)
    assert torch.allclose(wts, torch.softmax(val, dim=-1), atol=1e-6)
    # the same with the logits formed inside the kernel from the branch's input and the router's matrix
    for dtype in (torch.float32, torch.bfloat16):
        hx = torch.randn(n, 70, generator=g).to(dtype).cuda()
        router = torch.randn(E, 70, generator=g).cuda()
        ids2, wts2 = torch.empty_like(ids), torch.empty_like(wts)
        kernels.moe_route(hx, bias, top, ids2, wts2, router=router)
        val2, idx2 = torch.topk(hx.double() @ router.double().t() + bias.double(), top, dim=-1)
        sure = (val2[:, -1] - torch.topk(hx.double() @ router.double().t() + bias.double(), min(E, top + 1), dim=-1).values[:, -1]).abs() > 1e-3
        sure &= (val2[:, :-1] - val2[:, 1:]).min(dim=-1).values > 1e-3 if top > 1 else True
        if top == E:
            sure = torch.ones(n, dtype=torch.bool, device="cuda") & ((val2[:, :-1] - val2[:, 1:]).min(dim=-1).values > 1e-3 if top > 1 else True)
        assert torch.equal(ids2.long()[sure], idx2[sure])
        assert torch.allclose(wts2[sure].double(), torch.softmax(val2, dim=-1)[sure], atol=1e-4)
    rows = kernels.moe_plan_rows(n * top, E, tile)
    row_of = torch.empty(n, top, dtype=torch.int32, device="cuda")
    src = torch.empty(rows, dtype=torch.int32, device="cuda")
    tile_e = torch.empty(rows // tile, dtype=torch.int32, device="cuda")
    kernels.moe_plan(ids, E, tile, row_of, src, tile_e)
    r, s_, te = row_of.cpu(), src.cpu(), tile_e.cpu()
    assert sorted(r.flatten().tolist()) == sorted(i for i in range(rows) if s_[i] >= 0)      # every pair a row of its own
    for t in range(n):
        for j in range(top):
            assert s_[r[t, j]] == t and te[r[t, j] // tile] == ids[t, j]
    x = torch.randn(n, K, generator=g).cuda()
    w = torch.randn(E, N, K, generator=g).cuda()
    y = torch.zeros(rows, N, device="cuda")
    kernels.grouped_linear(x, src, w, tile_e, tile, y)
    for t in range(0, n, max(1, n // 7)):
        for j in range(top):
            want = w[ids[t, j]] @ x[t]
            assert torch.allclose(y[r[t, j]], want, atol=1e-4, rtol=1e-4)
    out = torch.empty(n, N, device="cuda")
    kernels.moe_combine(y, row_of, wts, out)
    want = torch.einsum("tj,tjn->tn", wts, torch.einsum("tjnk,tk->tjn", w[ids.long()], x))
    assert torch.allclose(out, want, atol=1e-4, rtol=1e-4)
    # the same sum made inside the addition of a block's two branches
    stream = torch.randn(n, N, generator=g).cuda()
    branch = torch.randn(2, n, N, generator=g).cuda()
    s1, s2 = torch.randn(N, generator=g).cuda(), torch.randn(N, generator=g).cuda()
    expect = stream + s1 * branch.sum(0) + s2 * want
    kernels.scaled_add_experts(stream, branch, s1, y, row_of, wts, s2)
    assert torch.allclose(stream, expect, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("H, dim, vdim, tau", [(3, 24, 40, 8.0), (2, 128, 64, 16.0), (1, 200, 36, 1.0), (5, 8, 8, 2.0), (2, 64, 100, 3.0)])
def test_gated_linear_attention_kernel_against_a_loop(H, dim, vdim, tau):
    g = torch.Generator().manual_seed(H * dim)
    lens, slots = [37, 1, 16, 70], [2, 0, 5, 3]
    n = sum(lens)
    width = 2 * H * dim + H * vdim + 5
    proj = torch.randn(n, width, generator=g).cuda()
    z = (torch.randn(n, H * dim, generator=g) * 2).cuda()
    zb = (torch.randn(H * dim, generator=g) + 2.0).cuda()
    state = torch.randn(6, H * vdim * dim, generator=g).cuda() * 0.1
    before = state.clone()
    parts = torch.empty(kernels.gla_slices(len(lens), H, dim, vdim, proj.device), n, H * vdim, device="cuda")
    q_col, k_col, v_col = 3, 3 + H * dim, 3 + 2 * H * dim
    z64 = (z + zb).double().cpu()
    kernels.gla(proj, q_col, k_col, v_col, z, zb, tau, state, step_of(lens, slots), H, dim, vdim, parts)      # z becomes the decays
    assert parts.shape[0] > 1 or dim <= 16                    # few blocks: the rows of the state are shared out
    out = parts.sum(dim=0)
    p64 = proj.double().cpu()
    alpha = torch.exp(torch.nn.functional.logsigmoid(z64) / tau).view(n, H, dim)
    assert torch.allclose(z.double().cpu().view(n, H, dim), alpha, atol=1e-6)
    q = p64[:, q_col:q_col + H * dim].view(n, H, dim) * dim ** -0.5
    k = p64[:, k_col:k_col + H * dim].view(n, H, dim)
    v = p64[:, v_col:v_col + H * vdim].view(n, H, vdim)
    t0 = 0
    for L, slot in zip(lens, slots):
        S = before[slot].double().cpu().view(H, vdim, dim).transpose(1, 2).clone()          # the kernel keeps [head][column][row]
        for t in range(t0, t0 + L):
            S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            want = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
            assert torch.allclose(out[t].double().cpu(), want, atol=2e-4, rtol=2e-4)
        assert torch.allclose(state[slot].double().cpu().view(H, vdim, dim).transpose(1, 2), S, atol=2e-4, rtol=2e-4)
        t0 += L
    assert torch.equal(state[1], before[1]) and torch.equal(state[4], before[4])                # slots of no sequence are untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_head_product_in_both_layouts(dtype):
    g = torch.Generator().manual_seed(3)
    n, H, n_in, n_out = 70, 3, 24, 40
    src = torch.randn(n, H * (n_in + 5), generator=g).cuda()                     # heads of n_in + 5 entries; the first n_in are read
    w = (torch.randn(H * n_in, n_out, generator=g) * 0.3).to(dtype).cuda()       # [head][in][out]
    out = torch.zeros(n, H, 64, dtype=dtype, device="cuda")                      # written into the first n_out of 64
    kernels.head_project(src, (src.stride(0), n_in + 5), w, (n_in * n_out, n_out, 1), out, (H * 64, 64), n, H, n_in, n_out)
    want = torch.einsum("thd,hdj->thj", src.view(n, H, n_in + 5)[:, :, :n_in].double(), w.view(H, n_in, n_out).double())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out[:, :, :n_out].double(), want, atol=tol, rtol=tol) and float(out[:, :, n_out:].abs().max()) == 0.0
    w2 = (torch.randn(H * n_out, n_in, generator=g) * 0.3).to(dtype).cuda()      # [head][out][in]
    out2 = torch.empty(n, H * n_out, dtype=torch.float32, device="cuda")
    kernels.head_project(src, (src.stride(0), n_in + 5), w2, (n_out * n_in, 1, n_in), out2, (H * n_out, n_out), n, H, n_in, n_out)
    want2 = torch.einsum("thd,hjd->thj", src.view(n, H, n_in + 5)[:, :, :n_in].double(), w2.view(H, n_out, n_in).double())
    assert torch.allclose(out2.view(n, H, n_out).double(), want2, atol=1e-4, rtol=1e-4)


def test_scaled_addition_of_two_branches():
    g = torch.Generator().manual_seed(4)
    n, d = 37, 100
    x = torch.randn(n, d, generator=g).cuda()
    y1, y2 = torch.randn(3, n, d, generator=g).cuda(), torch.randn(n, d, generator=g).cuda()
    s1, s2 = torch.randn(d, generator=g).cuda(), torch.randn(d, generator=g).cuda()
    want = x + s1 * y1.sum(0) + s2 * y2
    kernels.scaled_add(x, y1, s1, y2, s2)
    assert torch.allclose(x, want, atol=1e-5)
    want = x + y2
    kernels.scaled_add(x, y2, None)
    assert torch.allclose(x, want, atol=1e-6)


def windowed_case(impl, lens, q_lens, H, KV, hd, window, keep, dtype=torch.bfloat16, n_splits=1, row_tiles=4, in_cluster=False,
                  seed=0):
    """Sequences of `lens` cached tokens of which the last `q_lens` are the step's, through one attention kernel with a
    window that keeps `keep` first keys, against the plain masked softmax.  Queries are long, so single keys decide rows."""
    import math
    from test_kernels_gpu import make_paged
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(n, KV, hd, generator=g).to(dtype).float() for n in lens]
    vs = [torch.randn(n, KV, hd, generator=g).to(dtype).float() for n in lens]
    qs = [(torch.randn(n, H, hd, generator=g) * 3.0).to(dtype).float() for n in lens]
    kv = make_paged(ks, vs, dtype, seed=seed)
    q = torch.cat([qq[n - m:] for qq, n, m in zip(qs, lens, q_lens)]).to(dtype).cuda()
    N = q.shape[0]
    out = torch.empty_like(q)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    start = torch.tensor([n - m for n, m in zip(lens, q_lens)], dtype=torch.int32, device="cuda")
    part_ml = torch.empty(N * H * n_splits * 2, device="cuda") if n_splits > 1 and not in_cluster else None
    part_o = torch.empty(N * H * n_splits * hd, device="cuda") if n_splits > 1 and not in_cluster else None
    scale = 1.0 / math.sqrt(hd)
    args = (q.view(N, H * hd), out.view(N, H * hd), cu, start, len(lens), max(q_lens), H, kv, scale, window)
    if impl == "tcgen05":
        kernels.attention_tcgen05(*args, keep_first=keep)
        torch.cuda.synchronize()
        kernels.check_gemm_status(q.device)
    elif impl == "mma":
        kernels.attention_mma(*args, row_tiles, n_splits, part_ml, part_o, keep_first=keep)
    else:
        kernels.attention_simt(*args, n_splits, part_ml, part_o, keep_first=keep)
    want = torch.cat([pk.softmax_attention(qq.double(), k.double(), v.double(), scale, pk.visible(n, window, keep))[n - m:]
                      for qq, k, v, n, m in zip(qs, ks, vs, lens, q_lens)]).float()
    got = out.float().cpu().view(N, H, hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) <= tol * float(want.abs().max()), (impl, window, keep, float((got - want).abs().max()))


@pytest.mark.parametrize("window, keep", [(70, 4), (70, 65), (5, 9), (1, 0), (64, 64), (200, 130), (33, 1)])
def test_every_attention_kernel_keeps_the_first_keys_beside_the_window(window, keep):
    lens = [300, 70, 5, 131]
    for dtype in (torch.float32, torch.bfloat16):
        windowed_case("simt", lens, lens, 4, 2, 32, window, keep, dtype)                                   # whole prompts
        windowed_case("simt", [400, 129, 66], [1, 1, 1], 4, 2, 32, window, keep, dtype, n_splits=3, seed=1)    # single tokens, keys shared out
        windowed_case("simt", [400, 200], [37, 120], 6, 1, 24, window, keep, dtype, seed=2)                 # a portion behind a prefix
    for hd in (64, 128, 48):
        for row_tiles in (4, 2, 1):
            windowed_case("mma", lens, lens, 4, 2, hd, window, keep, row_tiles=row_tiles, seed=3)
        windowed_case("mma", [400, 200], [37, 120], 8, 2, hd, window, keep, n_splits=2, seed=4)
        windowed_case("mma", [400, 129, 66, 700], [1, 1, 1, 1], 4, 2, hd, window, keep, row_tiles=1, seed=5)                    # the decode form
        windowed_case("mma", [400, 129, 66, 700], [1, 1, 1, 1], 4, 2, hd, window, keep, row_tiles=1, n_splits=2, in_cluster=True, seed=6)
        windowed_case("mma", [900, 129], [1, 1], 4, 2, hd, window, keep, row_tiles=1, n_splits=4, seed=7)    # partial results merged by a second kernel
    for hd in (64, 128):
        windowed_case("tcgen05", lens, lens, 4, 2, hd, window, keep, seed=8)
        windowed_case("tcgen05", [400, 200], [37, 120], 8, 1, hd, window, keep, seed=9)


@pytest.mark.parametrize("n, E, top, K, inter", [(300, 5, 2, 96, 48), (1, 4, 4, 64, 8), (2048, 8, 2, 256, 320), (7, 33, 1, 128, 136)])
def test_the_grouped_tensor_core_product_against_plain_torch(n, E, top, K, inter):
    """Rows sorted by expert in runs padded to 128, gate/up with SiLU·mul in the epilogue, then down: against float64."""
    g = torch.Generator().manual_seed(n + E)
    tile = kernels.GROUPED_TILE
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).int().cuda()
    rows = kernels.moe_plan_rows(n * top, E, tile)
    row_of = torch.empty(n, top, dtype=torch.int32, device="cuda")
    src = torch.empty(rows, dtype=torch.int32, device="cuda")
    tile_e = torch.empty(rows // tile, dtype=torch.int32, device="cuda")
    kernels.moe_plan(ids, E, tile, row_of, src, tile_e)
    x = torch.randn(n, K, generator=g).bfloat16().cuda()
    gate = (torch.randn(E, inter, K, generator=g) * 0.2).bfloat16().cuda()
    up = (torch.randn(E, inter, K, generator=g) * 0.2).bfloat16().cuda()
    down = (torch.randn(E, K, inter, generator=g) * 0.2).bfloat16().cuda()
    gate_up = torch.stack([gate, up], dim=2).reshape(E, 2 * inter, K).contiguous()
    xs = torch.empty(rows, K, dtype=torch.bfloat16, device="cuda")
    kernels.moe_gather(x, src, xs)
    act = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05_grouped(xs, gate_up, tile_e, act, kernels.bindings.EPI_SILU_MUL)
    y = torch.empty(rows, K, dtype=torch.float32, device="cuda")
    kernels.gemm_tcgen05_grouped(act, down, tile_e, y, kernels.bindings.EPI_STORE)
    torch.cuda.synchronize()
    kernels.check_gemm_status(x.device)
    r = row_of.long().cpu()
    for t in range(0, n, max(1, n // 9)):
        for j in range(top):
            e = int(ids[t, j])
            a = pk.silu(gate[e].double() @ x[t].double()) * (up[e].double() @ x[t].double())
            assert torch.allclose(act[r[t, j]].double(), a, atol=3e-2, rtol=3e-2)
            want = down[e].double() @ act[r[t, j]].double()
            assert torch.allclose(y[r[t, j]].double(), want, atol=1e-3, rtol=1e-3)


# ------------------------------------------------------------------ the trace replay program

@pytest.mark.parametrize("dtype", DTYPES)
def test_the_replay_program_runs_batches_that_start_together_and_decode_together(dtype, tmp_path):
    """`bin/trace_run` as a process: four requests of unequal lengths start in one step, go on one token at a time, the
    shorter ones end earlier, then a second batch takes the freed slots and pages; every wanted row against the plain
    implementation."""
    import json
    import subprocess
    import sys
    import numpy as np
    name = "mixed"
    folder = folder_of(name)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    vocab = vocab_of(name)
    reqs = {f"q{i}": random_tokens(n, vocab, 300 + i) for i, n in enumerate([1 + 6, 45 + 9, 130 + 12, 70 + 12])}
    heads = {"q0": 1, "q1": 45, "q2": 130, "q3": 70}
    records, keys, step = [], [], 0
    for batch in (["q0", "q1", "q2"], ["q3", "q0#2"]):
        ids = {b: b.split("#")[0] for b in batch}
        records.append(dict(step=step, entries=[dict(id=b, tokens=reqs[ids[b]][:heads[ids[b]]], want=[0, heads[ids[b]] - 1]) for b in batch], end=[]))
        keys.append([(ids[b], p) for b in batch for p in (0, heads[ids[b]] - 1)])
        step += 1
        live, k = list(batch), 0
        while live:
            entries, ks, ends = [], [], []
            for b in live:
                toks, pos = reqs[ids[b]], heads[ids[b]] + k
                entries.append(dict(id=b, tokens=[toks[pos]], want=[0] if pos % 2 == 0 else []))
                if pos % 2 == 0:
                    ks.append((ids[b], pos))
                if pos == len(toks) - 1:
                    ends.append(b)
            records.append(dict(step=step, entries=entries, end=ends))
            keys.append(ks)
            live = [b for b in live if b not in ends]
            step += 1
            k += 1
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out), "--max-tokens", "600"],
                       input="".join(json.dumps(r) + "\n" for r in records), capture_output=True, text=True, timeout=900, cwd=root)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(records))]
    ref = {rid: oracle_logits(folder, toks) for rid, toks in reqs.items()}
    got, want = [], []
    for i, ks in enumerate(keys):
        path = out / f"{i}.f32"
        if not ks:
            assert not path.exists()
            continue
        rows = torch.from_numpy(np.fromfile(str(path), dtype="<f4").reshape(-1, vocab).copy())
        assert rows.shape[0] == len(ks)
        got.append(rows)
        want.append(torch.stack([ref[rid][pos] for rid, pos in ks]))
    check(torch.cat(got), torch.cat(want), dtype, "replayed batches", many=True)
