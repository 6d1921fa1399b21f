"""Mepolix through the engine against the plain implementation: each mixer alone, whole models, whole prompts against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, slots and pages
that are used again, keys far back and at page borders, long decoding, greedy generation through `LLM.generate`; and
the kernels of the recurrent mixers on their own against loops in plain torch."""
import math

import pytest
import torch

import helpers
import mepolix_helpers as mh
import plain_mepolix as pm
from helpers import random_tokens
from mepolix_helpers import check, folder_of, oracle_logits
from mini_llama_cpp_release_b200 import kernels
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.engine.batch import SequenceChunk
from mini_llama_cpp_release_b200.engine.step_info import StepInfo

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def vocab_of(name):
    return mh.CONFIGS[name]["vocab"]


def run_in_portions(ctx, tokens, cuts):
    """Feed `tokens` to a fresh slot in portions ending at `cuts` (the last one at len(tokens)); logits of every token."""
    slot = ctx.acquire()
    out, lo = [], 0
    for hi in cuts:
        out.append(ctx.forward_batch(MiniBatch([SequenceChunk(slot, tokens[lo:hi], list(range(hi - lo)))])).float().cpu())
        lo = hi
    ctx.release(slot)
    return torch.cat(out)


# ------------------------------------------------------------------ whole prompts

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, n", [("delta", 70), ("parallel", 70), ("mixed", 150), ("wide", 200), ("tall", 90)])
def test_whole_prompt_against_plain(name, n, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    tokens = random_tokens(n, vocab_of(name), 11)
    check(run_in_portions(ctx, tokens, [n]), oracle_logits(folder, tokens), dtype, f"{name} whole")
    ctx.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(dtype):
    """One, two and three tokens: the convolutions read zeros before the start, the recurrences start from zero, the
    softmax of the first token holds its own key and the sink alone."""
    for name in ("mixed", "wide"):
        folder = folder_of(name)
        ctx = helpers.engine(folder, dtype).context
        for n in (1, 2, 3):
            tokens = random_tokens(n, vocab_of(name), 20 + n)
            check(run_in_portions(ctx, tokens, [n]), oracle_logits(folder, tokens), dtype, f"{name} first {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd_a", "odd_b"])
def test_sizes_that_the_fast_paths_do_not_take(name, dtype):
    """A prompt, a portion of several tokens, and single tokens, for configurations whose sizes fall outside every
    fast path (see mepolix_helpers.ODD_A, ODD_B)."""
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    n = 110
    tokens = random_tokens(n, vocab_of(name), 17)
    want = oracle_logits(folder, tokens)
    check(run_in_portions(ctx, tokens, [n]), want, dtype, f"{name} whole", many=True)
    check(run_in_portions(ctx, tokens, [70, 77] + list(range(78, n + 1))), want, dtype, f"{name} in portions", many=True)
    ctx.cache.check()


# ------------------------------------------------------------------ decoding, portions

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide", "tall"])
def test_token_by_token_decoding_equals_the_whole_prompt(name, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    n = 75
    tokens = random_tokens(n, vocab_of(name), 31)
    want = oracle_logits(folder, tokens)
    one_by_one = run_in_portions(ctx, tokens, list(range(1, n + 1)))
    check(one_by_one, want, dtype, f"{name} token by token")
    if dtype == "float32":
        whole = run_in_portions(ctx, tokens, [n])
        assert helpers.rel_err(one_by_one, whole) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_portions_of_several_sizes_down_to_two_tokens(name, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    n = 140
    tokens = random_tokens(n, vocab_of(name), 41)
    want = oracle_logits(folder, tokens)
    for cuts in ([2, 4, 7, 64, 65, 66, 128, 130, n], [63, 64, 129, n], [1, 3, 100, n]):
        check(run_in_portions(ctx, tokens, cuts), want, dtype, f"{name} portions {cuts}")
    ctx.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_far_back_and_at_page_borders_in_prompts_and_in_decoding(dtype):
    """A prompt over eleven pages, then a short portion (few rows against many keys: the keys are shared out over blocks
    and merged), then single tokens (the clusters' merge), every token against the plain implementation.  The sinks
    weigh about as much as all keys together, so a merge that forgot or doubled them would show; the decays are slow,
    so the state still holds the first tokens at the end."""
    for name in ("mixed", "wide"):
        folder = folder_of(name, sink_mean=6.0)          # exp(6) = 403: a sink weighs as much as half the keys
        ctx = helpers.engine(folder, dtype).context
        n = 730
        tokens = random_tokens(n, vocab_of(name), 51)
        want = oracle_logits(folder, tokens)
        cuts = [640, 641, 660, 704, 705] + list(range(706, n + 1))
        check(run_in_portions(ctx, tokens, cuts), want, dtype, f"{name} long", many=True)


def test_a_far_key_decides_the_logits():
    """Weights made so that single keys carry the answer: the gains of the query and key norms are four times larger
    (the matrices themselves would be normalised away), which makes the scores sixteen times larger and the softmax of
    every row a choice of one or two keys, wherever in the 400 they lie; a kernel that lost a far key, or a page's edge,
    would miss whole rows."""
    from safetensors.torch import load_file, save_file
    import os
    base = folder_of("parallel", seed=5)
    folder = base + "_far"
    if not os.path.isdir(folder):
        os.makedirs(folder)
        w = load_file(os.path.join(base, "model.safetensors"))
        w["l0.mix.left.q.norm"] = (w["l0.mix.left.q.norm"].float() * 4.0).to(torch.bfloat16)
        w["l0.mix.left.k.norm"] = (w["l0.mix.left.k.norm"].float() * 4.0).to(torch.bfloat16)
        save_file(w, os.path.join(folder, "model.safetensors"))
        with open(os.path.join(base, "config.json")) as f, open(os.path.join(folder, "config.json"), "w") as g:
            g.write(f.read())
    tokens = random_tokens(400, vocab_of("parallel"), 61)
    cfg, w = mh.oracle(folder)
    want = pm.forward(cfg, w, tokens).float()
    # the plain attention is as peaked as claimed: in most rows the largest weight is above one half
    h = w["embed"][torch.as_tensor(tokens)]
    m = cfg["layers"][0]["mixer"]["left"]
    q = pm.rotate(pm.rms_norm((h @ w["l0.mix.left.q"].t()).view(400, m["heads"], m["dim"]), w["l0.mix.left.q.norm"], 1e-5), torch.arange(400), m["rot"])
    k = pm.rotate(pm.rms_norm((h @ w["l0.mix.left.k"].t()).view(400, m["kv_heads"], m["dim"]), w["l0.mix.left.k.norm"], 1e-5), torch.arange(400), m["rot"])
    s0 = (q[:, 0] @ k[:, 0].t()) * m["scale"]
    s0 = s0.masked_fill(torch.arange(400)[:, None] < torch.arange(400)[None, :], float("-inf"))
    assert float((torch.softmax(s0, dim=-1).max(dim=-1).values[100:] > 0.5).float().mean()) > 0.5
    for dtype in DTYPES:
        ctx = helpers.engine(folder, dtype).context
        check(run_in_portions(ctx, tokens, [390] + list(range(391, 401))), want, dtype, "far key")


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
    """Greedy ids by the plain implementation, and how many of them are decided by more than `margin`."""
    cfg, w = mh.oracle(folder)
    ids, sure = list(prompt), 0
    undecided = False
    for _ in range(n):
        row = pm.forward(cfg, w, ids)[-1]
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
    """150 generated tokens (the decode runner's graph, state carried by the graph's kernels from replay to replay, a
    page border crossed twice), each step's logits against the plain implementation run on the ids the engine chose."""
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

def step_of(lens, slots, device="cuda"):
    """A step's description for sequences of `lens` new tokens in `slots` (what the kernels below read of it)."""
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    tok_seq = [b for b, n in enumerate(lens) for _ in range(n)]
    return StepInfo(n_tokens=cu[-1], n_seqs=len(lens), max_q_len=max(lens), max_kv_len=0, tokens=i32([0] * cu[-1]),
                    positions=i32([0] * cu[-1]), tok_seq=i32(tok_seq), cu_seqlens=i32(cu), start_pos=i32([0] * len(lens)),
                    slots=i32(slots), want_rows=i32([]), page_tables=[])


@pytest.mark.parametrize("taps, silu", [(4, True), (2, False), (1, True), (7, False), (11, True)])
def test_causal_convolution_carries_its_last_inputs(taps, silu):
    g = torch.Generator().manual_seed(taps)
    C, pad = 37, 5                                       # channels are a column range of wider rows
    w = torch.randn(C, taps, generator=g)
    bias, in_bias = torch.randn(C, generator=g), torch.randn(C, generator=g)
    seqs = [torch.randn(n, C, generator=g) for n in (9, 1, 14)]
    state = torch.zeros(6, (taps - 1) * C + 3, device="cuda")[:, :(taps - 1) * C]      # rows of a wider state area
    slots = [4, 0, 2]
    want = [pm.causal_conv((x + in_bias).double(), w.double(), bias.double()) for x in seqs]
    if silu:
        want = [pm.silu(y) for y in want]
    got = [[] for _ in seqs]
    for portion in ([3, 1, 2], [1, None, 1], [5, None, 11]):          # then one token each, then the rest; the middle one ends
        live = [i for i, n in enumerate(portion) if n is not None]
        lens = [portion[i] for i in live]
        rows = torch.cat([seqs[i][sum(len(t) for t in got[i]):][:portion[i]] for i in live])
        x = torch.zeros(rows.shape[0], pad + C + 2)
        x[:, pad:pad + C] = rows
        out = torch.empty(rows.shape[0], C, device="cuda")
        kernels.causal_conv(x.cuda(), pad, w.cuda(), bias.cuda(), silu, state, step_of(lens, [slots[i] for i in live]), out,
                            in_bias=in_bias.cuda())
        at = 0
        for i, n in zip(live, lens):
            got[i].append(out[at:at + n].cpu())
            at += n
    for i in range(3):
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=2e-5, rtol=1e-5), (taps, i)


@pytest.mark.parametrize("H, G, dim, vdim", [(4, 2, 16, 24), (3, 3, 40, 20), (2, 1, 128, 64), (1, 1, 200, 33), (6, 2, 64, 128)])
def test_gated_delta_rule_kernel_against_a_loop(H, G, dim, vdim):
    g = torch.Generator().manual_seed(dim)
    lens, slots = [37, 1, 18], [1, 3, 0]
    n = sum(lens)
    cols = 2 * G * dim + H * vdim
    qkv = torch.randn(n, cols, generator=g)
    gates = torch.randn(n, 2 * H + 3, generator=g)
    A_log, dt_bias = torch.randn(H, generator=g) * 0.5 - 2.0, torch.randn(H, generator=g) * 0.5
    state = torch.randn(5, H * dim * vdim, generator=g) * 0.1
    out = torch.empty(n, H * vdim, device="cuda")
    dev_state = state.cuda()
    kernels.gated_delta_rule(qkv.cuda(), 0, G * dim, 2 * G * dim, gates.cuda(), 3, 3 + H, A_log.cuda(), dt_bias.cuda(), dev_state,
                             step_of(lens, slots), H, G, dim, vdim, out)
    at = 0
    for n_b, slot in zip(lens, slots):
        rows = qkv[at:at + n_b].double()
        q = rows[:, :G * dim].view(n_b, G, dim)
        k = rows[:, G * dim:2 * G * dim].view(n_b, G, dim)
        v = rows[:, 2 * G * dim:].view(n_b, H, vdim)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(gates[at:at + n_b, 3:3 + H].double())
        decay = torch.exp(-torch.exp(A_log.double()) * torch.nn.functional.softplus(gates[at:at + n_b, 3 + H:3 + 2 * H].double() + dt_bias.double()))
        for h in range(H):
            S = state[slot].double().view(H, dim, vdim)[h].clone()
            for t in range(n_b):
                S = decay[t, h] * S
                u = beta[t, h] * (v[t, h] - S.t() @ k[t, h // (H // G)])
                S = S + torch.outer(k[t, h // (H // G)], u)
                want = S.t() @ q[t, h // (H // G)]
                assert torch.allclose(out[at + t, h * vdim:(h + 1) * vdim].cpu().double(), want, atol=1e-5, rtol=1e-4), (h, t)
            assert torch.allclose(dev_state[slot].cpu().double().view(H, dim, vdim)[h], S, atol=1e-5, rtol=1e-4)
        at += n_b
    assert torch.equal(dev_state[2].cpu(), state[2]) and torch.equal(dev_state[4].cpu(), state[4])       # other slots untouched


@pytest.mark.parametrize("W, B", [(96, 3), (64, 1), (40, 5), (200, 2)])
def test_recurrence_gates_and_scan_against_a_loop(W, B):
    g = torch.Generator().manual_seed(W)
    lens, slots = [30, 1, 170], [2, 0, 1]              # the longest run takes the kernel that scans segments side by side
    n, bw = sum(lens), W // B
    u = torch.randn(n, W, generator=g)
    wr, wi = torch.randn(B, bw, bw, generator=g) * 0.3, torch.randn(B, bw, bw, generator=g) * 0.3
    br, bi, lam = torch.randn(W, generator=g), torch.randn(W, generator=g), torch.randn(W, generator=g) - 3.0
    y, yb = torch.randn(n, W + 4, generator=g), torch.randn(W, generator=g)
    a, drive = torch.empty(n, W, device="cuda"), torch.empty(n, W, device="cuda")
    kernels.block_gates(u.cuda(), wr.cuda(), wi.cuda(), br.cuda(), bi.cuda(), lam.cuda(), 8.0, a, drive)
    ud = u.double().view(n, B, bw)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ud, wr.double()).reshape(n, W) + br.double())
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ud, wi.double()).reshape(n, W) + bi.double())
    want_a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
    want_drive = torch.sqrt(1.0 - want_a * want_a) * i * u.double()
    assert torch.allclose(a.cpu().double(), want_a - 1.0, atol=1e-9, rtol=1e-5)          # the kernel leaves a - 1
    assert torch.allclose(drive.cpu().double(), want_drive, atol=1e-6, rtol=1e-4)
    state = (torch.randn(4, W, generator=g)).cuda()
    before = state.cpu().clone()
    out = torch.empty(n, W, device="cuda")
    kernels.linear_scan(a, drive, y.cuda(), 2, yb.cuda(), state, step_of(lens, slots), 0.75, out)
    at = 0
    for n_b, slot in zip(lens, slots):
        S = before[slot].double()
        for t in range(at, at + n_b):
            S = (1.0 + a[t].cpu().double()) * S + drive[t].cpu().double()
            want = S * pm.gelu_tanh(y[t, 2:2 + W].double() + yb.double()) * 0.75
            assert torch.allclose(out[t].cpu().double(), want, atol=1e-5, rtol=1e-4)
        assert torch.allclose(state[slot].cpu().double(), S, atol=1e-5, rtol=1e-4)
        at += n_b
    assert torch.equal(state[3].cpu(), before[3])


@pytest.mark.parametrize("d", [72, 128, 1000])
def test_layer_norm_of_the_stream_and_of_a_branch(d):
    g = torch.Generator().manual_seed(d)
    x, y = torch.randn(9, d, generator=g) * 3 + 1, torch.randn(2, 9, d, generator=g) * 2 - 0.5
    w = torch.randn(d, generator=g)
    xs = x.cuda().clone()
    out = torch.empty(9, d, device="cuda", dtype=torch.bfloat16)
    kernels.layernorm(xs, y.cuda(), w.cuda(), 1e-5, out, of_branch=True)
    want = x.double() + pm.layer_norm(y.double().sum(0), w.double(), 1e-5)
    assert torch.allclose(xs.cpu().double(), want, atol=1e-5, rtol=1e-5)
    assert torch.equal(out.cpu(), xs.cpu().to(torch.bfloat16))
    xs = x.cuda().clone()
    out = torch.empty(9, d, device="cuda")
    kernels.layernorm(xs, y.cuda()[0].contiguous(), w.cuda(), 1e-5, out, of_branch=False)
    assert torch.allclose(xs.cpu(), x + y[0], atol=1e-6)
    assert torch.allclose(out.cpu().double(), pm.layer_norm((x + y[0]).double(), w.double(), 1e-5), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("W, B, n_seqs", [(96, 3, 1), (64, 1, 11), (40, 5, 8), (200, 2, 9)])
def test_one_token_form_of_gates_and_recurrence(W, B, n_seqs):
    g = torch.Generator().manual_seed(W + n_seqs)
    bw = W // B
    u = torch.randn(n_seqs, W, generator=g)
    wr, wi = torch.randn(B, bw, bw, generator=g) * 0.3, torch.randn(B, bw, bw, generator=g) * 0.3
    br, bi, lam = torch.randn(W, generator=g), torch.randn(W, generator=g), torch.randn(W, generator=g) - 3.0
    y, yb = torch.randn(n_seqs, W + 4, generator=g), torch.randn(W, generator=g)
    slots = list(range(n_seqs + 2))[::-1][:n_seqs]
    state = torch.randn(n_seqs + 2, W, generator=g)
    dev_state = state.cuda()
    out = torch.empty(n_seqs, W, device="cuda")
    kernels.gates_scan_step(u.cuda(), wr.transpose(1, 2).contiguous().cuda(), wi.transpose(1, 2).contiguous().cuda(), br.cuda(),
                            bi.cuda(), lam.cuda(), 8.0, y.cuda(), 2, yb.cuda(), dev_state, step_of([1] * n_seqs, slots), 1.25, out)
    ud = u.double().view(n_seqs, B, bw)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ud, wr.double()).reshape(n_seqs, W) + br.double())
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ud, wi.double()).reshape(n_seqs, W) + bi.double())
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
    S = a * state[slots].double() + torch.sqrt(1.0 - a * a) * i * u.double()
    assert torch.allclose(dev_state[slots].cpu().double(), S, atol=1e-5, rtol=1e-4)
    assert torch.allclose(out.cpu().double(), S * pm.gelu_tanh(y[:, 2:2 + W].double() + yb.double()) * 1.25, atol=1e-5, rtol=1e-4)
    untouched = [s for s in range(n_seqs + 2) if s not in slots]
    assert torch.equal(dev_state[untouched].cpu(), state[untouched])


def test_the_rotation_table_grows_with_the_sequence(monkeypatch):
    """The model names no largest position: the table of cosines and sines is rebuilt, twice as long, whenever a step
    reaches beyond it.  With a table that starts at 64 positions a 300-token sequence makes it grow three times, in a
    prompt, in a portion and in single-token steps; the logits stay the plain implementation's."""
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200.parts.rotary import RopePartial
    monkeypatch.setattr(RopePartial, "MIN_POSITIONS", 64)
    folder = folder_of("mixed")
    llm = ml.load(folder, dtype="float32", max_tokens=1024)
    tokens = random_tokens(300, vocab_of("mixed"), 131)
    got = run_in_portions(llm.context, tokens, [50, 120] + list(range(121, 135)) + [300])
    check(got, oracle_logits(folder, tokens), "float32", "growing table")
    rope = llm.model.parts.blocks[0].mixer.left.position
    assert rope.table.shape[0] == 512 and len(rope._old) == 3
