"""Lonulix through the engine against the plain implementation: each mechanism alone, whole models, whole prompts
against token-by-token decoding, portions down to two tokens, unequal batches against each request alone, slots and
pages that are used again, keys far back, at page borders and just inside and outside the windows, long decoding, greedy
generation through `LLM.generate`; and the new kernels on their own against plain torch."""
import math
import os

import pytest
import torch

import helpers
import lonulix_helpers as lh
import plain_lonulix as pl
from helpers import random_tokens
from lonulix_helpers import check, folder_of, oracle_logits
from mini_llama_cpp_release_b200 import kernels
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.engine.batch import SequenceChunk
from test_mepolix_gpu import run_in_portions, step_of

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def vocab_of(name):
    return lh.CONFIGS[name]["vocab"]


# ------------------------------------------------------------------ whole prompts

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, n", [("latent", 150), ("hgrn2", 70), ("moe", 70), ("dense", 70), ("big_latent", 170),
                                     ("mixed", 150), ("wide", 200), ("odd", 90)])
def test_whole_prompt_against_plain(name, n, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    tokens = random_tokens(n, vocab_of(name), 11)
    check(run_in_portions(ctx, tokens, [n]), oracle_logits(folder, tokens), dtype, f"{name} whole prompt", many=n > 100)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_stream_after_every_layer(dtype):
    """The blocks one by one: the float32 stream behind each layer against the plain implementation's."""
    from mini_llama_cpp_release_b200.parts.base import MixerMemory
    for name in ("mixed", "odd"):
        folder = folder_of(name)
        ctx = helpers.engine(folder, dtype).context
        model, cache = ctx.model, ctx.cache
        tokens = random_tokens(75, vocab_of(name), 12)
        cfg, w = lh.oracle(folder)
        want = []
        pl.forward(cfg, w, tokens, want)
        slot = ctx.acquire()
        step = ctx.describe(MiniBatch([SequenceChunk(slot, tokens, [len(tokens) - 1])]))
        x = model.parts.embedding.forward(step.tokens)
        pending = None
        for k, entry in enumerate(model.spec.schedule):
            memory = MixerMemory(kv=cache.view(k, step.page_tables), state=cache.state[k], writes_cache=True)
            x, pending = model.parts.blocks[entry.layer].forward(x, pending, step, memory)
            assert pending is None and x.dtype == torch.float32
            err = helpers.rel_err(x, want[k].float())
            assert err <= (2e-5 if dtype == "float32" else 4e-2), (name, k, err)
        ctx.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(dtype):
    """One to five tokens: the recurrence starts from zero, the softmax of the first token holds its own key alone, the
    windows are not yet full."""
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
    against the plain implementation.  The forget gates are close to one, so the state still holds the first tokens at
    the end; the windows have long left the first pages, which were given back."""
    for name in ("mixed", "wide"):
        folder = folder_of(name)
        ctx = helpers.engine(folder, dtype).context
        n = 730
        tokens = random_tokens(n, vocab_of(name), 51)
        want = oracle_logits(folder, tokens)
        cuts = [640, 641, 660, 704, 705] + list(range(706, n + 1))
        check(run_in_portions(ctx, tokens, cuts), want, dtype, f"{name} long", many=True)
        ctx.cache.check()


def test_the_state_still_holds_the_first_tokens_after_hundreds():
    """Two prompts that differ in their first token alone: with gates close to one the logits 300 tokens on still differ,
    in the plain implementation and by the same amount in the engine, whose prompts are cut at different places (a state
    that was lost at a cut, or zeroed, would make them equal)."""
    folder = folder_of("hgrn2")
    ctx = helpers.engine(folder, "float32").context
    a = random_tokens(300, vocab_of("hgrn2"), 55)
    b = [(a[0] + 1) % vocab_of("hgrn2")] + a[1:]
    want = oracle_logits(folder, a)[-1] - oracle_logits(folder, b)[-1]
    got = run_in_portions(ctx, a, [150, 299, 300])[-1] - run_in_portions(ctx, b, [7, 300])[-1]
    assert float(want.abs().max()) > 1e-3
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("name", ["latent", "big_latent", "wide"])
def test_single_keys_decide_the_logits(name):
    """The query expansions are fifteen times larger, so the softmax of most rows is a choice of one or two keys, wherever among
    the visible ones they lie: the window's oldest key as well as the newest.  A kernel that lost the oldest key, or saw the
    one just outside the window, would miss whole rows."""
    folder = folder_of(name, seed=5, peaked=15.0)
    n = 400
    tokens = random_tokens(n, vocab_of(name), 61)
    cfg, w = lh.oracle(folder)
    want = pl.forward(cfg, w, tokens).float()
    if name == "latent":
        # the plain attention is as peaked as claimed, and its favourite keys include the window's edge
        m = cfg["layers"][0]["mixer"]
        x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
        probs = []
        pl.latent_attention(x, w, "l0.mix.", m, cfg["norm"]["eps"], torch.arange(n), probs)
        best = torch.stack([torch.stack([p.max(dim=-1).values, p.argmax(dim=-1).double()]) for p in probs])   # [heads, 2, n]
        assert float((best[:, 0, 100:] > 0.5).double().mean()) > 0.4
        dist = torch.arange(n)[None, 100:] - best[:, 1, 100:].long()
        assert int((dist == m["mask"]["size"] - 1).sum()) > 0 and int(dist.max()) == m["mask"]["size"] - 1
    # through the three layers of the wide model the sharp softmaxes multiply the 16-bit engine's rounding beyond what a
    # comparison can bound; the one-layer models run in both types
    for dtype in (DTYPES if name != "wide" else ["float32"]):
        ctx = helpers.engine(folder, dtype).context
        check(run_in_portions(ctx, tokens, [n]), want, dtype, f"{name} peaked, whole", many=True)
        check(run_in_portions(ctx, tokens, [300] + list(range(301, n + 1))), want, dtype, f"{name} peaked, decoded", many=True)
        check(run_in_portions(ctx, tokens, [190, 200, 333, n]), want, dtype, f"{name} peaked, portions", many=True)


# ------------------------------------------------------------------ batches, slots, pages

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide", "odd"])
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
    mine = [torch.cat(rows) for rows in got]
    want = [oracle_logits(folder, p)[:m.shape[0]] for p, m in zip(prompts, mine)]
    if dtype == "float32":
        for i, p in enumerate(prompts):
            check(mine[i], want[i], dtype, f"{name} request {i} in a batch", many=mine[i].shape[0] > 32)
            alone = run_in_portions(ctx, p[:mine[i].shape[0]], [lens[i]] + list(range(lens[i] + 1, mine[i].shape[0] + 1)))
            check(mine[i], alone, dtype, f"{name} request {i}: batch against alone")
    else:
        # a router that sees 16-bit inputs may choose otherwise where two choice scores nearly tie; the rows of all requests
        # are held to the bound together, so that the few such rows are spared whichever request they fall into
        check(torch.cat(mine), torch.cat(want), dtype, f"{name} requests in a batch", many=True)
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


def test_the_windows_give_pages_back_as_they_move_on():
    folder = folder_of("wide")
    ctx = helpers.engine(folder, "float32").context
    cache = ctx.cache
    by_window = {layout.need.window: i for i, layout in enumerate(cache.groups) if layout.need.kind == "window"}
    assert sorted(by_window) == [64, 130]
    s = ctx.acquire()
    ctx.forward_batch(MiniBatch.from_tokens(s, random_tokens(400, vocab_of("wide"), 83)))
    # the next token, position 400, reads back to position 271 (page 4) under the window of 130 and to 337 (page 5) under 64
    wide, narrow = cache.page_lists[s][by_window[130]], cache.page_lists[s][by_window[64]]
    assert wide[:4] == [-1] * 4 and all(p >= 0 for p in wide[4:]) and narrow[:5] == [-1] * 5 and all(p >= 0 for p in narrow[5:])
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
    cfg, w = lh.oracle(folder)
    ids, sure = list(prompt), 0
    undecided = False
    for _ in range(n):
        row = pl.forward(cfg, w, ids)[-1]
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
    border crossed twice; the windows of 40 and 70 pass over decoded tokens), each step's logits against the plain
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

@pytest.mark.parametrize("n, d, groups", [(37, 96, 3), (1, 100, 5), (70, 128, 1), (9, 1024, 2), (5, 2048, 64), (3, 40, 40)])
def test_norm_in_groups_alone_and_behind_a_gated_sum(n, d, groups):
    g = torch.Generator().manual_seed(n + d)
    rnd = lambda *s: torch.randn(*s, generator=g).cuda()
    gain, eps = rnd(d), 3e-5
    wide = rnd(n, d + 7)
    x = wide[:, 3:3 + d]                                                        # rows of a wider matrix
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.empty(n, d, dtype=out_dtype, device="cuda")
        kernels.group_norm(x, groups, gain, eps, out=out)
        want = pl.group_norm(x.double().cpu(), gain.double().cpu(), groups, eps)
        assert helpers.rel_err(out, want) <= (2e-6 if out_dtype == torch.float32 else 5e-3)
    # a gain as long as one part, shared by the parts (the norm of each head of a row of heads)
    out = torch.empty(n, d, device="cuda")
    kernels.group_norm(x, groups, gain[:d // groups].contiguous(), eps, out=out)
    want = pl.group_norm(x.double().cpu(), gain[:d // groups].double().cpu().repeat(groups), groups, eps)
    assert helpers.rel_err(out, want) <= 2e-6
    # behind the sum alpha x + sigmoid(z + b) * (y1 + y2): into x itself and a 16-bit copy
    y, z, b = rnd(2, n, d), rnd(n, d + 5) * 2, rnd(d)
    for alpha, gated, biased in ((1.7, True, True), (1.0, True, False), (0.5, False, False)):
        stream = rnd(n, d)
        v = alpha * stream.double() + (torch.sigmoid(z[:, 5:].double() + (b.double() if biased else 0.0)) if gated else 1.0) * y.double().sum(0)
        want = pl.group_norm(v.cpu(), gain.double().cpu(), groups, eps)
        copy = torch.empty(n, d, dtype=torch.bfloat16, device="cuda")
        kernels.group_norm(stream, groups, gain, eps, out=copy, write_x=True, alpha=alpha, y=y, gate=z if gated else None, gate_col=5,
                           gate_bias=b if biased else None)
        assert helpers.rel_err(stream, want) <= 1e-5 and helpers.rel_err(copy, want) <= 5e-3
    # the branch as the weighted sum of a token's expert rows; a negative row is the token's own input
    top, n_rows = 3, 50
    rows, wts = rnd(n_rows, d), torch.rand(n, top, generator=g).cuda()
    row_of = torch.randint(-1, n_rows, (n, top), generator=g).int().cuda()
    for ident_dtype in (torch.float32, torch.bfloat16, None):
        ident = rnd(n, d).to(ident_dtype) if ident_dtype is not None else None
        stream = rnd(n, d)
        picked = torch.where(row_of[:, :, None] >= 0, rows[row_of.clamp_min(0).long()].double(),
                             ident.double()[:, None, :] if ident is not None else torch.zeros(n, 1, d, dtype=torch.float64, device="cuda"))
        v = 2.0 * stream.double() + torch.sigmoid(z[:, :d].double() + b.double()) * (wts.double()[:, :, None] * picked).sum(1)
        want = pl.group_norm(v.cpu(), gain.double().cpu(), groups, eps)
        kernels.group_norm(stream, groups, gain, eps, write_x=True, alpha=2.0, expert_rows=(rows, row_of, wts, ident), gate=z, gate_bias=b)
        assert helpers.rel_err(stream, want) <= 1e-5


@pytest.mark.parametrize("H, dim, vdim", [(3, 24, 40), (2, 128, 64), (1, 200, 36), (5, 8, 8), (2, 64, 100)])
def test_forget_gate_attention_kernel_against_a_loop(H, dim, vdim):
    g = torch.Generator().manual_seed(H * dim)
    lens, slots = [37, 1, 16, 70], [2, 0, 5, 3]
    n = sum(lens)
    q_col, f_col, v_col = 3, 3 + H * dim + 2, 3 + 2 * H * dim + 4              # three column ranges of wider rows
    proj = torch.randn(n, v_col + H * vdim + 5, generator=g).cuda()
    proj[:, f_col:f_col + H * dim] *= 3.0                                       # gates from nearly closed to nearly open
    bias = (torch.randn(H * dim, generator=g) + 2.0).cuda()
    lower = torch.rand(H * dim, generator=g).cuda()
    for f_bias, low in ((bias, lower), (None, None)):
        state = torch.randn(6, H * vdim * dim, generator=g).cuda() * 0.1
        before = state.clone()
        parts = torch.empty(kernels.gla_slices(len(lens), H, dim, vdim, proj.device), n, H * vdim, device="cuda")
        kernels.forget_gate_attention(proj, q_col, f_col, v_col, f_bias, low, state, step_of(lens, slots), H, dim, vdim, parts)
        out = parts.sum(dim=0)
        p64 = proj.double().cpu()
        q = pl.silu(p64[:, q_col:q_col + H * dim]).view(n, H, dim)
        zf = p64[:, f_col:f_col + H * dim] + (f_bias.double().cpu() if f_bias is not None else 0.0)
        lo = low.double().cpu() if low is not None else torch.zeros(H * dim, dtype=torch.float64)
        f = (lo + (1.0 - lo) * torch.sigmoid(zf)).view(n, H, dim)
        v = p64[:, v_col:v_col + H * vdim].view(n, H, vdim)
        t0 = 0
        for L, slot in zip(lens, slots):
            S = before[slot].double().cpu().view(H, vdim, dim).transpose(1, 2).clone()      # the kernel keeps [head][column][row]
            for t in range(t0, t0 + L):
                S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
                want = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
                assert torch.allclose(out[t].double().cpu(), want, atol=2e-4, rtol=2e-4)
            assert torch.allclose(state[slot].double().cpu().view(H, vdim, dim).transpose(1, 2), S, atol=2e-4, rtol=2e-4)
            t0 += L
        assert torch.equal(state[1], before[1]) and torch.equal(state[4], before[4])        # slots of no sequence are untouched


@pytest.mark.parametrize("n, E, top, groups, keep", [(50, 6, 2, 3, 2), (1, 4, 4, 1, 1), (300, 33, 1, 1, 1), (17, 200, 7, 8, 3),
                                                     (64, 20, 4, 4, 3), (40, 9, 9, 3, 3), (25, 12, 2, 6, 1)])
def test_routing_by_scores_against_plain_torch(n, E, top, groups, keep):
    g = torch.Generator().manual_seed(n + E)
    K = 70
    router = torch.randn(E, K, generator=g).cuda() * 0.4
    corr = (torch.randn(E, generator=g) * 0.3).cuda()
    for dtype in (torch.float32, torch.bfloat16):
        for correction in (corr, None):
            hx = torch.randn(n, K, generator=g).to(dtype).cuda()
            ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
            wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
            kernels.moe_route_scored(hx, router, correction, top, groups, keep, 1.75, ids, wts)
            s = torch.softmax(hx.double() @ router.double().t(), dim=-1)
            choice = s + (correction.double() if correction is not None else 0.0)
            sure = torch.ones(n, dtype=torch.bool, device="cuda")
            if groups > 1:
                best = choice.view(n, groups, E // groups).max(dim=-1).values
                order = torch.sort(best, dim=-1, descending=True)
                if keep < groups:
                    sure &= (order.values[:, keep - 1] - order.values[:, keep]) > 1e-5
                kept = torch.zeros(n, groups, dtype=torch.bool, device="cuda").scatter_(1, order.indices[:, :keep], True)
                choice = choice.masked_fill(~kept[:, :, None].expand(-1, -1, E // groups).reshape(n, E), float("-inf"))
            val, idx = torch.topk(choice, top, dim=-1)
            if top > 1:
                sure &= (val[:, :-1] - val[:, 1:]).min(dim=-1).values > 1e-5
            if top < E:
                sure &= (val[:, -1] - torch.topk(choice, top + 1, dim=-1).values[:, -1]) > 1e-5
            assert int(sure.sum()) >= n * 0.5
            assert torch.equal(ids.long()[sure], idx[sure])
            w = s.gather(1, idx)
            w = w / (w.sum(dim=-1, keepdim=True) + 1e-20) * 1.75
            assert torch.allclose(wts[sure].double(), w[sure], atol=1e-5, rtol=1e-4)


def test_choice_scores_below_zero_still_beat_a_closed_group():
    """Corrections far below zero on every expert of the kept groups: the chosen ones still come from there, not from the
    closed group, whose choice scores are larger."""
    E, K, n = 6, 16, 20
    g = torch.Generator().manual_seed(7)
    router = torch.randn(E, K, generator=g).cuda() * 0.1
    corr = torch.tensor([5.0, -3.0, -3.0, -3.0, 4.0, -3.0]).cuda()             # groups (0,1) and (4,5) are kept, (2,3) closed
    hx = torch.randn(n, K, generator=g).cuda()
    ids = torch.empty(n, 4, dtype=torch.int32, device="cuda")
    wts = torch.empty(n, 4, dtype=torch.float32, device="cuda")
    kernels.moe_route_scored(hx, router, corr, 4, 3, 2, 1.0, ids, wts)
    assert sorted(set(ids.flatten().tolist())) == [0, 1, 4, 5]
    assert torch.allclose(wts.sum(dim=-1), torch.ones(n, device="cuda"), atol=1e-5)


def test_identity_experts_in_the_weighted_sum():
    g = torch.Generator().manual_seed(9)
    n, d, top = 23, 40, 3
    y = torch.randn(30, d, generator=g).cuda()
    row_of = torch.randint(-1, 30, (n, top), generator=g).int().cuda()
    row_of[0] = -1                                                               # a token whose choices are all identity experts
    wts = torch.rand(n, top, generator=g).cuda()
    for dtype in (torch.float32, torch.bfloat16):
        h = torch.randn(n, d, generator=g).to(dtype).cuda()
        out = torch.empty(n, d, device="cuda")
        kernels.moe_combine(y, row_of, wts, out, ident=h)
        picked = torch.where(row_of[:, :, None] >= 0, y[row_of.clamp_min(0).long()], h.float()[:, None, :])
        assert torch.allclose(out, (wts[:, :, None] * picked).sum(1), atol=1e-5)
        assert torch.allclose(out[0], wts[0].sum() * h[0].float(), atol=1e-5)


@pytest.mark.parametrize("interleaved", [True, False])
def test_latent_rows_and_queries_with_either_pairing(interleaved):
    """The kernel that norms the latent, rotates and lays out the query rows, with the query heads read from rows of their
    own (the expansion of a query latent) and either pairing of the rotated entries."""
    g = torch.Generator().manual_seed(11)
    n, H, dim, rot, rank, D = 45, 3, 10, 6, 20, 32
    lens = [30, 15]
    positions = torch.tensor(list(range(100, 130)) + list(range(15)), dtype=torch.int32).cuda()
    tok_seq = torch.tensor([0] * 30 + [1] * 15, dtype=torch.int32).cuda()
    proj = torch.randn(n, 4 + rank + rot, generator=g).cuda()                   # [4 other columns | latent | shared rotated part]
    q_rows = torch.randn(n, 2 + H * (dim + rot), generator=g).cuda()
    gain = torch.randn(rank, generator=g).cuda()
    base = 300.0
    f = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32).cuda()
    table = kernels.rope_table(f, 256, 1.0)
    q_out = torch.full((n, H * D), 7.0, device="cuda")
    kernels.latent_prepare(proj, 2, 4, gain, 1e-5, positions, tok_seq, table, H, dim, rot, rank, q_out, None, q_rows=q_rows,
                           interleaved=interleaved)
    q = q_rows[:, 2:].double().cpu().view(n, H, dim + rot)[..., dim:]
    if interleaved:
        want = pl.rotate_neighbours(q, positions.cpu().long(), rot, base)
    else:
        a = positions.cpu().double()[:, None] * f.double().cpu()[None, :]
        c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
        u, v = q[..., :rot // 2], q[..., rot // 2:]
        want = torch.cat([u * c - v * s, v * c + u * s], dim=-1)
    got = q_out.view(n, H, D)
    assert torch.allclose(got[:, :, rank:rank + rot].double().cpu(), want, atol=1e-4)
    assert float(got[:, :, rank + rot:].abs().max()) == 0.0


def test_activations_and_the_scaled_embedding():
    g = torch.Generator().manual_seed(13)
    z = (torch.randn(1000, generator=g) * 3).cuda()
    for kind, want in (("silu", pl.silu(z.double())), ("gelu", pl.gelu_erf(z.double())),
                       ("gelu_tanh", 0.5 * z.double() * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z.double() + 0.044715 * z.double() ** 3))))):
        out = torch.empty_like(z)
        kernels.activation(z, kind, out)
        assert torch.allclose(out.double(), want, atol=1e-6)
        out16 = torch.empty(1000, dtype=torch.bfloat16, device="cuda")
        kernels.activation(z.bfloat16(), kind, out16)
        assert torch.allclose(out16.double(), want, atol=5e-2, rtol=2e-2)
    table = torch.randn(50, 24, generator=g).bfloat16().cuda()
    ids = torch.randint(0, 50, (17,), generator=g).int().cuda()
    out = torch.empty(17, 24, device="cuda")
    kernels.embed(table, ids, out, 2.5)
    assert torch.equal(out, table[ids.long()].float() * 2.5)


@pytest.mark.parametrize("n, E, top, K, inter", [(300, 5, 2, 96, 48), (1, 4, 4, 64, 16), (2048, 8, 2, 256, 320), (7, 33, 1, 128, 144)])
def test_the_grouped_tensor_core_product_with_an_activation_behind_it(n, E, top, K, inter):
    """Ungated experts: rows sorted by expert in runs padded to 128, up with the erf GELU in the epilogue, then down,
    against float64."""
    g = torch.Generator().manual_seed(n + E)
    tile = kernels.GROUPED_TILE
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).int().cuda()
    rows = kernels.moe_plan_rows(n * top, E, tile)
    row_of = torch.empty(n, top, dtype=torch.int32, device="cuda")
    src = torch.empty(rows, dtype=torch.int32, device="cuda")
    tile_e = torch.empty(rows // tile, dtype=torch.int32, device="cuda")
    kernels.moe_plan(ids, E, tile, row_of, src, tile_e)
    x = torch.randn(n, K, generator=g).bfloat16().cuda()
    up = (torch.randn(E, inter, K, generator=g) * 0.2).bfloat16().cuda()
    down = (torch.randn(E, K, inter, generator=g) * 0.2).bfloat16().cuda()
    xs = torch.empty(rows, K, dtype=torch.bfloat16, device="cuda")
    kernels.moe_gather(x, src, xs)
    for kind, fn in (("gelu", pl.gelu_erf), ("silu", pl.silu)):
        act = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
        kernels.gemm_tcgen05_grouped(xs, up, tile_e, act, kernels.bindings.EPI_ACT[kind])
        y = torch.empty(rows, K, dtype=torch.float32, device="cuda")
        kernels.gemm_tcgen05_grouped(act, down, tile_e, y, kernels.bindings.EPI_STORE)
        torch.cuda.synchronize()
        kernels.check_gemm_status(x.device)
        r = row_of.long().cpu()
        for t in range(0, n, max(1, n // 9)):
            for j in range(top):
                e = int(ids[t, j])
                a = fn(up[e].double() @ x[t].double())
                assert torch.allclose(act[r[t, j]].double(), a, atol=3e-2, rtol=3e-2)
                assert torch.allclose(y[r[t, j]].double(), down[e].double() @ act[r[t, j]].double(), atol=1e-3, rtol=1e-3)


# ------------------------------------------------------------------ the trace replay program

@pytest.mark.parametrize("dtype", DTYPES)
def test_the_replay_program_runs_batches_that_start_together_and_decode_together(dtype, tmp_path):
    """`bin/trace_run` as a process: three requests of unequal lengths start in one step, go on one token at a time, the
    shorter ones end earlier, then a second batch takes the freed slots and pages; every wanted row against the plain
    implementation."""
    import json
    import subprocess
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
