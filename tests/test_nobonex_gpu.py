"""Nobonex through the engine against the plain implementation: each mechanism alone, whole models, whole prompts against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, slots and pages that are
used again, keys far back, at page borders and just inside and outside the chunks, long decoding, greedy generation through
`LLM.generate`; and the new kernels on their own against plain torch."""
import math

import pytest
import torch

import helpers
import nobonex_helpers as nh
import plain_nobonex as pn
from helpers import random_tokens
from nobonex_helpers import check, folder_of, oracle_logits
from mini_llama_cpp_release_b200 import kernels
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.engine.batch import SequenceChunk
from test_mepolix_gpu import run_in_portions, step_of

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def vocab_of(name):
    return nh.CONFIGS[name]["vocab"]


# ------------------------------------------------------------------ whole prompts, layer by layer

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, n", [("gated", 150), ("conv", 90), ("mamba", 90), ("moe", 70), ("dense", 70), ("shared", 160),
                                     ("mixed", 150), ("wide", 200), ("odd", 90)])
def test_whole_prompt_against_plain(name, n, dtype):
    folder = folder_of(name)
    ctx = helpers.engine(folder, dtype).context
    tokens = random_tokens(n, vocab_of(name), 11)
    check(run_in_portions(ctx, tokens, [n]), oracle_logits(folder, tokens), dtype, f"{name} whole prompt", many=n > 100)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_stream_after_every_layer(dtype):
    """The blocks one by one: the float32 stream behind each layer (with the addition the block left for the next one carried
    out) against the plain implementation's."""
    from mini_llama_cpp_release_b200.parts.base import MixerMemory
    from mini_llama_cpp_release_b200.parts.block import DEFERRED, finish_deferred
    for name in ("mixed", "odd"):
        folder = folder_of(name)
        ctx = helpers.engine(folder, dtype).context
        model, cache = ctx.model, ctx.cache
        tokens = random_tokens(75, vocab_of(name), 12)
        cfg, w = nh.oracle(folder)
        want = []
        pn.forward(cfg, w, tokens, want)
        slot = ctx.acquire()
        step = ctx.describe(MiniBatch([SequenceChunk(slot, tokens, [len(tokens) - 1])]))
        x = model.parts.embedding.forward(step.tokens)
        pending = None
        for k, entry in enumerate(model.spec.schedule):
            memory = MixerMemory(kv=cache.view(k, step.page_tables), state=cache.state[k], writes_cache=entry.reads_cache_of is None)
            x, pending = model.parts.blocks[entry.layer].forward(x, pending, step, memory)
            assert pending is None and x.dtype == torch.float32 and DEFERRED in step.handover
            left = step.handover[DEFERRED]
            now = x.clone()
            type(left)(now, left.norm, left.mult, y=left.y, expert_rows=left.expert_rows).finish()     # on a copy: the next block does it itself
            if dtype == "float32":
                err = helpers.rel_err(now, want[k].float())
                assert err <= 2e-5, (name, k, err)
            else:
                # a router that sees 16-bit inputs may choose another expert for a token whose two best scores nearly tie,
                # and that token's row is then another row: a few rows are spared
                rows = sorted(helpers.rel_err(now[t], want[k][t].float()) for t in range(now.shape[0]))
                assert rows[int(0.9 * len(rows))] <= 4e-2, (name, k, rows[-8:])
        finish_deferred(step)
        ctx.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(dtype):
    """One to five tokens: the state starts from zero, the convolutions reach before the start, the softmax of the first
    token holds its own key alone."""
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
    for cuts in ([2, 4, 7, 49, 50, 51, 64, 65, 66, 128, 130, n], [63, 64, 129, n], [1, 3, 100, n]):
        check(run_in_portions(ctx, tokens, cuts), want, dtype, f"{name} portions {cuts}", many=True)
    ctx.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_far_back_and_at_page_borders_in_prompts_and_in_decoding(dtype):
    """A prompt over eleven pages, then short portions (few rows against many keys), then single tokens, every token against
    the plain implementation.  The state-space layers decay slowly, so their state still holds the first tokens at the end;
    the chunked layers have long given their first pages back."""
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
    """Two prompts that differ in their first ten tokens alone: with slow decays the logits 300 tokens on still differ, in the plain
    implementation and by the same amount in the engine, whose prompts are cut at different places (a state that was lost at
    a cut, or zeroed, would make them equal)."""
    folder = folder_of("mamba")
    ctx = helpers.engine(folder, "float32").context
    a = random_tokens(300, vocab_of("mamba"), 55)
    b = [(t + 1) % vocab_of("mamba") for t in a[:10]] + a[10:]
    want = oracle_logits(folder, a)[-1] - oracle_logits(folder, b)[-1]
    got = run_in_portions(ctx, a, [150, 299, 300])[-1] - run_in_portions(ctx, b, [7, 300])[-1]
    assert float(want.abs().max()) > 1e-3
    assert float((got - want).abs().max()) <= 5e-2 * float(want.abs().max())


@pytest.mark.parametrize("name", ["gated", "conv", "shared"])
def test_single_keys_decide_the_logits(name):
    """The query norms' gains are eight times larger, so the softmax of most rows is a choice of one or two keys, wherever
    among the visible ones they lie: the chunk's first key as well as the newest, keys hundreds of places back in the layer
    without a mask.  A kernel that lost the chunk's first key, or saw the one just before it, would miss whole rows."""
    folder = folder_of(name, seed=5, peaked=8.0)
    n = 400
    tokens = random_tokens(n, vocab_of(name), 61)
    cfg, w = nh.oracle(folder)
    want = pn.forward(cfg, w, tokens).float()
    if name == "gated":
        # the plain attention is as peaked as claimed, and its favourite keys include the chunk's first
        m = cfg["layers"][0]["mixer"]
        x = pn.tanh_norm(w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"], w, "l0.norm1")
        probs = []
        pn.gated_attention(x, w, "l0.mix.", m, cfg["norm"]["eps"], torch.arange(n), {}, 0, probs)
        best = torch.stack([p.argmax(dim=-1) for p in probs])                      # [heads, n]
        big = torch.stack([p.max(dim=-1).values for p in probs])
        assert float((big[:, 100:] > 0.5).double().mean()) > 0.3
        first_of_chunk = (torch.arange(n) // m["mask"]["size"]) * m["mask"]["size"]
        assert int((best == first_of_chunk[None, :])[:, 100:].sum()) > 0
    if name == "conv":
        m = cfg["layers"][0]["mixer"]
        x = pn.tanh_norm(w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"], w, "l0.norm1")
        probs = []
        pn.conv_attention(x, w, "l0.mix.", m, cfg["norm"]["eps"], torch.arange(n), {}, probs)
        far = torch.stack([torch.arange(n) - p.argmax(dim=-1) for p in probs])
        assert int(far.max()) > 250                                                 # some row's favourite key lies far back
    for dtype in DTYPES:
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
        # a router that sees 16-bit inputs may choose otherwise where two scores nearly tie; the rows of all requests are held
        # to the bound together, so that the few such rows are spared whichever request they fall into
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


def test_the_chunks_give_pages_back_as_the_sequence_leaves_them():
    folder = folder_of("wide")
    ctx = helpers.engine(folder, "float32").context
    cache = ctx.cache
    by_chunk = {layout.need.window: i for i, layout in enumerate(cache.groups) if layout.need.kind == "chunk"}
    assert sorted(by_chunk) == [64, 130]
    s = ctx.acquire()
    ctx.forward_batch(MiniBatch.from_tokens(s, random_tokens(400, vocab_of("wide"), 83)))
    # the next token, position 400, reads back to position 390 (page 6) under chunks of 130 and to 384 (page 6) under 64
    wide, narrow = cache.page_lists[s][by_chunk[130]], cache.page_lists[s][by_chunk[64]]
    assert wide[:6] == [-1] * 6 and all(p >= 0 for p in wide[6:]) and narrow[:6] == [-1] * 6 and all(p >= 0 for p in narrow[6:])
    ctx.release(s)
    cache.check()
    # a layer whose keys another layer reads under another mask keeps all of them
    odd = helpers.engine(folder_of("odd"), "float32").context.cache
    assert any(layout.need.kind == "all" and 0 in layout.entries for layout in odd.groups)


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
    cfg, w = nh.oracle(folder)
    ids, sure = list(prompt), 0
    undecided = False
    for _ in range(n):
        row = pn.forward(cfg, w, ids)[-1]
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
    """150 generated tokens (the decode runner's graph; state and convolution inputs carried by the graph's kernels from replay
    to replay; a page border crossed twice; chunks of 50 begin and end among the decoded tokens), each step's logits against
    the plain implementation run on the ids the engine chose."""
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

@pytest.mark.parametrize("n, d", [(37, 96), (1, 100), (70, 128), (9, 1024), (3, 41)])
def test_tanh_norm_in_all_its_uses(n, d):
    g = torch.Generator().manual_seed(n + d)
    rnd = lambda *s: torch.randn(*s, generator=g).cuda()
    T = lambda v, t: torch.tanh(t[0] * v.double()) * t[1].double() + t[2].double()
    na, nb = (0.7, rnd(d), rnd(d)), (1.9, rnd(d), rnd(d))
    x = rnd(n, d)
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.empty(n, d, dtype=out_dtype, device="cuda")
        kernels.tanh_norm(x, next_norm=na, out=out)
        assert helpers.rel_err(out, T(x, na)) <= (2e-6 if out_dtype == torch.float32 else 5e-3)
    # a branch in slices, normed and added with a factor; then the next norm of the new stream in the same kernel
    y = rnd(3, n, d)
    stream, before = x.clone(), x.double()
    out = torch.empty(n, d, dtype=torch.bfloat16, device="cuda")
    kernels.tanh_norm(stream, y=y, branch_norm=nb, mult=0.6, next_norm=na, out=out)
    want = before + 0.6 * T(y.double().sum(0), nb)
    assert helpers.rel_err(stream, want) <= 2e-6 and helpers.rel_err(out, T(want, na)) <= 5e-3
    # the branch as the plain sum of a token's expert rows (a negative row adds nothing); no next norm
    rows = rnd(50, d)
    row_of = torch.randint(-1, 50, (n, 3), generator=g).int().cuda()
    stream = x.clone()
    kernels.tanh_norm(stream, expert_rows=(rows, row_of), branch_norm=nb, mult=1.3)
    picked = torch.where(row_of[:, :, None] >= 0, rows[row_of.clamp_min(0).long()].double(), torch.zeros(1, dtype=torch.float64, device="cuda"))
    assert helpers.rel_err(stream, before + 1.3 * T(picked.sum(1), nb)) <= 2e-6
    # a plain addition (no norm on the branch)
    stream = x.clone()
    kernels.tanh_norm(stream, y=y[0].contiguous(), mult=1.0)
    assert helpers.rel_err(stream, before + y[0].double()) <= 1e-6


@pytest.mark.parametrize("kind", ["silu", "gelu_tanh", "clamped"])
def test_gated_units_against_plain_torch(kind):
    g = torch.Generator().manual_seed(3)
    n, inter = 33, 56
    gu = (torch.randn(n, 2 * inter, generator=g) * 3).cuda()
    gate, up = gu[:, :inter].double(), gu[:, inter:].double()
    want = {"silu": pn.silu(gate) * up, "gelu_tanh": pn.gelu_tanh(gate) * up,
            "clamped": (lambda a, b: a * torch.sigmoid(1.702 * a) * (b + 1))(gate.clamp(max=1.5), up.clamp(-1.5, 1.5))}[kind]
    out = torch.empty(n, inter, device="cuda")
    kernels.glu(gu, out, kind, limit=1.5, alpha=1.702)
    assert helpers.rel_err(out, want) <= 3e-6
    inter_leaved = torch.stack([gu[:, :inter], gu[:, inter:]], dim=2).reshape(n, 2 * inter).to(torch.bfloat16).contiguous()
    out16 = torch.empty(n, inter, dtype=torch.bfloat16, device="cuda")
    kernels.glu(inter_leaved, out16, kind, interleaved=True, limit=1.5, alpha=1.702)
    assert helpers.rel_err(out16, want) <= 2e-2


@pytest.mark.parametrize("H, G, N, vdim, groups", [(3, 1, 24, 16, 3), (4, 2, 128, 64, 1), (5, 5, 10, 12, 5), (6, 3, 20, 12, 2), (2, 1, 200, 40, 4)])
def test_state_space_kernel_against_a_loop(H, G, N, vdim, groups):
    g = torch.Generator().manual_seed(H * N)
    lens, slots = [37, 1, 16, 70], [2, 0, 5, 3]
    n, inner = sum(lens), H * vdim
    z_col, dt_col = 3, 3 + inner + 2
    proj = torch.randn(n, dt_col + H + 4, generator=g).cuda()
    xbc = torch.randn(n, inner + 2 * G * N + 3, generator=g).cuda()
    dt_bias, A_log, D, gain = (torch.randn(k, generator=g).cuda() for k in (H, H, H, inner))
    A_log = A_log - 2.0
    state = torch.randn(6, inner * N, generator=g).cuda() * 0.1
    before = state.clone()
    for out_dtype in (torch.float32, torch.bfloat16):
        state.copy_(before)
        out = torch.empty(n, inner, dtype=out_dtype, device="cuda")
        kernels.state_space(proj, z_col, dt_col, xbc, inner, inner + G * N, dt_bias, A_log, D, gain, 1e-5, groups, state,
                            step_of(lens, slots), H, G, N, vdim, out)
        p64, x64 = proj.double().cpu(), xbc.double().cpu()
        x = x64[:, :inner].view(n, H, vdim)
        B, C = x64[:, inner:inner + G * N].view(n, G, N), x64[:, inner + G * N:inner + 2 * G * N].view(n, G, N)
        dt = torch.nn.functional.softplus(p64[:, dt_col:dt_col + H] + dt_bias.double().cpu())
        decay = torch.exp(-torch.exp(A_log.double().cpu()) * dt)
        zz = p64[:, z_col:z_col + inner]
        t0 = 0
        for L, slot in zip(lens, slots):
            S = before[slot].double().cpu().view(H, vdim, N).transpose(1, 2).clone()       # the kernel keeps [head][column][row]
            for t in range(t0, t0 + L):
                Bh, Ch = B[t].repeat_interleave(H // G, dim=0), C[t].repeat_interleave(H // G, dim=0)
                S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bh[:, :, None] * x[t][:, None, :]
                y = torch.einsum("hnv,hn->hv", S, Ch) + D.double().cpu()[:, None] * x[t]
                y = (y.reshape(-1) * pn.silu(zz[t])).view(groups, -1)
                y = (y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + 1e-5)).reshape(-1) * gain.double().cpu()
                tol = 3e-4 if out_dtype == torch.float32 else 3e-2
                assert torch.allclose(out[t].double().cpu(), y, atol=tol, rtol=tol), (t, float((out[t].double().cpu() - y).abs().max()))
            assert torch.allclose(state[slot].double().cpu().view(H, vdim, N).transpose(1, 2), S, atol=2e-4, rtol=2e-4)
            t0 += L
        assert torch.equal(state[1], before[1]) and torch.equal(state[4], before[4])       # slots of no sequence are untouched


@pytest.mark.parametrize("n, E, top", [(50, 6, 2), (1, 4, 4), (300, 33, 1), (17, 200, 7)])
def test_routing_by_sigmoid_scores_and_weights_on_the_input(n, E, top):
    g = torch.Generator().manual_seed(n + E)
    K = 72
    router = torch.randn(E, K, generator=g).cuda() * 0.4
    for dtype in (torch.float32, torch.bfloat16):
        hx = torch.randn(n, K, generator=g).to(dtype).cuda()
        ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
        kernels.moe_route(hx, None, top, ids, wts, router=router, weighting="sigmoid")
        s = torch.sigmoid(hx.double() @ router.double().t())
        val, idx = torch.topk(s, top, dim=-1)
        sure = torch.ones(n, dtype=torch.bool, device="cuda")
        if top > 1:
            sure &= (val[:, :-1] - val[:, 1:]).min(dim=-1).values > 1e-6
        if top < E:
            sure &= (val[:, -1] - torch.topk(s, top + 1, dim=-1).values[:, -1]) > 1e-6
        assert int(sure.sum()) >= n * 0.5
        assert torch.equal(ids.long()[sure], idx[sure]) and torch.allclose(wts[sure].double(), val[sure], atol=1e-6, rtol=1e-5)
        # the rows of the sorted order, each multiplied by its own pair's weight
        tile = 64
        rows = kernels.moe_plan_rows(n * top, E, tile)
        row_of = torch.empty(n, top, dtype=torch.int32, device="cuda")
        src_tok = torch.empty(rows, dtype=torch.int32, device="cuda")
        tile_expert = torch.empty(rows // tile, dtype=torch.int32, device="cuda")
        kernels.moe_plan(ids, E, tile, row_of, src_tok, tile_expert)
        hs = torch.full((rows, K), 7.0, dtype=dtype, device="cuda")
        kernels.moe_gather(hx, src_tok, hs, wts, row_of)
        want = torch.zeros(rows, K, dtype=torch.float64, device="cuda")
        want[row_of.long().reshape(-1)] = (wts.double()[:, :, None] * hx.double()[:, None, :]).reshape(n * top, K)
        assert helpers.rel_err(hs, want) <= (1e-6 if dtype == torch.float32 else 5e-3)


def test_attention_with_chunks_and_a_soft_cap_against_plain_torch():
    """The float32-arithmetic attention kernel on a cache filled by hand: chunks of 1, 5, a page and 70 over prompts, portions
    and single tokens, with and without the cap; one key per row made to stand out so that a mask that is one off shows."""
    from mini_llama_cpp_release_b200.kernels import KVView
    g = torch.Generator().manual_seed(9)
    H, KV, hd, page = 4, 2, 32, 64
    total = 200
    k = torch.randn(total, KV, hd, generator=g)
    v = torch.randn(total, KV, hd, generator=g)
    qs = torch.randn(total, H, hd, generator=g) * 3.0
    n_pages = (total + page - 1) // page
    k_pool = torch.zeros(1, n_pages, KV, page, hd)
    v_pool = torch.zeros(1, n_pages, KV, page, hd)
    for p in range(total):
        k_pool[0, p // page, :, p % page] = k[p]
        v_pool[0, p // page, :, p % page] = v[p]
    table = torch.arange(n_pages, dtype=torch.int32).view(1, -1).cuda()
    kv = KVView(k_pool.cuda(), v_pool.cuda(), 0, table, page, KV, hd)
    for chunk in (1, 5, 64, 70, 0):
        for cap in (0.0, 2.5):
            mask = pn.visible(total, chunk or None)
            want = pn.softmax_attention(qs.double(), k.double(), v.double(), 0.3, mask, softcap=cap or None).reshape(total, H * hd)
            for start, q_len in ((0, total), (130, 70), (139, 1), (140, 1), (199, 1)):
                q = qs[start:start + q_len].reshape(q_len, H * hd).contiguous().cuda()
                o = torch.empty_like(q)
                i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
                kernels.attention_simt(q, o, i32([0, q_len]), i32([start]), 1, q_len, H, kv, 0.3, chunk=chunk, softcap=cap)
                assert helpers.rel_err(o, want[start:start + q_len]) <= 2e-5, (chunk, cap, start, q_len)


def chunked_case(impl, lens, q_lens, H, KV, hd, chunk, cap, n_splits=1, row_tiles=4, in_cluster=False, seed=0):
    """Sequences of `lens` cached tokens of which the last `q_lens` are the step's, through one tensor-core attention kernel
    with a mask of chunks and a soft cap, against the plain masked softmax.  Queries are long, so single keys decide rows
    and scores reach into the cap's bend."""
    from test_kernels_gpu import make_paged
    dtype = torch.bfloat16
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
    args = (q.view(N, H * hd), out.view(N, H * hd), cu, start, len(lens), max(q_lens), H, kv, scale, 0)
    if impl == "tcgen05":
        kernels.attention_tcgen05(*args, chunk=chunk, softcap=cap)
        torch.cuda.synchronize()
        kernels.check_gemm_status(q.device)
    else:
        kernels.attention_mma(*args, row_tiles, n_splits, part_ml, part_o, chunk=chunk, softcap=cap)
    want = torch.cat([pn.softmax_attention(qq.double(), k.double(), v.double(), scale, pn.visible(n, chunk or None), softcap=cap or None)[n - m:]
                      for qq, k, v, n, m in zip(qs, ks, vs, lens, q_lens)]).float()
    got = out.float().cpu().view(N, H, hd)
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max()), (impl, chunk, cap, float((got - want).abs().max()))


@pytest.mark.parametrize("hd", [64, 128, 32])
@pytest.mark.parametrize("chunk, cap", [(50, 4.0), (64, 0.0), (130, 2.5), (1, 3.0), (0, 5.0), (300, 0.0)])
def test_tensor_core_attention_with_chunks_and_a_soft_cap(hd, chunk, cap):
    lens, q_lens = [330, 64, 129, 7], [330, 64, 70, 7]
    for H, KV in ((4, 2), (3, 3)):
        if hd in (64, 128):
            chunked_case("tcgen05", lens, q_lens, H, KV, hd, chunk, cap, seed=hd + chunk)
        for row_tiles in (4, 1):
            chunked_case("mma", lens, q_lens, H, KV, hd, chunk, cap, row_tiles=row_tiles, seed=hd + chunk + 1)
        chunked_case("mma", lens, q_lens, H, KV, hd, chunk, cap, n_splits=3, row_tiles=4, seed=hd + chunk + 2)
        # single tokens: the decode form, keys shared out inside a cluster and through partial results
        dec = [331, 65, 130, 200, 1, 51]
        chunked_case("mma", dec, [1] * len(dec), H, KV, hd, chunk, cap, n_splits=1, row_tiles=1, seed=hd + chunk + 3)
        chunked_case("mma", dec, [1] * len(dec), H, KV, hd, chunk, cap, n_splits=2, row_tiles=1, in_cluster=True, seed=hd + chunk + 4)
        chunked_case("mma", dec, [1] * len(dec), H, KV, hd, chunk, cap, n_splits=3, row_tiles=1, seed=hd + chunk + 5)


@pytest.mark.parametrize("glu", ["gelu_tanh", ("clamped", 1.5, 1.702), "silu"])
def test_gated_units_in_the_epilogues_of_the_tensor_core_products(glu):
    """gate and up rows alternate in w; the product's epilogue forms the gated unit from the float32 accumulators: the
    few-token form, the prompt form on one SM and on a pair of SMs, and the grouped form."""
    g = torch.Generator().manual_seed(17)
    K, inter = 192, 256
    w = (torch.randn(2 * inter, K, generator=g) * 0.2).bfloat16().cuda()
    gate_w, up_w = w[0::2].double(), w[1::2].double()

    def want_of(x, gw=gate_w, uw=up_w):
        gate, up = x.double() @ gw.t(), x.double() @ uw.t()
        if glu == "silu":
            return pn.silu(gate) * up
        if glu == "gelu_tanh":
            return pn.gelu_tanh(gate) * up
        gc, uc = gate.clamp(max=glu[1]), up.clamp(-glu[1], glu[1])
        return gc * torch.sigmoid(glu[2] * gc) * (uc + 1.0)
    for n, form in ((5, "few"), (40, "few"), (300, "rows"), (512, "pair")):
        x = torch.randn(n, K, generator=g).bfloat16().cuda()
        out = torch.empty(n, inter, dtype=torch.bfloat16, device="cuda")
        if form == "few":
            kernels.gemm_tcgen05(x, w, out, kernels.bindings.EPI_SILU_MUL, glu=glu)
        elif form == "rows":
            kernels.gemm_tcgen05_rows(x, w, out, kernels.bindings.EPI_SILU_MUL, glu=glu)
        else:
            kernels.gemm_tcgen05_pair(x, w, out, kernels.bindings.EPI_SILU_MUL, glu=glu)
        torch.cuda.synchronize()
        kernels.check_gemm_status(x.device)
        assert helpers.rel_err(out, want_of(x)) <= 1.5e-2, (form, n)
    # grouped: three matrices, tiles of 128 rows each with a group of its own, one tile skipped
    w3 = (torch.randn(3, 2 * inter, K, generator=g) * 0.2).bfloat16().cuda()
    x = torch.randn(4 * 128, K, generator=g).bfloat16().cuda()
    tiles = torch.tensor([2, 0, -1, 1], dtype=torch.int32, device="cuda")
    out = torch.zeros(4 * 128, inter, dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05_grouped(x, w3, tiles, out, kernels.bindings.EPI_SILU_MUL, glu=glu)
    torch.cuda.synchronize()
    kernels.check_gemm_status(x.device)
    for t, e in enumerate(tiles.tolist()):
        rows = slice(128 * t, 128 * (t + 1))
        if e < 0:
            assert float(out[rows].abs().max()) == 0.0
        else:
            assert helpers.rel_err(out[rows], want_of(x[rows], w3[e, 0::2].double(), w3[e, 1::2].double())) <= 1.5e-2, t
