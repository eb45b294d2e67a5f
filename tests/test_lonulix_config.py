"""Lonulix without a GPU: its configuration, what its layers ask of the cache and of the state, the names of its tensors,
the cache's bookkeeping under its windows, and the plain implementation's mechanisms against each other."""
import copy
import math

import pytest
import torch

import lonulix_helpers as lh
import plain_lonulix as pl
from mini_llama_cpp_release_b200.cache.paged import SlotBook, plan_groups
from mini_llama_cpp_release_b200.config import ModelConfig
from mini_llama_cpp_release_b200.config.model_config import ConfigError
from mini_llama_cpp_release_b200.config.registry import build_model_spec
from mini_llama_cpp_release_b200.engine.model import build_parts
from mini_llama_cpp_release_b200.parts.base import CacheNeed

rnd_gen = torch.Generator().manual_seed(0)


def rnd(*shape):
    return torch.randn(*shape, generator=rnd_gen, dtype=torch.float64)


def test_config_round_trip_and_checks():
    cfg = ModelConfig.from_dict(lh.MIXED)
    assert cfg.architecture == "Lonulix" and cfg.vocab_size == 300 and cfg.hidden_size == 96
    assert (cfg.norm_groups, cfg.alpha, cfg.embedding_scale, cfg.norm_eps) == (3, 1.5, 2.5, 1e-5)
    assert ModelConfig.from_dict(cfg.to_dict()) == cfg
    for path, value in [(("layers", 0, "type"), "conv"), (("norm", "groups"), 5), (("layers", 1, "mlp", "kind"), "sparse"),
                        (("norm", "eps"), 0.0)]:
        bad = copy.deepcopy(lh.MIXED)
        d = bad
        for key in path[:-1]:
            d = d[key]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            ModelConfig.from_dict(bad)
    # what the parts refuse when the model is built: rot.dims other than rot_dim, experts that do not fill equal groups,
    # fewer experts in the kept groups than are chosen
    for path, value in [(("layers", 0, "mixer", "rot", "dims"), 4), (("layers", 0, "mlp", "router", "groups", "count"), 4),
                        (("layers", 0, "mlp", "router", "groups", "keep"), 0), (("layers", 0, "mlp", "router", "top"), 5)]:
        bad = copy.deepcopy(lh.MIXED)
        d = bad
        for key in path[:-1]:
            d = d[key]
        d[path[-1]] = value
        with pytest.raises((ConfigError, ValueError)):
            build_parts(build_model_spec(ModelConfig.from_dict(bad)))


def test_what_the_layers_ask_of_the_cache_and_the_state_and_which_tensors_they_read():
    spec = build_model_spec(ModelConfig.from_dict(lh.MIXED))
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 4] and all(l.block.kind == "post_norm" for l in spec.layers)
    parts = build_parts(spec)
    mixers = [parts.blocks[e.layer].mixer for e in spec.schedule]
    needs = [m.cache_need() for m in mixers]
    assert needs[0] == CacheNeed("window", 1, 48, 40, 0, True)                 # ceil16(40 + 8), values inside the key rows
    assert needs[3] == CacheNeed("window", 1, 48, 70, 0, True) and needs[1] is None and needs[2] is None and needs[4] is None
    groups, where = plan_groups(needs, [None] * len(needs))
    assert len(groups) == 2 and where[0][0] != where[3][0]                     # two windows, two groups of pages
    states = [m.state_spec().shape if getattr(m, "state_spec", None) and m.state_spec() else None for m in mixers]
    assert states == [None, (3 * 24 * 40,), (2 * 16 * 24,), None, (40 * 16,)]
    names = {t.name: tuple(t.shape) for p in parts.all_parts() for t in p.all_tensors()}
    assert names["embed"] == (300, 96) and names["head"] == (300, 96) and names["final.norm"] == (96,)
    assert names["l0.mix.dq"] == (28, 96) and names["l0.mix.dq.norm"] == (28,) and names["l0.mix.uq"] == (3 * 32, 28)
    assert names["l0.mix.dkv"] == (48, 96) and names["l0.mix.uk"] == (72, 40) and names["l0.mix.uv"] == (60, 40)
    assert names["l0.mlp.router"] == (6, 96) and names["l0.mlp.correction"] == (6,) and names["l0.mlp.e4.up"] == (48, 96)
    assert "l0.mlp.e5.up" not in names and "l0.mlp.e0.gate" not in names and "l0.mix.q" not in names    # an identity expert has no tensors
    assert names["l1.mix.f.b"] == (72,) and names["l1.mix.lower"] == (72,) and names["l1.mix.norm"] == (40,)
    assert names["l1.mlp.gate"] == (112, 96) and names["l2.rg1"] == (96, 96) and names["l2.rg1.b"] == (96,)
    assert "l2.rg2" not in names and "l2.norm2" not in names and names["l3.norm2"] == (96,)
    # a layer without a window keeps every position
    odd = build_parts(build_model_spec(ModelConfig.from_dict(lh.ODD)))
    assert odd.blocks[4].mixer.cache_need() == CacheNeed("all", 1, 32, None, 0, True)
    assert odd.blocks[1].mixer.cache_need().window == 1


def test_a_window_gives_back_the_pages_it_has_left():
    need = CacheNeed("window", 1, 48, window=70, shared_kv=True)
    book = SlotBook(plan_groups([need], [None])[0], max_tokens=1024, max_seqs=4)
    s = book.acquire()
    book.reserve(s, 400)
    book.commit(s, 400)
    pages = book.page_lists[s][0]
    assert pages[:5] == [-1] * 5 and all(p >= 0 for p in pages[5:])           # position 330 is the oldest a later token reads
    for _ in range(200):
        book.reserve(s, 1)
        book.commit(s, 1)
    pages = book.page_lists[s][0]
    assert all(p == -1 for p in pages[:8]) and pages[8] >= 0
    book.check()
    book.release(s)
    book.check()
    assert book.pages[0].n_held == 0


def test_plain_norm_in_groups():
    x, w = rnd(7, 12), rnd(12)
    assert torch.allclose(pl.group_norm(x, w, 1, 1e-5), pl.rms_norm(x, w, 1e-5))
    got = pl.group_norm(x, w, 3, 1e-5)
    for g in range(3):
        part = x[:, 4 * g:4 * g + 4]
        assert torch.allclose(got[:, 4 * g:4 * g + 4], part / torch.sqrt((part ** 2).mean(-1, keepdim=True) + 1e-5) * w[4 * g:4 * g + 4])


def test_plain_rotation_turns_neighbours_and_scores_depend_on_the_distance():
    x = rnd(9, 2, 10)
    pos = torch.arange(9)
    y = pl.rotate_neighbours(x, pos, 6, 50.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    a = 5 * 50.0 ** (-2.0 / 6)                                                  # position 5, pair 1
    assert torch.allclose(y[5, :, 2], x[5, :, 2] * math.cos(a) - x[5, :, 3] * math.sin(a), atol=1e-6)
    assert torch.allclose(y[5, :, 3], x[5, :, 3] * math.cos(a) + x[5, :, 2] * math.sin(a), atol=1e-6)
    q, k = rnd(1, 1, 6).expand(9, 1, 6), rnd(1, 1, 6).expand(9, 1, 6)
    s = pl.rotate_neighbours(q, pos, 6, 50.0)[:, 0] @ pl.rotate_neighbours(k, pos, 6, 50.0)[:, 0].t()
    assert torch.allclose(s[7, 3], s[5, 1], atol=1e-5) and torch.allclose(s[8, 8], s[0, 0], atol=1e-5)


def test_plain_window():
    m = pl.window_mask(12, 4)
    assert m[11].tolist() == [False] * 8 + [True] * 4 and m[2].tolist() == [True] * 3 + [False] * 9
    assert pl.window_mask(5, None).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()
    assert pl.window_mask(6, 1).tolist() == torch.eye(6, dtype=torch.bool).tolist()


def test_plain_routing_by_scores():
    h = rnd(40, 6)
    w = {"r.router": rnd(9, 6), "r.correction": rnd(9) * 0.3}
    router = {"experts": 7, "identity": 2, "top": 3, "scale": 2.5, "groups": {"count": 3, "keep": 2}}
    idx, wt = pl.route(h, w, "r.", router)
    s = torch.softmax(h @ w["r.router"].t(), dim=-1)
    choice = s + w["r.correction"]
    best = choice.view(40, 3, 3).max(dim=-1).values
    worst_group = best.argmin(dim=-1)
    assert not bool((idx // 3 == worst_group[:, None]).any())                  # nothing from the group that was dropped
    assert torch.allclose(wt.sum(dim=-1), torch.full((40,), 2.5, dtype=torch.float64))
    assert torch.allclose(wt[:, 0] / wt[:, 1], s.gather(1, idx)[:, 0] / s.gather(1, idx)[:, 1])     # weights from the scores alone
    open_choice = choice.masked_fill((torch.arange(9)[None, :] // 3) == worst_group[:, None], float("-inf"))
    assert torch.equal(idx, torch.topk(open_choice, 3, dim=-1).indices)
    assert int((idx >= 7).sum()) > 0                                           # identity experts are chosen like the others
    # one group, no correction, one chosen: the largest score with the weight `scale`
    idx1, wt1 = pl.route(h, {"r.router": w["r.router"]}, "r.", {"experts": 9, "top": 1, "scale": 0.5})
    assert torch.equal(idx1[:, 0], s.argmax(dim=-1)) and torch.allclose(wt1, torch.full((40, 1), 0.5, dtype=torch.float64))


def test_plain_identity_experts_return_their_input():
    h = rnd(5, 6)
    w = {"m.router": rnd(4, 6), "m.correction": torch.tensor([-9.0, -9.0, 0.0, 0.0], dtype=torch.float64),
         "m.e0.up": rnd(3, 6), "m.e0.down": rnd(6, 3), "m.e1.up": rnd(3, 6), "m.e1.down": rnd(6, 3)}
    mlp = {"router": {"experts": 2, "identity": 2, "top": 2, "scale": 3.0, "groups": {"count": 1, "keep": 1}}}
    assert torch.allclose(pl.moe_ff(h, w, "m.", mlp), 3.0 * h)                 # both choices are identity experts


def test_plain_forget_gate_attention_in_closed_form():
    """o_t = sum_{s<=t} (prod_{s<r<=t} f_r) * (1 - f_s) * q_t, channel by channel, times v_s."""
    T, H, d, dv, width = 9, 2, 3, 4, 5
    m = {"heads": H, "dim": d, "vdim": dv}
    w = {"q": rnd(H * d, width), "f": rnd(H * d, width), "f.b": rnd(H * d), "lower": torch.rand(H * d, dtype=torch.float64),
         "v": rnd(H * dv, width), "norm": rnd(dv), "o": torch.eye(H * dv, dtype=torch.float64)}
    h = rnd(T, width)
    f = pl.forget_gates(h, w, "", m)
    assert bool((f >= w["lower"].view(H, d)).all()) and bool((f < 1).all())
    q = pl.silu(h @ w["q"].t()).view(T, H, d)
    v = (h @ w["v"].t()).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            carry = f[s + 1:t + 1].prod(dim=0)
            o[t] += torch.einsum("hd,hv->hv", carry * (1 - f[s]) * q[t], v[s])
    want = pl.rms_norm(o, w["norm"], 1e-6).reshape(T, H * dv)
    states = []
    assert torch.allclose(pl.hgrn2(h, w, "", m, 1e-6, states), want, atol=1e-10)
    # cut in two: the second half from the first half's state is what the recurrence promises
    assert states[0].shape == (H, d, dv)


def test_plain_latent_attention_equals_attention_on_the_cached_rows():
    """The form the engine computes (key expansion on the query's side, value expansion behind the sum, one cached row
    [latent | rotated shared part] per token) against the plain form (keys and values expanded per head)."""
    T, H, d, r, dv, rank, qr, width = 11, 3, 6, 4, 5, 7, 8, 10
    m = {"heads": H, "dim": d, "rot_dim": r, "vdim": dv, "kv_rank": rank, "q_rank": qr, "scale": 0.3,
         "rot": {"dims": r, "base": 100.0}, "mask": {"size": 4}}
    w = {"dq": rnd(qr, width), "dq.norm": rnd(qr), "uq": rnd(H * (d + r), qr), "dkv": rnd(rank + r, width), "dkv.norm": rnd(rank),
         "uk": rnd(H * d, rank), "uv": rnd(H * dv, rank), "o": rnd(width, H * dv)}
    h = rnd(T, width)
    pos = torch.arange(T)
    want = pl.latent_attention(h, w, "", m, 1e-5, pos)
    q = (pl.rms_norm(h @ w["dq"].t(), w["dq.norm"], 1e-5) @ w["uq"].t()).view(T, H, d + r)
    down = h @ w["dkv"].t()
    c = pl.rms_norm(down[:, :rank], w["dkv.norm"], 1e-5)
    rows = torch.cat([c, pl.rotate_neighbours(down[:, None, rank:], pos, r, 100.0)[:, 0]], dim=-1)
    q2 = torch.cat([torch.einsum("thd,hdr->thr", q[..., :d], w["uk"].view(H, d, rank)),
                    pl.rotate_neighbours(q[..., d:], pos, r, 100.0)], dim=-1)
    mask = pl.window_mask(T, 4)
    o = torch.stack([torch.softmax((q2[:, hd] @ rows.t() * 0.3).masked_fill(~mask, float("-inf")), dim=-1) @ c for hd in range(H)], dim=1)
    got = torch.einsum("thr,hvr->thv", o, w["uv"].view(H, dv, rank)).reshape(T, H * dv) @ w["o"].t()
    assert torch.allclose(got, want, atol=1e-10)
