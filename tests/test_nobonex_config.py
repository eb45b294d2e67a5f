"""Nobonex without a GPU: its configuration, what its layers ask of the cache and of the state, the names of its tensors, the
cache's bookkeeping under masks of chunks, and the plain implementation's mechanisms against each other."""
import copy
import math

import pytest
import torch

import nobonex_helpers as nh
import plain_nobonex as pn
from mini_llama_cpp_release_b200.cache.paged import SlotBook, plan_groups
from mini_llama_cpp_release_b200.config import ModelConfig
from mini_llama_cpp_release_b200.config.model_config import ConfigError
from mini_llama_cpp_release_b200.config.registry import build_model_spec
from mini_llama_cpp_release_b200.engine.model import build_parts
from mini_llama_cpp_release_b200.parts.base import CacheNeed

rnd_gen = torch.Generator().manual_seed(0)


def rnd(*shape):
    return torch.randn(*shape, generator=rnd_gen, dtype=torch.float64)


def changed(config, path, value):
    bad = copy.deepcopy(config)
    d = bad
    for key in path[:-1]:
        d = d[key]
    d[path[-1]] = value
    return bad


def test_config_round_trip_and_checks():
    cfg = ModelConfig.from_dict(nh.MIXED)
    assert cfg.architecture == "Nobonex" and cfg.vocab_size == 300 and cfg.hidden_size == 96
    assert (cfg.residual_mult, cfg.embedding_scale, cfg.norm_eps) == (0.6, 3.0, 1e-5)
    assert ModelConfig.from_dict(cfg.to_dict()) == cfg
    for path, value in [(("layers", 0, "type"), "conv"), (("layers", 1, "mlp", "kind"), "sparse"), (("norm", "eps"), 0.0),
                        (("layers", 3, "mixer", "kv_from"), 3), (("layers", 3, "mixer", "kv_from"), 1),
                        (("layers", 3, "mixer", "kv_heads"), 1), (("layers", 2, "mixer", "kv_from"), 0)]:
        with pytest.raises(ConfigError):
            ModelConfig.from_dict(changed(nh.MIXED, path, value))
    # what the parts refuse when the model is built
    for path, value in [(("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "kv_heads"), 3),
                        (("layers", 1, "mixer", "groups"), 2), (("layers", 1, "mixer", "norm_groups"), 5),
                        (("layers", 0, "mlp", "router", "top"), 6), (("layers", 2, "mixer", "vdim"), 8),
                        (("layers", 0, "mixer", "softcap"), -1.0)]:
        with pytest.raises((ConfigError, ValueError)):
            build_parts(build_model_spec(ModelConfig.from_dict(changed(nh.MIXED, path, value))))


def test_what_the_layers_ask_of_the_cache_and_the_state_and_which_tensors_they_read():
    spec = build_model_spec(ModelConfig.from_dict(nh.MIXED))
    assert [(e.layer, e.reads_cache_of) for e in spec.schedule] == [(0, None), (1, None), (2, None), (3, 0), (4, None)]
    assert all(l.block.kind == "sandwich" for l in spec.layers)
    parts = build_parts(spec)
    mixers = [parts.blocks[e.layer].mixer for e in spec.schedule]
    needs = [m.cache_need() for m in mixers]
    assert needs[0] == CacheNeed("chunk", 2, 32, 50) and needs[3] == needs[0]          # ceil16(max(24, 20))
    assert needs[2] == CacheNeed("all", 3, 16) and needs[1] is None and needs[4] is None
    groups, where = plan_groups(needs, [e.reads_cache_of for e in spec.schedule])
    assert len(groups) == 2 and where[3] == where[0] and groups[where[0][0]].entries == [0]   # the reader owns no pages
    states = [m.state_spec().shape if m.state_spec() else None for m in mixers]
    assert states == [None, (3 * 16 * 24 + 2 * (48 + 48),), (3 * (96 + 48),), None, (4 * 8 * 40 + 1 * (32 + 160),)]
    names = {t.name: tuple(t.shape) for p in parts.all_parts() for t in p.all_tensors()}
    assert names["embed"] == (300, 96) and names["head"] == (300, 96)
    assert names["final.norm"] == (96,) and names["final.norm.b"] == (96,) and names["final.norm.alpha"] == ()
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert names[f"l0.{n}"] == (96,) and names[f"l0.{n}.b"] == (96,) and names[f"l0.{n}.alpha"] == ()
    assert "l2.norm2" not in names and "l2.norm2b" not in names and "l2.norm1b" in names
    assert names["l0.mix.q"] == (96, 96) and names["l0.mix.q.b"] == (96,) and names["l0.mix.k"] == (48, 96) and names["l0.mix.v"] == (40, 96)
    assert names["l0.mix.v.b"] == (40,) and names["l0.mix.q.norm"] == (24,) and names["l0.mix.k.norm"] == (24,)
    assert names["l0.mix.g"] == (80, 96) and names["l0.mix.o"] == (96, 80)
    assert names["l3.mix.q"] == (96, 96) and names["l3.mix.g"] == (80, 96) and names["l3.mix.q.norm"] == (24,)
    assert not any(k.startswith(("l3.mix.k", "l3.mix.v")) for k in names)                   # the reader has no keys of its own
    assert names["l2.mix.q"] == (96, 96) and names["l2.mix.k"] == (48, 96) and "l2.mix.v" not in names
    assert names["l2.mix.q.norm"] == (96,) and names["l2.mix.k.norm"] == (48,) and names["l2.mix.q.conv"] == (96, 4) and names["l2.mix.k.conv"] == (48, 4)
    assert names["l1.mix.in"] == (2 * 48 + 2 * 24 + 3, 96) and names["l1.mix.conv"] == (96, 3) and names["l1.mix.conv.b"] == (96,)
    assert names["l1.mix.dt_bias"] == (3,) and names["l1.mix.A_log"] == (3,) and names["l1.mix.D"] == (3,) and names["l1.mix.norm"] == (48,)
    assert names["l0.mlp.router"] == (5, 96) and names["l0.mlp.e4.gate"] == (48, 96) and names["l0.mlp.e4.down"] == (96, 48)
    assert "l0.mlp.e5.up" not in names and names["l1.mlp.gate"] == (112, 96)
    # a layer without a mask keeps every position; a layer whose reader has another mask keeps every position too
    odd = build_parts(build_model_spec(ModelConfig.from_dict(nh.ODD)))
    assert odd.blocks[4].mixer.cache_need() == CacheNeed("all", 1, 32)
    assert odd.blocks[0].mixer.cache_need() == CacheNeed("all", 5, 16) and odd.blocks[0].mixer.chunk == 7
    assert odd.blocks[2].mixer.cache_need().kind == "chunk" and odd.blocks[2].mixer.chunk == 1
    assert odd.blocks[3].mixer.state_spec() is None                                          # one tap: nothing to remember


def test_a_mask_of_chunks_gives_back_the_pages_the_sequence_has_left():
    need = CacheNeed("chunk", 2, 32, window=70)
    groups, where = plan_groups([need, None, need], [None, None, 0])
    assert len(groups) == 1 and where[2] == where[0]
    book = SlotBook(groups, max_tokens=64 * 12, max_seqs=4)
    s = book.acquire()
    book.reserve(s, 300)
    book.commit(s, 300)
    # the next token, position 300, reads from 280 on (page 4)
    assert book.page_lists[s][0][:4] == [-1] * 4 and all(p >= 0 for p in book.page_lists[s][0][4:])
    for _ in range(50):
        book.reserve(s, 1)
        book.commit(s, 1)
    assert book.page_lists[s][0][:5] == [-1] * 5 and book.page_lists[s][0][5] >= 0          # position 350 opens a chunk (page 5)
    book.check()
    book.release(s)
    book.check()
    assert book.pages[0].n_free == book.n_pages
    # a reader under another mask, or under none, cannot share an entry whose owner gives pages back
    with pytest.raises(ValueError):
        plan_groups([need, CacheNeed("chunk", 2, 32, window=50)], [None, 0])
    with pytest.raises(ValueError):
        plan_groups([need, CacheNeed("all", 2, 32)], [None, 0])
    plan_groups([CacheNeed("all", 2, 32), CacheNeed("chunk", 2, 32, window=50)], [None, 0])


def test_plain_mechanisms_against_each_other():
    T = 40
    pos = torch.arange(T)
    # both pairings rotate by the same angles: permuting the entries turns one into the other
    v = rnd(T, 2, 12)
    r = {"dims": 8, "base": 100.0}
    perm = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11])              # neighbours (2i, 2i+1) -> halves (i, i+4)
    a = pn.rotate(v, pos, r, neighbours=True)[..., perm]
    b = pn.rotate(v[..., perm], pos, r, neighbours=False)
    assert torch.allclose(a, b, atol=1e-12)
    assert torch.equal(pn.rotate(v, pos, r, True)[..., 8:], v[..., 8:])       # entries beyond rot.dims pass
    # stretched frequencies: fast pairs keep theirs, slow ones are divided by the factor; cos and sin get the multiplier
    f, mult = pn.frequencies(32, 1e4, {"factor": 4.0, "original": 128, "fast": 32.0, "slow": 1.0})
    f0, one = pn.frequencies(32, 1e4, None)
    assert one == 1.0 and f[0] == f0[0] and math.isclose(f[-1], f0[-1] / 4.0) and math.isclose(mult, 0.1 * math.log(4.0) + 1.0)
    # a mask of chunks: the chunk's first row sees itself alone, its last row the whole chunk and nothing before
    m = pn.visible(20, 7)
    assert m[7].sum() == 1 and m[13].sum() == 7 and not bool(m[13, 6]) and m[14].sum() == 1 and bool(pn.visible(20, None)[19].all())
    # the short convolution against a loop, with the last tap on the current token
    u, taps = rnd(T, 5), rnd(5, 3)
    y = pn.short_conv(u, taps)
    assert torch.allclose(y[0], taps[:, 2] * u[0]) and torch.allclose(y[5], taps[:, 0] * u[3] + taps[:, 1] * u[4] + taps[:, 2] * u[5])
    # a weight on an expert's input is not a weight on its output
    w = {"x.gate": rnd(6, 8), "x.up": rnd(6, 8), "x.down": rnd(8, 6)}
    h = rnd(3, 8)
    assert not torch.allclose(pn.expert(0.5 * h, w, "x.", 1.0), 0.5 * pn.expert(h, w, "x.", 1.0), atol=1e-3)
    # the state-space walk in chunks equals the walk at once when the state is carried: the last state of the first half,
    # put in front of the second half, is what the whole sequence leaves
    cfgm = nh.mamba2(2, 4, 6, 1, 3, 2)
    inner = 8
    wm = {"m.in": rnd(2 * inner + 12 + 2, 10) * 0.3, "m.conv": rnd(inner + 12, 3), "m.conv.b": rnd(inner + 12), "m.dt_bias": rnd(2),
          "m.A_log": rnd(2) - 1.0, "m.D": rnd(2), "m.norm": rnd(inner), "m.o": rnd(10, inner)}
    hm = rnd(T, 10)
    states = []
    full = pn.mamba2(hm, wm, "m.", cfgm, 1e-5, states)
    assert full.shape == (T, 10) and states[0].shape == (2, 6, 4) and float(states[0].abs().max()) > 0
