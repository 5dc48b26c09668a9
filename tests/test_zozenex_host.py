"""Zozenex on the host: configuration and its errors, tensor names, cache needs (a mixer with several), pages of a
cache entry with one row per block of positions, and the plain implementation's own consistency."""
import copy

import pytest
import torch

import plain_zozenex as pz
from zozenex_util import ZOZ, ZOZ_A, ZOZ_B, ZOZ_C


def test_configuration_round_trip_and_spec():
    from tiny_llm_b200.config import ZozenexConfig, config_from_dict
    for cfg, _, _ in ZOZ.values():
        c = config_from_dict(cfg)
        assert isinstance(c, ZozenexConfig) and ZozenexConfig.from_dict(c.to_dict()) == c
        spec = c.model_spec()
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"] and len(spec.layers) == len(cfg["layers"])
        assert spec.max_positions == cfg["max_positions"] and spec.after_embedding.kind == "learned_positions"
        for ls, l in zip(spec.layers, cfg["layers"]):
            assert ls.mixer.kind == {"retention": "retention", "parallel": "side_by_side"}[l["type"]]
            assert (ls.ffn is None) == (l["mlp"] is None) and (ls.norm2 is None) == (l["mlp"] is None)


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), None, "vocab"), (("layers", 0, "type"), "conv", "unknown mixer type"),
    (("layers", 0, "mixer", "decay"), [0.5], "decay"), (("layers", 1, "mixer", "left", "kv_heads"), 3, "multiple"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "dims"), (("layers", 1, "mixer", "right", "tau"), 0, "tau"),
    (("layers", 0, "mlp", "router", "top"), 7, "top"), (("layers", 0, "mlp", "kind"), "dense", "unknown kind"),
    (("norm",), None, "norm"), (("max_positions",), 0, "max_positions")])
def test_configuration_errors_name_the_key(path, value, word):
    from tiny_llm_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(ZOZ_A)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_tensor_names_and_cache_needs():
    from tiny_llm_b200.cache import CacheManager, KVNeed, StateNeed
    from tiny_llm_b200.config import config_from_dict
    from tiny_llm_b200.parts import DecoderModel
    model = DecoderModel(config_from_dict(ZOZ_A).model_spec())
    names = set(model.weight_specs())
    for n in ("embed", "pos", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.g", "l0.mix.o",
              "l0.mlp.router", "l0.mlp.correction", "l0.mlp.e5.up", "l0.mlp.e0.down", "l0.mlp.shared.sg",
              "l1.mix.left.q", "l1.mix.left.pb", "l1.mix.left.out", "l1.mix.right.a1", "l1.mix.right.a2.b",
              "l1.mix.right.norm", "l1.mix.right.out", "l2.mlp.e3.up"):
        assert n in names, n
    assert "l1.norm2" not in names and "l2.mlp.shared.up" not in names and "l0.mlp.e6.up" not in names
    assert model.weight_specs()["l2.mix.right.a1"].shape == (5, 64) and model.weight_specs()["l1.mix.right.a1"].shape == (None, 64)
    needs = model.cache_needs()
    assert needs[0] == StateNeed((2, 16, 24), torch.float32)
    tokens, blocks, state = needs[1]
    assert tokens == KVNeed(2, 16, 20, value_dim=24) and blocks == KVNeed(2, 16, None, value_dim=24, stride=8)
    assert state == StateNeed((2, 16, 32), torch.float32)
    assert needs[2][0].window == 16            # a pool larger than the window keeps a token until its block is complete
    cache = CacheManager(needs, max_tokens=64, page_size=4, max_slots=2)
    assert len(cache.groups) == 4 and len(cache.slots.needs) == 3
    assert isinstance(cache.refs[1], tuple) and [r.group for r in cache.refs[1][:2]] == [0, 1] and cache.refs[1][2].state == 1
    model_c = DecoderModel(config_from_dict(ZOZ_C).model_spec())
    n_c = model_c.cache_needs()
    assert len(n_c[1]) == 2 and n_c[1][0].window == 12 and n_c[2][0].window is None    # no pool: no block entry


def test_pages_of_an_entry_with_one_row_per_block():
    from tiny_llm_b200.cache import CacheManager, KVNeed
    cache = CacheManager([(KVNeed(1, 8, 6), KVNeed(1, 8, None, stride=5))], max_tokens=40, page_size=4, max_slots=2)
    tok, blk = cache.groups
    assert [blk.pages_for(n) for n in (0, 4, 5, 19, 20, 21, 24, 25)] == [0, 0, 1, 1, 1, 1, 1, 2]
    cache.add_request("a")
    held = []
    for n in (3, 2, 1, 14, 1, 4, 15):
        assert cache.reserve("a", n)
        cache.commit("a", n)
        total = cache.kv_len["a"]
        held.append((len([p for p in tok.tables["a"] if p >= 0]), len(blk.tables["a"])))
        assert len(blk.tables["a"]) == -(-(total // 5) // 4)
        assert tok.tables["a"][:max(0, total - 6 + 1) // 4] == [-1] * (max(0, total - 6 + 1) // 4)
        cache.check()
    assert held[-1][0] <= 3 and held[-1][1] == 2
    with pytest.raises(ValueError):
        CacheManager([KVNeed(1, 8, 6, stride=2)], max_tokens=16, page_size=4, max_slots=1)
    cache.free_request("a")
    assert tok.pool.num_used == 0 and blk.pool.num_used == 0


def test_step_metadata_names_the_block_a_token_completes():
    from tiny_llm_b200.cache import CacheManager, KVNeed
    from tiny_llm_b200.engine.step import ModelRunner, StepEntry
    from types import SimpleNamespace
    cache = CacheManager([(KVNeed(1, 8, 8), KVNeed(1, 8, None, stride=3))], max_tokens=64, page_size=4, max_slots=4)
    model = SimpleNamespace(loaded=True, graph_safe=False, spec=SimpleNamespace(max_positions=64, vocab_size=50))
    runner = ModelRunner(model, cache, torch.float32, "cpu", max_tokens_per_step=32, max_requests_per_step=4)
    for rid in "ab":
        cache.add_request(rid)
    entries = [StepEntry("a", [1] * 7, [0]), StepEntry("b", [2], [0])]
    for e in entries:
        assert cache.reserve(e.rid, len(e.tokens))
    b = runner.build_batch(entries)
    table = cache.groups[1].tables["a"]
    assert b.groups[1].slot_mapping.tolist() == [-1, -1, table[0] * 4, -1, -1, table[0] * 4 + 1, -1, -1]
    for e in entries:
        cache.commit(e.rid, len(e.tokens))
    # decode-only step: request a writes position 7 (no block ends), b position 1; then b position 2 ends block 0
    for want_b in (-1, None):
        entries = [StepEntry("a", [1], [0]), StepEntry("b", [2], [0])]
        for e in entries:
            assert cache.reserve(e.rid, 1)
        got = runner.build_batch(entries).groups[1].slot_mapping.tolist()
        for e in entries:
            cache.commit(e.rid, 1)
        if want_b == -1:
            assert got == [-1, -1]
        else:
            assert got == [cache.groups[1].tables["a"][0] * 4 + 2, cache.groups[1].tables["b"][0] * 4]


def _random_weights(cfg, seed):
    from tiny_llm_b200.config import config_from_dict
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights.random_init import random_state
    spec = config_from_dict(cfg).model_spec()
    return random_state(DecoderModel(spec).weight_specs(), seed, spec.initializer_range, torch.float32)


def test_the_plain_recurrences_carry_over():
    """The plain implementation against itself: a sequence in two halves with the state carried equals the whole."""
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(30, 2, 6, generator=g, dtype=torch.float64), torch.randn(30, 2, 6, generator=g, dtype=torch.float64)
    v, a = torch.randn(30, 2, 5, generator=g, dtype=torch.float64), torch.rand(30, 2, 6, generator=g, dtype=torch.float64)
    whole, s = pz.linear_recurrence(q, k, v, a)
    first, s1 = pz.linear_recurrence(q[:11], k[:11], v[:11], a[:11])
    second, s2 = pz.linear_recurrence(q[11:], k[11:], v[11:], a[11:], s1)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-12) and torch.allclose(s2, s, atol=1e-12)
    # closed form of a fixed decay: o_t = sum_j d^(t-j) (q_t . k_j) v_j
    d = torch.tensor([0.9, 0.5], dtype=torch.float64)
    o, _ = pz.linear_recurrence(q, k, v, d)
    t, h = 17, 1
    ref = sum(d[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
    assert torch.allclose(o[t, h], ref, atol=1e-10)


def test_the_plain_window_sees_what_the_rule_says():
    assert [pz.visible_blocks(i, 7, 3) for i in (8, 9, 11, 12, 13)] == [0, 1, 1, 2, 2]
    g = torch.Generator().manual_seed(1)
    t = 40
    q = torch.randn(t, 2, 4, generator=g, dtype=torch.float64)
    k, v = torch.randn(t, 1, 4, generator=g, dtype=torch.float64), torch.randn(t, 1, 3, generator=g, dtype=torch.float64)
    pb = torch.tensor([0.1, -0.2], dtype=torch.float64)
    out = pz.window_pool_sum(q, k, v, 0.5, None, pb, 7, 3)
    i, h = 25, 1
    ref = torch.zeros(3, dtype=torch.float64)
    for j in range(i - 6, i + 1):
        ref += torch.sigmoid(q[i, h] @ k[j, 0] * 0.5 + pb[h]) * v[j, 0]
    for b in range(6):          # blocks 0..5 end at 2, 5, .., 17 <= 25 - 7; block 6 ends at 20: not yet seen
        ref += torch.sigmoid(q[i, h] @ k[3 * b:3 * b + 3, 0].mean(0) * 0.5 + pb[h]) * v[3 * b:3 * b + 3, 0].mean(0)
    assert torch.allclose(out[i, h], ref, atol=1e-12)
    # positions 18, 19, 20 are neither in the window (19..25) nor in a seen block: moving them changes nothing
    k2 = k.clone()
    k2[18] += 5.0
    assert torch.allclose(pz.window_pool_sum(q, k2, v, 0.5, None, pb, 7, 3)[i], out[i], atol=1e-12)
    assert not torch.allclose(pz.window_pool_sum(q, k2, v, 0.5, None, pb, 7, 3)[27], out[27], atol=1e-6)   # block 6 ends at 20 = 27 - 7


@pytest.mark.parametrize("cfg", [ZOZ_A, ZOZ_C])
def test_the_plain_model_is_causal_and_its_quantised_run_is_close(cfg):
    w = _random_weights(cfg, 1)
    toks = torch.randint(0, cfg["vocab"], (45,), generator=torch.Generator().manual_seed(2)).tolist()
    full = pz.forward(cfg, w, toks, torch.float64)
    assert torch.allclose(pz.forward(cfg, w, toks[:20], torch.float64), full[:20], atol=1e-9)
    rounded = pz.forward(cfg, w, toks, torch.float64, quant=pz.bf16_quant)
    assert 0 < float((rounded - full).abs().max()) < 0.1 * float(full.abs().max())
