"""Dunelix on the host: configuration, run order, weight names, cache needs, and the plain implementation's own
consistency (a recurrence carried from a state, attention over earlier keys)."""
import copy
import json
import os

import pytest
import torch

import plain_dunelix as pd
from dunelix_util import DUNE, DUNE_A, DUNE_B, DUNE_C


def test_config_reads_every_key_and_names_the_wrong_one():
    from tiny_llm_b200.config import ConfigError, DunelixConfig, config_from_dict
    cfg = config_from_dict(copy.deepcopy(DUNE_A))
    assert isinstance(cfg, DunelixConfig) and (cfg.vocab, cfg.width, cfg.residual_mult, cfg.norm_eps) == (200, 64, 0.5, 1e-5)
    assert cfg.loop == (0, 2, 3)
    assert config_from_dict(cfg.to_dict()) == cfg
    for path, value, word in [(("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "type"), "lstm", "lstm"),
                              (("layers", 1, "mixer", "rot", "dims"), 18, "dims"), (("loop", "stop"), 9, "loop"),
                              (("layers", 0, "mlp", "kind"), "moe", "moe"), (("width",), None, "width")]:
        d = copy.deepcopy(DUNE_A)
        at = d
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError) as e:
            config_from_dict(d)
        assert word in str(e.value)


def test_run_order_repeats_the_span_and_adds_the_embedding_before_later_passes():
    from tiny_llm_b200.config import DunelixConfig
    order = DunelixConfig.from_dict(DUNE_A).model_spec().order
    assert [(c.layer, c.add_embedding) for c in order] == [(0, False), (1, False), (0, True), (1, False), (0, True), (1, False),
                                                           (2, False), (3, False)]
    order = DunelixConfig.from_dict(DUNE_B).model_spec().order
    assert [(c.layer, c.add_embedding) for c in order] == [(0, False), (1, False), (2, False), (1, True), (2, False)]
    assert [c.layer for c in DunelixConfig.from_dict(DUNE_C).model_spec().order] == [0, 1]
    assert pd.run_order(DUNE_A) == [(c.layer, c.add_embedding) for c in DunelixConfig.from_dict(DUNE_A).model_spec().order]


def test_weight_names_cache_needs_and_a_layer_without_feed_forward():
    from tiny_llm_b200.cache import CacheManager, KVNeed, StateNeed
    from tiny_llm_b200.config import DunelixConfig
    from tiny_llm_b200.parts import DecoderModel
    model = DecoderModel(DunelixConfig.from_dict(DUNE_A).model_spec())
    names = set(model.weight_specs())
    assert {"embed", "head", "final.norm", "final.norm.b", "final.norm.alpha", "l0.mix.z", "l0.mix.z.b", "l0.mix.x.b", "l0.mix.g",
            "l0.mix.o", "l1.mix.q", "l1.mix.lq1", "l1.mix.lk2", "l1.norm2.alpha", "l3.mlp.down", "l2.norm1"} <= names
    assert not any(n.startswith("l2.mlp") or n.startswith("l2.norm2") for n in names)
    assert model.weight_specs()["l1.mix.q"].shape == (4 * 2 * 16, 64) and model.weight_specs()["l1.mix.v"].shape == (2 * 40, 64)
    assert model.weight_specs()["final.norm.alpha"].shape == ()
    needs = model.cache_needs()
    assert len(needs) == 8 and needs[0] == needs[2] == needs[4] == StateNeed((96,), torch.float32)
    assert needs[1] == needs[3] == KVNeed(2, 16, None, value_dim=40, key_rows=2, chunk=24)
    assert needs[7] == KVNeed(2, 32, None, value_dim=24, key_rows=2, chunk=None)
    cache = CacheManager(needs, max_tokens=64, page_size=16, max_slots=2)
    cache.allocate_storage(torch.float32, "cpu")
    assert len(cache.groups) == 2 and cache.groups[0].num_entries == 3
    assert cache.groups[0].k.shape == (3, 4, 4, 16, 16) and cache.groups[0].v.shape == (3, 4, 2, 16, 40)
    assert [t.shape for t in cache.slots.tensors] == [(2, 96)] * 3 + [(2, 48)]


def test_pages_behind_the_chunk_go_back_to_the_pool():
    from tiny_llm_b200.cache import CacheManager, KVNeed
    cache = CacheManager([KVNeed(1, 8, None, value_dim=4, key_rows=2, chunk=24)], max_tokens=64, page_size=16, max_slots=2)
    cache.add_request("a")
    g = cache.groups[0]
    assert cache.reserve("a", 23)
    cache.commit("a", 23)           # next token 23: chunk [0, 24), nothing passed
    assert g.tables["a"] == [0, 1]
    assert cache.reserve("a", 1)
    cache.commit("a", 1)            # next token 24: chunk [24, 48) starts inside page 1; page 0 is passed
    assert g.tables["a"] == [-1, 1] and g.pool.num_free == 3
    assert cache.reserve("a", 30)
    cache.commit("a", 30)           # next token 54: chunk [48, 72) starts with page 3
    assert g.tables["a"] == [-1, -1, -1, g.tables["a"][3]] and g.pool.num_used == 1
    cache.check()
    cache.free_request("a")
    assert g.pool.num_used == 0


def test_frequencies_of_the_product_and_of_the_plain_implementation_agree():
    from tiny_llm_b200.parts import scaled_pair_frequencies
    for dims, base, scaling in [(8, 100.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}), (24, 5000.0, None),
                                (16, 10000.0, {"factor": 8.0, "low": 2.0, "high": 6.0, "original": 300})]:
        a, b = scaled_pair_frequencies(dims, base, scaling), pd.scaled_frequencies(dims, base, scaling)
        assert a.shape == (dims // 2,) and torch.allclose(a, b, rtol=1e-6, atol=0)
    # all three regimes occur in the first set: kept, blended, divided by the factor
    f = pd.scaled_frequencies(8, 100.0, None)
    g = pd.scaled_frequencies(8, 100.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
    ratio = (g / f).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-6 and any(0.26 < r < 0.99 for r in ratio)


def test_plain_recurrence_and_attention_carry_on_from_what_came_before():
    g = torch.Generator().manual_seed(0)
    t, h, w = 19, 12, 10
    x = torch.randn(t, h, generator=g)
    ws = [torch.randn(w, h, generator=g) * 0.5 for _ in range(3)] + [torch.randn(h, w, generator=g)]
    bz, bx = torch.randn(w, generator=g), torch.randn(w, generator=g)
    whole, s_whole = pd.min_gru(x, ws[0], bz, ws[1], bx, ws[2], ws[3])
    a, s = pd.min_gru(x[:7], ws[0], bz, ws[1], bx, ws[2], ws[3])
    b, s2 = pd.min_gru(x[7:], ws[0], bz, ws[1], bx, ws[2], ws[3], state=s)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-6) and torch.allclose(s2, s_whole, atol=1e-6)
    assert (pd.min_gru_candidate(torch.tensor([-50.0, -1e-9, 0.0, 3.0])) > 0).all()
    p = dict(heads=4, kv_heads=2, dim=6, vdim=5, scale=0.4, diff=0.3, mask={"size": 8}, rot={"dims": 4, "base": 50.0})
    wq, wk, wv = torch.randn(48, h, generator=g), torch.randn(24, h, generator=g), torch.randn(10, h, generator=g)
    wo = torch.randn(h, 20, generator=g)
    lam = [torch.randn(6, generator=g) * 0.3 for _ in range(4)]
    pos = torch.arange(t)
    whole, _, _ = pd.differential_attention(x, pos, p, wq, wk, wv, wo, *lam, 1e-5)
    first, k, v = pd.differential_attention(x[:11], pos[:11], p, wq, wk, wv, wo, *lam, 1e-5)
    rest, _, _ = pd.differential_attention(x[11:], pos[11:], p, wq, wk, wv, wo, *lam, 1e-5, k_past=k, v_past=v,
                                           past_positions=pos[:11])
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-5)
    m = pd.chunk_mask(torch.tensor([7, 8, 15, 16]), torch.arange(17), 8)
    assert m[0].nonzero().flatten().tolist() == list(range(8)) and m[1].nonzero().flatten().tolist() == [8]
    assert m[2].nonzero().flatten().tolist() == list(range(8, 16)) and m[3].nonzero().flatten().tolist() == [16]


def test_random_weights_mode_writes_a_model_the_plain_implementation_reads(tmp_path):
    from tiny_llm_b200.config import DunelixConfig, load_config
    from tiny_llm_b200.weights import write_random_model
    cfg, _page, seed = DUNE["C"]
    d = write_random_model(str(tmp_path / "m"), DunelixConfig.from_dict(cfg), seed=seed, dtype=torch.float32)
    assert load_config(d) == DunelixConfig.from_dict(cfg)
    with open(os.path.join(d, "config.json")) as f:
        assert json.load(f)["architecture"] == "Dunelix"
    logits, streams = pd.forward(pd.load_config(d), pd.load_weights(d), [3, 1, 4, 1, 5, 9, 2, 6, 5, 3], return_layers=True)
    assert logits.shape == (10, 128) and streams.shape == (2, 10, 48) and torch.isfinite(logits).all()
