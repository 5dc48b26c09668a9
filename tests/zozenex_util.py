"""Tiny Zozenex configurations for the tests and the plain implementation's logits for them.

The configurations differ from one another in every size and option: widths, head counts and grouping, key size
against value size, windows and pools that are and are not multiples of the page (a pool larger than its window in
one), rotation over part of the key / the whole key / none (and then no rotated values), a cap on the scores or none,
a window without pooled blocks, attention without any mask, layers without a feed-forward, experts with and without
a shared expert, every expert chosen / one chosen, ranks of the decay's projection that are and are not multiples
of 8, and the order of the layer kinds."""
import torch

import plain_zozenex as pz


def left(heads, kv, dim, vdim, scale, softcap=None, size=None, pool=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if size:
        m["mask"] = {"size": size, **({"pool": pool} if pool else {})}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def right(heads, dim, vdim, tau, rank=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, **({"rank": rank} if rank else {})}


def moe(experts, top, ff, scale, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale},
            **({"shared": {"ff": shared}} if shared else {})}


def retention(heads, dim, vdim, decay, mlp):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def parallel(le, ri, mlp):
    return {"type": "parallel", "mixer": {"left": le, "right": ri}, "mlp": mlp}


ZOZ_A = {
    "architecture": "Zozenex", "vocab": 200, "width": 64, "max_positions": 512, "norm": {"eps": 1e-5},
    "initializer_range": 0.1,
    "layers": [
        retention(2, 16, 24, [0.9, 0.97], moe(6, 2, 40, 1.5, shared=48)),
        parallel(left(4, 2, 16, 24, 0.3, softcap=5.0, size=20, pool=8, rot=(8, 100.0)), right(2, 16, 32, 4.0), None),
        parallel(left(2, 2, 24, 16, 0.25, size=9, pool=16, rot=(24, 1000.0)), right(3, 8, 8, 1.0, rank=5), moe(4, 1, 24, 1.0)),
    ],
}
ZOZ_B = {
    "architecture": "Zozenex", "vocab": 331, "width": 96, "max_positions": 400, "norm": {"eps": 1e-6},
    "initializer_range": 0.08,
    "layers": [
        parallel(left(3, 1, 32, 48, 0.2, softcap=20.0, size=33, pool=5, rot=(16, 5000.0)), right(1, 40, 24, 8.0, rank=24),
                 moe(9, 3, 56, 2.5, shared=32)),
        retention(3, 24, 40, [0.8, 0.95, 0.999], moe(5, 2, 72, 0.7, shared=16)),
        retention(1, 8, 72, [0.99], None),
    ],
}
ZOZ_C = {
    "architecture": "Zozenex", "vocab": 128, "width": 48, "max_positions": 256, "norm": {"eps": 1e-4},
    "initializer_range": 0.15,
    "layers": [
        parallel(left(6, 3, 8, 8, 0.5, softcap=2.0, size=7, pool=3), right(2, 24, 20, 2.5, rank=8), moe(3, 3, 16, 0.5, shared=8)),
        parallel(left(2, 1, 12, 10, 0.4, size=12, rot=(2, 10.0)), right(1, 16, 16, 3.0), None),
        parallel(left(1, 1, 16, 6, 0.3, rot=(16, 50.0)), right(4, 4, 12, 1.5, rank=3), moe(7, 4, 8, 3.0)),
    ],
}
# sizes that are multiples of nothing convenient: a width of 44, keys of 6 and 10, values of 10 and 14, a vocabulary of 97
ZOZ_D = {
    "architecture": "Zozenex", "vocab": 97, "width": 44, "max_positions": 300, "norm": {"eps": 1e-5},
    "initializer_range": 0.12,
    "layers": [
        retention(3, 6, 10, [0.5, 0.9, 0.99], moe(5, 2, 12, 1.2, shared=20)),
        parallel(left(3, 3, 10, 14, 0.35, softcap=8.0, size=11, pool=4, rot=(6, 20.0)), right(2, 6, 6, 2.0, rank=2),
                 moe(2, 1, 6, 0.9)),
    ],
}
ZOZ = {"A": (ZOZ_A, 16, 3), "B": (ZOZ_B, 8, 4), "C": (ZOZ_C, 4, 5), "D": (ZOZ_D, 4, 6)}   # config, page size, seed


def write_models(tmp_path_factory):
    from tiny_llm_b200.config import ZozenexConfig
    from tiny_llm_b200.weights import write_random_model

    out = {}
    for name, (cfg, _page, seed) in ZOZ.items():
        d = tmp_path_factory.mktemp(f"zoz_{name}")
        write_random_model(str(d), ZozenexConfig.from_dict(cfg), seed=seed, dtype=torch.float32)
        out[name] = str(d)
    return out


def plain_model(model_dir, dtype):
    """Configuration, weights and storage rounding of the plain implementation for one of the engine's two paths."""
    cfg, w = pz.load_config(model_dir), pz.load_weights(model_dir)
    if dtype == "bfloat16":
        w = {k: (v if v.dim() < 2 else v.to(torch.bfloat16).float()) for k, v in w.items()}
    return cfg, w, (pz.no_quant if dtype == "float32" else pz.bf16_quant)


def plain_logits(model_dir, reqs, dtype):
    """What the engine's logits are held against: the plain implementation in 64-bit with the path's weights (rounded
    to bfloat16 for the bfloat16 path) and NO rounding of activations, i.e. the result the path approximates."""
    cfg, w, _ = plain_model(model_dir, dtype)
    return {rid: pz.forward(cfg, w, toks, torch.float64).float() for rid, toks in reqs.items()}


def tolerances(model_dir, reqs, dtype):
    """Per request, how far the engine may be from the plain implementation's 64-bit logits.  32-bit: 2e-5, or four
    times what 32-bit rounding does to the plain implementation itself where that is more.  bfloat16: twice what
    bfloat16 rounding of the activations does to the plain implementation for this very request.  The engine rounds
    at the same places but sums in another order, so its error is another draw of the same size.  (A fault -- a
    wrong key, a lost state, a window edge off by one -- is caught by the 32-bit runs of the same code.)"""
    out = {}
    for rid, toks in reqs.items():
        cfg, w, quant = plain_model(model_dir, dtype)
        f64 = pz.forward(cfg, w, toks, torch.float64)
        if dtype == "float32":
            f32 = pz.forward(cfg, w, toks, torch.float32)
            out[rid] = max(2e-5, 4.0 * float((f32.double() - f64).abs().max()))
        else:
            out[rid] = 2.0 * float((pz.forward(cfg, w, toks, torch.float64, quant=quant) - f64).abs().max())
    return out


def compare(got, ref, prefix, tol, what):
    worst = 0.0
    for rid, r in ref.items():
        g = got[prefix + rid]
        assert g.shape == r.shape, (what, rid, g.shape, r.shape)
        diff = (g - r).abs()
        if not float(diff.max()) <= tol[rid]:
            bad = (~(diff.max(dim=1).values <= tol[rid])).nonzero().flatten()
            raise AssertionError(f"{what}: request {rid} differs from the plain implementation first at position "
                                 f"{int(bad[0])} of {r.shape[0]} (max |diff| {float(diff.max()):.3e}, tolerance "
                                 f"{tol[rid]:.3e}; wrong positions: {bad.tolist()[:20]})")
        worst = max(worst, float(diff.max()) / tol[rid])
    import replay_util
    replay_util.record_margin(what, "", worst)   # printed, and appended to the file TLLM_MARGIN_FILE names
    return worst
