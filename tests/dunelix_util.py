"""Tiny Dunelix configurations for the tests and the plain implementation's logits for them.

The configurations differ from one another in every size and option: widths, heads and grouping, key size against
value size (equal to twice the key size in none of them), chunk sizes that are and are not multiples of the page
size, rotation over part of the key / the whole key / none, frequency scaling on and off, a layer without a
feed-forward, a residual multiplier that is and is not 1, a looped span at the front, in the middle, and none."""
import torch

import plain_dunelix as pd


def attention(heads, kv, dim, vdim, scale, diff, mask=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if mask:
        m["mask"] = {"size": mask}
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


DUNE_A = {
    "architecture": "Dunelix", "vocab": 200, "width": 64, "residual_mult": 0.5, "norm": {"eps": 1e-5},
    "initializer_range": 0.1,
    "layers": [
        with_mlp(gru(96), 80),
        with_mlp(attention(4, 2, 16, 40, 0.3, 0.3, mask=24,
                           rot={"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}), 72),
        with_mlp(gru(48), None),
        with_mlp(attention(2, 2, 32, 24, 0.2, 0.7), 64),
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}
DUNE_B = {
    "architecture": "Dunelix", "vocab": 331, "width": 96, "residual_mult": 1.0, "norm": {"eps": 1e-6},
    "initializer_range": 0.08,
    "layers": [
        with_mlp(attention(3, 1, 32, 48, 0.3, 0.5, mask=64, rot={"dims": 32, "base": 5000.0}), 136),   # sizes the tensor-core kernel takes
        with_mlp(gru(128), 104),
        with_mlp(gru(72), 88),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
DUNE_C = {
    "architecture": "Dunelix", "vocab": 128, "width": 48, "residual_mult": 0.8, "norm": {"eps": 1e-4},
    "initializer_range": 0.15,
    "layers": [
        with_mlp(attention(6, 3, 8, 8, 0.5, 0.2, mask=7, rot={"dims": 2, "base": 10.0}), None),
        with_mlp(gru(40), 56),
    ],
}
DUNE = {"A": (DUNE_A, 16, 3), "B": (DUNE_B, 8, 4), "C": (DUNE_C, 4, 5)}   # config, page size, seed


def write_models(tmp_path_factory):
    from tiny_llm_b200.config import DunelixConfig
    from tiny_llm_b200.weights import write_random_model

    out = {}
    for name, (cfg, _page, seed) in DUNE.items():
        d = tmp_path_factory.mktemp(f"dune_{name}")
        write_random_model(str(d), DunelixConfig.from_dict(cfg), seed=seed, dtype=torch.float32)
        out[name] = str(d)
    return out


def plain_model(model_dir, dtype):
    """Configuration, weights and storage rounding of the plain implementation for one of the engine's two paths."""
    cfg, w = pd.load_config(model_dir), pd.load_weights(model_dir)
    if dtype == "bfloat16":
        w = {k: (v if v.dim() < 2 else v.to(torch.bfloat16).float()) for k, v in w.items()}
    return cfg, w, (pd.no_quant if dtype == "float32" else pd.bf16_quant)


def plain_logits(model_dir, reqs, dtype):
    """What the engine's logits are held against: the plain implementation with the path's weights (rounded to
    bfloat16 for the bfloat16 path) and NO rounding of activations, i.e. the result the path approximates."""
    cfg, w, _ = plain_model(model_dir, dtype)
    return {rid: pd.forward(cfg, w, toks) for rid, toks in reqs.items()}


def tolerances(model_dir, reqs, dtype):
    """Per request, how far the engine may be from the plain implementation's logits in the path's precision.
    32-bit: 2e-5, or four times what 32-bit rounding does to the plain implementation itself (its distance from its
    own 64-bit run) where that is more.  bfloat16: twice what bfloat16 rounding of the activations does to the plain
    implementation for this very request, 2 max |plain(bfloat16 roundings) - plain(no rounding)|.  The engine rounds
    at the same places but sums in another order, so its error is another draw of the same size; the largest of
    one draw over all positions and logits can exceed the largest of another, hence the factor.  (A fault -- a wrong
    key, a lost state, a chunk edge off by one -- is caught by the 32-bit runs of the same code at 2e-5.)"""
    cfg, w, _ = plain_model(model_dir, "float32")
    out = {}
    for rid, toks in reqs.items():
        f32 = pd.forward(cfg, w, toks)
        if dtype == "float32":
            f64 = pd.forward(cfg, w, toks, dtype=torch.float64)
            out[rid] = max(2e-5, 4.0 * float((f32.double() - f64).abs().max()))
        else:
            cb, wb, quant = plain_model(model_dir, "bfloat16")
            out[rid] = 2.0 * float((pd.forward(cb, wb, toks, quant=quant) - pd.forward(cb, wb, toks)).abs().max())
    return out


def compare(got, ref, prefix, tol, what):
    worst = 0.0
    for rid, r in ref.items():
        g = got[prefix + rid]
        assert g.shape == r.shape, (what, rid, g.shape, r.shape)
        diff = (g - r).abs()
        if float(diff.max()) > tol[rid]:
            bad = (diff.max(dim=1).values > tol[rid]).nonzero().flatten()
            raise AssertionError(f"{what}: request {rid} differs from the plain implementation first at position "
                                 f"{int(bad[0])} of {r.shape[0]} (max |diff| {float(diff.max()):.3e}, tolerance "
                                 f"{tol[rid]:.3e}; wrong positions: {bad.tolist()[:20]})")
        worst = max(worst, float(diff.max()) / tol[rid])
    import replay_util
    replay_util.record_margin(what, "", worst)   # printed, and appended to the file TLLM_MARGIN_FILE names
    return worst
