"""Plain, slow Dunelix decoder for the tests: whole sequences, no cache, one function per mechanism.

Written from the design's equations with plain torch arithmetic on the CPU; it shares no code with the
`tiny_llm_b200` package (config.json is read with `json`, weights with the `safetensors` library).

Notation.  x[t, :] is the residual stream of token t (positions count from 0), m the residual
multiplier.  A layer is  x += m * mixer(dyt1(x));  x += m * ffn(dyt2(x))  (the second line only when the
layer has a feed-forward).  Layers `start .. stop-1` of the loop run `times` times in a row with the same
weights, every pass with a state of its own; before each pass but the first the embedding output is added
to x.  The model ends with a Dynamic Tanh and the output matrix.

`quant` is the storage rounding of the path that is being checked: the identity for the 32-bit path; for
the bfloat16 path a round-trip through bfloat16 where that path stores bfloat16 (norm outputs, projection
outputs, activations), while norms, rotation, scores, softmax, the recurrence and the residual stay in
32-bit (or in `dtype`, when the caller asks for 64-bit).
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

Quant = Callable[[torch.Tensor], torch.Tensor]


def no_quant(x: torch.Tensor) -> torch.Tensor:
    return x


def bf16_quant(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def load_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def load_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            out[k] = t.to(dtype) if t.is_floating_point() else t
    return out


# ----------------------------------------------------------------------------- mechanisms


def dynamic_tanh(x, weight, bias, alpha):
    """y = tanh(alpha * x) * w + b: no mean, no variance."""
    return torch.tanh(alpha * x) * weight + bias


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def min_gru_candidate(u):
    """u + 1/2 where u >= 0, sigmoid(u) where u < 0."""
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def min_gru_scan(z, cand, state=None):
    """S_t = (1 - z_t) S_(t-1) + z_t cand_t, element by element, from S_(-1) = state (zero when None).
    Returns all S_t [T, W] and the last one."""
    t, w = z.shape
    s = torch.zeros(w, dtype=z.dtype) if state is None else state.clone()
    out = torch.empty_like(z)
    for i in range(t):
        s = (1.0 - z[i]) * s + z[i] * cand[i]
        out[i] = s
    return out, s


def min_gru(h, wz, bz, wx, bx, wg, wo, quant: Quant = no_quant, state=None):
    """Gates read the current token only: z = sigmoid(Wz h + bz), u = Wx h + bx; output Wo (S_t * silu(Wg h))."""
    zl = quant(h @ wz.T)
    ul = quant(h @ wx.T)
    gl = quant(h @ wg.T)
    z = torch.sigmoid(zl + bz)
    cand = min_gru_candidate(ul + bx)
    s_all, s_last = min_gru_scan(z, cand, state)
    y = quant(s_all * silu(gl))
    return y @ wo.T, s_last


def scaled_frequencies(dims: int, base: float, scaling: Optional[dict], dtype=torch.float32):
    """f_i = base^(-2i/dims); wavelengths l = 2 pi / f shorter than original/high keep f, longer than
    original/low use f / factor, between them the two are blended by s = (original/l - low) / (high - low)."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = torch.pow(torch.tensor(base, dtype=dtype), -2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    wave = 2.0 * math.pi / f
    s = (orig / wave - low) / (high - low)
    blended = (1.0 - s) * f / factor + s * f
    out = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, blended))
    return out


def rotate_interleaved(x, positions, freqs):
    """x [T, heads, d]; the first 2*len(freqs) values of every head are rotated, pair (2i, 2i+1) by the angle
    p * f_i; the rest pass unchanged."""
    n = freqs.numel()
    ang = positions.to(freqs.dtype)[:, None] * freqs[None, :]          # [T, n]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


def chunk_mask(q_pos, k_pos, size: int):
    """True where key j is visible to query i: j <= i and both in the same chunk of `size` positions."""
    i, j = q_pos[:, None], k_pos[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def softmax_attention(q, k, v, mask, scale: float):
    """q [Tq, d], k [Tk, d], v [Tk, dv], mask [Tq, Tk] -> [Tq, dv]."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def differential_lambda(lq1, lk1, lq2, lk2, diff: float):
    return torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + diff


def differential_attention(h, positions, p: dict, wq, wk, wv, wo, lq1, lk1, lq2, lk2, eps: float,
                           quant: Quant = no_quant, k_past=None, v_past=None, past_positions=None):
    """Two softmax maps per head over the same values, o = a1 - lambda a2, o / rms(o) * (1 - diff)."""
    t = h.shape[0]
    heads, kvh, d, dv = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = quant(h @ wq.T).view(t, heads * 2, d)          # head by head [map 1, map 2]
    k = quant(h @ wk.T).view(t, kvh * 2, d)
    v = quant(h @ wv.T).view(t, kvh, dv)
    rot = p.get("rot")
    if rot:
        f = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"), dtype=torch.float32).to(h.dtype) \
            if h.dtype == torch.float32 else scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"), dtype=h.dtype)
        q = quant(rotate_interleaved(q, positions, f))
        k = quant(rotate_interleaved(k, positions, f))
    k_pos = positions
    if k_past is not None:
        k, v, k_pos = torch.cat([k_past, k]), torch.cat([v_past, v]), torch.cat([past_positions, positions])
    size = p["mask"]["size"] if p.get("mask") else None
    if size is None:
        mask = k_pos[None, :] <= positions[:, None]
    else:
        mask = chunk_mask(positions, k_pos, size)
    lam = differential_lambda(lq1, lk1, lq2, lk2, p["diff"])
    group = heads // kvh
    out = torch.empty(t, heads, dv, dtype=h.dtype)
    for hd in range(heads):
        g = hd // group
        a1 = softmax_attention(q[:, 2 * hd], k[:, 2 * g], v[:, g], mask, p["scale"])
        a2 = softmax_attention(q[:, 2 * hd + 1], k[:, 2 * g + 1], v[:, g], mask, p["scale"])
        o = a1 - lam * a2
        o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)
        out[:, hd] = o * (1.0 - p["diff"])
    y = quant(out.reshape(t, heads * dv))
    return y @ wo.T, k, v


def gated_ffn(h, wg, wu, wd, quant: Quant = no_quant):
    return quant(silu(h @ wg.T) * (h @ wu.T)) @ wd.T


# ----------------------------------------------------------------------------- the model


def run_order(cfg: dict) -> List[tuple]:
    """(layer, first of a later pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, False) for i in range(a)]
    for rep in range(times):
        out += [(i, rep > 0 and i == a) for i in range(a, b)]
    return out + [(i, False) for i in range(b, n)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, quant: Quant = no_quant, dtype=torch.float32,
            return_layers: bool = False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    tok = torch.as_tensor(tokens, dtype=torch.long)
    t = tok.numel()
    pos = torch.arange(t)
    m = float(cfg["residual_mult"])
    eps = float(cfg["norm"]["eps"])
    emb = w["embed"][tok]
    x = emb.clone()
    streams = []

    def norm(name, x):
        return quant(dynamic_tanh(x, w[name], w[name + ".b"], w[name + ".alpha"]))

    for layer, reinject in run_order(cfg):
        spec = cfg["layers"][layer]
        pre = f"l{layer}."
        if reinject:
            x = x + emb
        h = norm(pre + "norm1", x)
        mx = pre + "mix."
        if spec["type"] == "mingru":
            y, _ = min_gru(h, w[mx + "z"], w[mx + "z.b"], w[mx + "x"], w[mx + "x.b"], w[mx + "g"], w[mx + "o"], quant)
        elif spec["type"] == "attention":
            y, _, _ = differential_attention(h, pos, spec["mixer"], w[mx + "q"], w[mx + "k"], w[mx + "v"], w[mx + "o"],
                                             w[mx + "lq1"], w[mx + "lk1"], w[mx + "lq2"], w[mx + "lk2"], eps, quant)
        else:
            raise ValueError(f"unknown mixer {spec['type']!r}")
        x = x + m * y
        if spec.get("mlp"):
            if spec["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward {spec['mlp']['kind']!r}")
            f = pre + "mlp."
            x = x + m * gated_ffn(norm(pre + "norm2", x), w[f + "gate"], w[f + "up"], w[f + "down"], quant)
        streams.append(x.clone())
    logits = norm("final.norm", x) @ w["head"].T
    if return_layers:
        return logits, torch.stack(streams)
    return logits
