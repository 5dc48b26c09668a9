"""A plain, slow implementation of the Zozenex decoder, one function per mechanism, written from the design's
equations and sharing no code with the package.  Everything is torch on the CPU in the dtype of the weights it
is handed (float64 for an oracle); sequences are walked token by token where the design has a recurrence.

The design.  x = embed[token] + pos[p].  Every layer: x += mixer(rms(x) w1); x += ff(rms(x) w2) (no ff when the layer
has none).  Mixers:
  retention  S_t = d_h S_(t-1) + (k_t / sqrt(dim)) v_t^T, o_t = S_t^T q_t per head with a fixed decay d_h; o / rms(o)
             per head, times silu(Wg h), times Wo.
  parallel   (L + R) / 2 with L = rms(left(h)) w_left_out, R = rms(right(h)) w_right_out over the model width.
    left     attention without softmax: weight of a visible key = sigmoid(cap * tanh(q.k scale / cap) + pb_h); queries
             and keys rotated (halves layout) on their first rot dims, values rotated over their whole size and the
             head's output turned back by the query's position; visible: the last `size` tokens, and one mean key / mean
             value for every block of `pool` tokens that lies wholly before that window.
    right    gated linear attention: S_t = diag(a_t) S_(t-1) + k_t v_t^T with a_t = sigmoid(Wa2 Wa1 h + b)^(1/tau) per
             key channel, o_t = S_t^T (q_t / sqrt(dim)); rms(o) * w_norm per head, times silu(Wg h), times Wo.
Feed-forward: experts W_down gelu(W_up h) chosen by the largest sigmoid(router) + correction, weighted by the sigmoid
times a constant, plus a shared expert times sigmoid(w_sg . h)."""
from __future__ import annotations

import json
import math
import os

import torch


def no_quant(x):
    return x


def bf16_quant(x):
    """Rounds to bfloat16 and back: what the engine's bfloat16 path does to an activation it stores."""
    return x.to(torch.bfloat16).to(x.dtype)


def load_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def load_weights(model_dir):
    """Reads model.safetensors with this file's own reader: 8 bytes of length, a JSON header, raw little-endian data."""
    import numpy as np
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = bytes(data[lo:hi])
        if info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif info["dtype"] == "BF16":
            t = (torch.from_numpy(np.frombuffer(raw, dtype="<u2").astype(np.int32).copy()) << 16).view(torch.float32)
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(info["dtype"])
        out[name] = t.reshape(info["shape"])
    return out


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def rotate_halves(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float, sign: float = 1.0) -> torch.Tensor:
    """x [T, rows, D]; the first `dims` values of every row are rotated: value i with value i + dims/2 by the angle
    sign * pos * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    f = torch.pow(torch.tensor(base, dtype=x.dtype), -2.0 * i / dims)
    a = sign * pos.to(x.dtype)[:, None, None] * f[None, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def linear_recurrence(q, k, v, a, s0=None):
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head.  q, k [T, heads, dim], v [T, heads, vdim];
    a [T, heads, dim] (a decay per key channel and token) or [heads] (one per head); s0 [heads, dim, vdim] or None.
    Returns o [T, heads, vdim] and the last state."""
    t, heads, dim = q.shape
    vdim = v.shape[-1]
    s = torch.zeros(heads, dim, vdim, dtype=q.dtype) if s0 is None else s0.clone().to(q.dtype)
    out = torch.zeros(t, heads, vdim, dtype=q.dtype)
    for i in range(t):
        for hd in range(heads):
            decay = a[hd] if a.dim() == 1 else a[i, hd][:, None]
            s[hd] = decay * s[hd] + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s[hd].T @ q[i, hd]
    return out, s


def gate_decay(z, tau):
    """sigmoid(z)^(1/tau)."""
    return torch.pow(torch.sigmoid(z), 1.0 / float(tau))


def retention(h, w, p, m, eps, quant=no_quant):
    """h [T, W]; w(name) gives the mixer's tensors; m the mixer's config."""
    t = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = quant(h @ w(p + "q").T).view(t, heads, dim)
    k = quant(h @ w(p + "k").T).view(t, heads, dim) * dim ** -0.5
    v = quant(h @ w(p + "v").T).view(t, heads, vdim)
    g = quant(h @ w(p + "g").T)
    out, _ = linear_recurrence(q, k, v, torch.tensor([float(d) for d in m["decay"]], dtype=h.dtype))
    out = quant(rms_unit(out, eps).reshape(t, heads * vdim) * silu(g))
    return out @ w(p + "o").T


def gated_linear_attention(h, w, p, m, eps, quant=no_quant):
    t = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = quant(h @ w(p + "q").T).view(t, heads, dim) * dim ** -0.5
    k = quant(h @ w(p + "k").T).view(t, heads, dim)
    v = quant(h @ w(p + "v").T).view(t, heads, vdim)
    g = quant(h @ w(p + "g").T)
    z = quant(h @ w(p + "a1").T) @ w(p + "a2").T + w(p + "a2.b")
    out, _ = linear_recurrence(q, k, v, gate_decay(z, m["tau"]).view(t, heads, dim))
    out = quant((rms_unit(out, eps) * w(p + "norm")).reshape(t, heads * vdim) * silu(g))
    return out @ w(p + "o").T


def visible_blocks(i, size, pool):
    """How many pooled blocks position i sees: block b iff b pool + pool - 1 <= i - size."""
    b = 0
    while b * pool + pool - 1 <= i - size:
        b += 1
    return b


def window_pool_sum(q, k, v, scale, cap, pb, size, pool, quant=no_quant, first=0):
    """q [n, heads, dim] are the queries of positions first .. first + n - 1; k [T, kvh, dim], v [T, kvh, vdim] the
    keys and values of positions 0 .. T - 1 as the cache holds them.  out[i, h] = sum over the visible keys of
    sigmoid(cap tanh(q.k scale / cap) + pb_h) value: the tokens of the window, and the mean key / mean value of
    every block that lies wholly before it."""
    n, heads, _ = q.shape
    kvh, vdim = k.shape[1], v.shape[-1]
    out = torch.zeros(n, heads, vdim, dtype=q.dtype)
    for x in range(n):
        i = first + x
        lo = 0 if size is None else max(0, i - size + 1)
        keys, vals = [k[lo:i + 1]], [v[lo:i + 1]]
        if size is not None and pool:
            for b in range(visible_blocks(i, size, pool)):
                keys.append(quant(k[b * pool:(b + 1) * pool].mean(dim=0, keepdim=True)))
                vals.append(quant(v[b * pool:(b + 1) * pool].mean(dim=0, keepdim=True)))
        kk, vv = torch.cat(keys), torch.cat(vals)          # [n, kvh, *]
        for hd in range(heads):
            kv = hd // (heads // kvh)
            s = (kk[:, kv] @ q[x, hd]) * float(scale)
            if cap:
                s = cap * torch.tanh(s / cap)
            out[x, hd] = torch.sigmoid(s + pb[hd]) @ vv[:, kv]
    return out


def pooled_window_attention(h, w, p, m, quant=no_quant):
    t = h.shape[0]
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    rot = m.get("rot") or {}
    rd, base = rot.get("dims", 0), float(rot.get("base", 10000.0))
    q = quant(rotate_halves(quant(h @ w(p + "q").T).view(t, heads, dim), pos, rd, base))
    k = quant(rotate_halves(quant(h @ w(p + "k").T).view(t, kvh, dim), pos, rd, base))
    v = quant(h @ w(p + "v").T).view(t, kvh, vdim)
    if rot:
        v = quant(rotate_halves(v, pos, vdim, base))
    mask = m.get("mask") or {}
    out = window_pool_sum(q, k, v, m["scale"], m.get("softcap"), w(p + "pb"), mask.get("size"), mask.get("pool"), quant)
    if rot:
        out = rotate_halves(out, pos, vdim, base, sign=-1.0)
    return quant(out.reshape(t, heads * vdim)) @ w(p + "o").T


def parallel(h, w, p, m, eps, quant=no_quant):
    left = pooled_window_attention(h, w, p + "left.", m["left"], quant)
    right = gated_linear_attention(h, w, p + "right.", m["right"], eps, quant)
    return 0.5 * (rms_norm(left, w(p + "left.out"), eps) + rms_norm(right, w(p + "right.out"), eps))


def route(logits, correction, top, scale):
    """Chosen experts [T, top] (largest sigmoid(logit) + correction first) and their weights sigmoid(logit) * scale."""
    s = torch.sigmoid(logits)
    idx = torch.topk(s + correction, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx) * float(scale)


def moe(h, w, p, mlp, quant=no_quant):
    r = mlp["router"]
    n, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w(p + "router").T)                # [T, n]
    idx, _ = route(h @ w(p + "router").T, w(p + "correction"), top, r["scale"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e in idx[i].tolist():
            y = w(p + f"e{e}.down") @ quant(gelu_erf(w(p + f"e{e}.up") @ h[i]))
            out[i] += s[i, e] * float(r["scale"]) * y
    if mlp.get("shared") is not None:
        y = quant(gelu_erf(quant(h @ w(p + "shared.up").T))) @ w(p + "shared.down").T
        out += torch.sigmoid(h @ w(p + "shared.sg").T) * y
    return out


def forward(config: dict, weights: dict, tokens, dtype=torch.float64, layers_out=None, quant=no_quant):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out`: a list that receives the stream after
    every layer.  `quant`: applied wherever the engine stores an activation in its own dtype."""
    def w(name):
        return weights[name].to(dtype)
    eps = float(config["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = w("embed")[tok] + w("pos")[: len(tok)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = quant(rms_norm(x, w(p + "norm1"), eps))
        if layer["type"] == "retention":
            x = x + retention(h, w, p + "mix.", layer["mixer"], eps, quant)
        elif layer["type"] == "parallel":
            x = x + parallel(h, w, p + "mix.", layer["mixer"], eps, quant)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + moe(quant(rms_norm(x, w(p + "norm2"), eps)), w, p + "mlp.", layer["mlp"], quant)
        if layers_out is not None:
            layers_out.append(x.clone())
    return quant(rms_norm(x, w("final.norm"), eps)) @ w("head").T
