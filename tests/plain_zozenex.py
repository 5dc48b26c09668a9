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

import math

import torch


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


def retention(h, w, p, m, eps):
    """h [T, W]; w(name) gives the mixer's tensors; m the mixer's config."""
    t = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = (h @ w(p + "q").T).view(t, heads, dim)
    k = (h @ w(p + "k").T).view(t, heads, dim) * dim ** -0.5
    v = (h @ w(p + "v").T).view(t, heads, vdim)
    g = h @ w(p + "g").T
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for hd in range(heads):
        s = torch.zeros(dim, vdim, dtype=h.dtype)
        d = float(m["decay"][hd])
        for i in range(t):
            s = d * s + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s.T @ q[i, hd]
    out = rms_unit(out, eps).reshape(t, heads * vdim) * silu(g)
    return out @ w(p + "o").T


def gated_linear_attention(h, w, p, m, eps):
    t = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = (h @ w(p + "q").T).view(t, heads, dim) * dim ** -0.5
    k = (h @ w(p + "k").T).view(t, heads, dim)
    v = (h @ w(p + "v").T).view(t, heads, vdim)
    g = h @ w(p + "g").T
    z = (h @ w(p + "a1").T) @ w(p + "a2").T + w(p + "a2.b")
    alpha = torch.pow(torch.sigmoid(z), 1.0 / float(m["tau"])).view(t, heads, dim)
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for hd in range(heads):
        s = torch.zeros(dim, vdim, dtype=h.dtype)
        for i in range(t):
            s = alpha[i, hd][:, None] * s + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s.T @ q[i, hd]
    out = (rms_unit(out, eps) * w(p + "norm")).reshape(t, heads * vdim) * silu(g)
    return out @ w(p + "o").T


def pooled_window_attention(h, w, p, m):
    t = h.shape[0]
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    rot = m.get("rot") or {}
    rd, base = rot.get("dims", 0), float(rot.get("base", 10000.0))
    q = rotate_halves((h @ w(p + "q").T).view(t, heads, dim), pos, rd, base)
    k = rotate_halves((h @ w(p + "k").T).view(t, kvh, dim), pos, rd, base)
    v = (h @ w(p + "v").T).view(t, kvh, vdim)
    if rot:
        v = rotate_halves(v, pos, vdim, base)
    mask = m.get("mask") or {}
    size, pool = mask.get("size"), mask.get("pool")
    cap = m.get("softcap")
    pb = w(p + "pb")
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for i in range(t):
        lo = 0 if size is None else max(0, i - size + 1)
        keys, vals = [k[lo:i + 1]], [v[lo:i + 1]]
        if size is not None and pool:
            b = 0
            while b * pool + pool - 1 <= i - size:
                keys.append(k[b * pool:(b + 1) * pool].mean(dim=0, keepdim=True))
                vals.append(v[b * pool:(b + 1) * pool].mean(dim=0, keepdim=True))
                b += 1
        kk, vv = torch.cat(keys), torch.cat(vals)          # [n, kvh, *]
        for hd in range(heads):
            kv = hd // (heads // kvh)
            s = (kk[:, kv] @ q[i, hd]) * float(m["scale"])
            if cap:
                s = cap * torch.tanh(s / cap)
            out[i, hd] = torch.sigmoid(s + pb[hd]) @ vv[:, kv]
    if rot:
        out = rotate_halves(out, pos, vdim, base, sign=-1.0)
    return out.reshape(t, heads * vdim) @ w(p + "o").T


def parallel(h, w, p, m, eps):
    left = pooled_window_attention(h, w, p + "left.", m["left"])
    right = gated_linear_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w(p + "left.out"), eps) + rms_norm(right, w(p + "right.out"), eps))


def moe(h, w, p, mlp):
    r = mlp["router"]
    n, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w(p + "router").T)                # [T, n]
    choice = s + w(p + "correction")
    idx = torch.topk(choice, top, dim=-1).indices
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e in idx[i].tolist():
            y = w(p + f"e{e}.down") @ gelu_erf(w(p + f"e{e}.up") @ h[i])
            out[i] += s[i, e] * float(r["scale"]) * y
    if mlp.get("shared") is not None:
        y = gelu_erf(h @ w(p + "shared.up").T) @ w(p + "shared.down").T
        out += torch.sigmoid(h @ w(p + "shared.sg").T) * y
    return out


def forward(config: dict, weights: dict, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out`: a list that receives the stream after
    every layer."""
    def w(name):
        return weights[name].to(dtype)
    eps = float(config["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = w("embed")[tok] + w("pos")[: len(tok)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w(p + "norm1"), eps)
        if layer["type"] == "retention":
            x = x + retention(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + moe(rms_norm(x, w(p + "norm2"), eps), w, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w("final.norm"), eps) @ w("head").T
