"""A plain, slow implementation of the Safesun decoder, for tests only.

Whole sequences, no cache, one function per mechanism, torch on the CPU in float32 or
float64; it shares no code with ``rocml_b200`` (the model folder is read with the
``safetensors`` package).  Notation: W is stored [out, in] and applied as W x;
rms(x) = x / sqrt(mean(x^2) + eps);  n(x, w) = rms(x) * (1 + w)  (the weight is stored around zero).

    embedding           x = n(E[id], w_e)
    layer               x += mix(n(x, w1)) + ff(n(x, w2))                   (two norms of the same x, side by side)
    attention "a"       q = Wq h, k = Wk h, v = Wv h;  q and k per head: rms * w_q (w_k), plain weight;  then rotation
    attention "b"       q = Wq h + bq, k = Wk h + bk, v = Wv h + bv;  rotation;  then q and k per head: rms, no weight
    rotation            the first `dims` entries of a head, entry i with entry i + dims / 2, by p * f_i, f_i = base^(-2i / dims);
                        with scaling {factor, original, fast, slow}: d(t) = dims ln(original / (2 pi t)) / (2 ln base),
                        lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
                        f_i <- r_i f_i / factor + (1 - r_i) f_i, and cos and sin times 0.1 ln(factor) + 1
    mask                query i sees key j when j <= i and (i - j < size or j < keep_first)
    weights             "a": softmax((q . k) scale);  "b": exp(s_j) / (1 + sum_j exp(s_j))  (one more term of score 0 without a value)
    value mixing        in the layers that say v_mix, except the first of them: v <- (1 - lam) v + lam v_first, v_first the
                        first such layer's v of the same token (what later queries read is the mixed v)
    gate, output        Wo (concat_heads(sum_j a_ij v_j) * sigmoid(Wg h))
    dense ff            Wdown (silu(Wgate h) * (Wup h))
    output              logits = E n(x, w_f)
"""
from __future__ import annotations

import json
import math
import os

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(rot, dtype=torch.float64):
    """(f_i for i < dims / 2, the factor on cos and sin)."""
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        def d(t):
            return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(d(sc["fast"])), 0)
        hi = min(math.ceil(d(sc["slow"])), dims - 1)
        for i in range(dims // 2):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / sc["factor"] * r + f[i] * (1.0 - r)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    return torch.tensor(f, dtype=dtype), mag


def rotate_half(x, positions, rot):
    """x [T, heads, dim]: entries (i, i + dims / 2), i < dims / 2, turned by positions * f_i; the rest unchanged."""
    dims = rot["dims"]
    if dims == 0:
        return x
    f, mag = frequencies(rot, x.dtype)
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    out = x.clone()
    out[..., : dims // 2] = u * c - v * s
    out[..., dims // 2: dims] = v * c + u * s
    return out


def visible(positions, size, keep_first):
    p = torch.as_tensor(positions)
    i, j = p[:, None], p[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def weights_softmax(s, seen):
    return torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1)


def weights_one_more(s, seen):
    """exp(s_j) / (1 + sum exp(s_j)) over the visible keys."""
    s = s.masked_fill(~seen, float("-inf"))
    top = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - top)
    return e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))


def mix_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def attention(h, w, pre, kind, m, eps, v_first=None, positions=None):
    """h [T, D] -> ([T, D], this layer's v before mixing).  ``kind`` is "attention" or "attention_2"; ``m`` the
    layer's mixer dictionary; ``v_first`` None (no mixing in this layer, or it is the first that mixes) or [T, G, vdim]."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = list(range(T)) if positions is None else positions
    q, k, v = h @ w[pre + "q"].t(), h @ w[pre + "k"].t(), h @ w[pre + "v"].t()
    if kind == "attention_2":
        q, k, v = q + w[pre + "q.b"], k + w[pre + "k.b"], v + w[pre + "v.b"]
    q, k, v = q.reshape(T, H, dim), k.reshape(T, G, dim), v.reshape(T, G, vdim)
    rot = m.get("rot") or {"dims": 0}
    if kind == "attention":
        q, k = rms(q, eps) * w[pre + "q.norm"], rms(k, eps) * w[pre + "k.norm"]
        q, k = rotate_half(q, pos, rot), rotate_half(k, pos, rot)
    else:
        q, k = rotate_half(q, pos, rot), rotate_half(k, pos, rot)
        q, k = rms(q, eps), rms(k, eps)
    v_own = v
    if v_first is not None:
        v = mix_values(v, v_first, w[pre + "vmix"])
    mask = m.get("mask") or {"size": T + max(pos) + 1, "keep_first": 0}        # no mask: every earlier key
    seen = visible(pos, mask["size"], mask.get("keep_first", 0))
    out = torch.empty((T, H, vdim), dtype=h.dtype)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].t()) * m["scale"]
        a = weights_softmax(s, seen) if kind == "attention" else weights_one_more(s, seen)
        out[:, n] = a @ v[:, g]
    gate = torch.sigmoid(h @ w[pre + "g"].t())
    return (out.reshape(T, H * vdim) * gate) @ w[pre + "o"].t(), v_own


def dense_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].t()) * (h @ w[pre + "up"].t())) @ w[pre + "down"].t()


def load(folder, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = norm_one_plus(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], eps)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        mixes = bool(L["mixer"].get("v_mix"))
        y, v_own = attention(norm_one_plus(x, w[pre + "norm1"], eps), w, pre + "mix.", L["type"], L["mixer"], eps,
                             v_first if mixes else None)
        if mixes and v_first is None:
            v_first = v_own
        if L.get("mlp") is not None:
            y = y + dense_ff(norm_one_plus(x, w[pre + "norm2"], eps), w, pre + "mlp.")
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, w["final.norm"], eps) @ w["embed"].t()
