"""A plain, slow implementation of the Tibenex decoder, for tests only.

Whole sequences, no cache, one function per mechanism, torch on the CPU in float32 or float64; it shares
no code with ``rocml_b200`` (the model folder is read with the ``safetensors`` package).  Notation: W is
stored [out, in] and applied as W x;  rms(x) = x / sqrt(mean(x^2) + eps);  n(x, w) = rms(x) * w.

    embedding          x = E[id] * s_e
    layer              h = x + (x_prev - x) * mu   (x_prev: the token before, zeros at the start)
                       x <- n(alpha x + g1 * mix(h), w1);   x <- n(alpha x + g2 * ff(x), w2)
    latent attention   cq = n(Wdq h, w_q), q = Wuq cq  (per head: `dim` plain entries, then `rot_dim` rotated)
                       [c | kr] = Wdkv h,  c <- n(c, w_c);  k_h = Wuk_h c,  v_h = Wuv_h c;  kr is shared by all heads
                       s_ij = (q_plain . k + rot(q_rot, i) . rot(kr, j)) * scale;  rotate-half pairs, frequencies along a ramp
                       o_h = sigmoid(Wg h)_h * sum_j softmax_j(s_ij) v_j;  out = Wo concat(o)
    attention          q, k, v = W. h;  q <- n(q, w_qn) and k <- n(k, w_kn) over the WHOLE projection;  neighbouring pairs
                       (2i, 2i + 1) of the first `dims` entries of every head turn;  s = (q . k) * scale * temp_h;
                       a = softmax;  a'_h = sum_g T[h, g] a_g;  o_h = sum_j a'_h v_(kv head of h);  out = Wo concat(o)
    mamba2             [z | x | B | C | dt] = Win h;  x, B, C <- silu(causal conv + bias);  dt <- softplus(dt + dt_bias)
                       S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T;  y_t = S_t^T C_t + D x_t
                       out = Wo (n_parts(y * silu(z)) * w)     (the rows normalised in `norm_groups` equal parts)
    dense ff           Wdown (silu(Wgate h) * (Wup h))
    output             logits = Whead n(x, w_f)
"""
from __future__ import annotations

import json
import math
import os

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def token_shift(x, mu, before=None):
    """x [T, D]: x_t + (x_(t-1) - x_t) * mu; ``before`` is the row ahead of the first (zeros when None)."""
    first = torch.zeros_like(x[:1]) if before is None else before.reshape(1, -1).to(x.dtype)
    prev = torch.cat([first, x[:-1]], dim=0)
    return x + (prev - x) * mu


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


def rotate(x, positions, rot, pairs):
    """x [T, heads, dim]: the first `dims` entries turn by positions * f_i; ``pairs`` "half": entry i with entry
    i + dims / 2; "neighbours": entry 2i with entry 2i + 1.  The rest passes unchanged."""
    dims = rot["dims"]
    if dims == 0:
        return x
    f, mag = frequencies(rot, x.dtype)
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    if pairs == "half":
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * c - v * s
        out[..., dims // 2: dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def causal_softmax(scores, positions):
    """scores [heads, T, T] -> weights; query i sees key j when position j <= position i."""
    p = torch.as_tensor(positions)
    seen = p[None, :] <= p[:, None]
    return torch.softmax(scores.masked_fill(~seen[None], float("-inf")), dim=-1)


def latent_attention(h, positions, m, w, eps):
    """m: the mixer's sizes; w: its tensors by short name."""
    T = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = dict(m.get("rot") or {"base": 10000.0}, dims=rd)
    cq = norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, dim + rd)
    dkv = h @ w["dkv"].T
    c = norm(dkv[:, :rank], w["dkv.norm"], eps)
    kr = rotate(dkv[:, None, rank:], positions, rot, "half")              # [T, 1, rd], one for all heads
    qr = rotate(q[..., dim:], positions, rot, "half")
    k = (c @ w["uk"].T).reshape(T, H, dim)
    v = (c @ w["uv"].T).reshape(T, H, vd)
    s = (torch.einsum("ihd,jhd->hij", q[..., :dim], k) + torch.einsum("ihd,jd->hij", qr, kr[:, 0])) * m["scale"]
    a = causal_softmax(s, positions)
    o = torch.einsum("hij,jhd->ihd", a, v)
    o = o * torch.sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * vd) @ w["o"].T


def attention(h, positions, m, w, eps):
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = norm(h @ w["q"].T, w["q.norm"], eps).reshape(T, H, dim)
    k = norm(h @ w["k"].T, w["k.norm"], eps).reshape(T, G, dim)
    v = (h @ w["v"].T).reshape(T, G, vd)
    if m.get("rot") is not None:
        q = rotate(q, positions, m["rot"], "neighbours")
        k = rotate(k, positions, m["rot"], "neighbours")
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"] * w["temp"].reshape(H, 1, 1)
    a = causal_softmax(s, positions)
    a = torch.einsum("hg,gij->hij", w["talk"], a)
    o = torch.einsum("hij,jhd->ihd", a, v[:, kv_of])
    return o.reshape(T, H * vd) @ w["o"].T


def causal_conv(u, taps_w, bias, before=None):
    """u [T, C]; taps_w [C, taps], the last column multiplies the current token; zeros (or ``before``
    [taps - 1, C]) ahead of the first token."""
    taps = taps_w.shape[1]
    first = torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype) if before is None else before.to(u.dtype)
    padded = torch.cat([first, u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + padded[j: j + u.shape[0]] * taps_w[:, j]
    return out + bias


def mamba2(h, m, w, eps, state=None, conv_before=None, return_state=False):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zxbcdt = h @ w["in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner: 2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc_act = silu(causal_conv(xbc, w["conv"], w["conv.b"], conv_before))
    x = xbc_act[:, :inner].reshape(T, H, P)
    B = xbc_act[:, inner: inner + G * N].reshape(T, G, N)
    C = xbc_act[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)                       # [T, H]
    group_of = torch.arange(H) // (H // G)
    S = torch.zeros((H, N, P), dtype=h.dtype) if state is None else state.clone()
    y = torch.zeros((T, H, P), dtype=h.dtype)
    for t in range(T):
        Bt, Ct = B[t, group_of], C[t, group_of]                          # [H, N]
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ct) + w["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    out = y @ w["o"].T
    if return_state:
        return out, S, torch.cat([torch.zeros((w["conv"].shape[1] - 1, xbc.shape[1]), dtype=h.dtype) if conv_before is None
                                  else conv_before.to(h.dtype), xbc], dim=0)[-(w["conv"].shape[1] - 1):]
    return out


def dense_ff(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer(x, positions, cfg, i, tensors):
    """One layer on a whole sequence x [T, D]."""
    L = cfg["layers"][i]
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    p = f"l{i}."
    h = token_shift(x, tensors[p + "shift"])
    w = sub(tensors, p + "mix.")
    if L["type"] == "latent_attention":
        y = latent_attention(h, positions, L["mixer"], w, eps)
    elif L["type"] == "attention":
        y = attention(h, positions, L["mixer"], w, eps)
    elif L["type"] == "mamba2":
        y = mamba2(h, L["mixer"], w, eps)
    else:
        raise ValueError(L["type"])
    x = norm(alpha * x + y * tensors[p + "ls1"], tensors[p + "norm1"], eps)
    if L.get("mlp") is not None:
        y = dense_ff(x, sub(tensors, p + "mlp."))
        x = norm(alpha * x + y * tensors[p + "ls2"], tensors[p + "norm2"], eps)
    return x


def forward(cfg, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out``: a list that receives the stream after every layer."""
    x = tensors["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    positions = list(range(len(tokens)))
    for i in range(len(cfg["layers"])):
        x = layer(x, positions, cfg, i, tensors)
        if layers_out is not None:
            layers_out.append(x)
    return norm(x, tensors["final.norm"], cfg["norm"]["eps"]) @ tensors["head"].T


def load_folder(folder, dtype=torch.float64):
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            tensors[k] = t.to(dtype) if t.is_floating_point() else t
    return cfg, tensors
