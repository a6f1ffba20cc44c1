"""Safesun on the GPU against the plain implementation (tests/plain_safesun.py): each mechanism alone, then the
engine in every way of cutting and batching, in 32-bit and in bfloat16.

Tolerances are a fraction of the largest |logit| of the row compared.  float32: sums of a few hundred terms in
another order than the plain implementation's float64.  bfloat16: activations are rounded to 8 bits of mantissa
between kernels, a dozen roundings a layer.
"""
import json
import math

import pytest
import torch

import plain_safesun as P
from tiny_models import SAFESUN, prompt, write_model, write_safesun

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 3e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"


def rel_err(got, want):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


def close(got, want, tol):
    want = want.double()
    got = got.double().cpu()
    return float((got - want).abs().max()) <= tol * max(1e-30, float(want.abs().max()))


# ---- each mechanism alone -------------------------------------------------------------------------------------

@pytest.mark.parametrize("rot", [
    {"base": 10000.0, "dims": 16},
    {"base": 1e6, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
    {"base": 500.0, "dims": 32, "scaling": {"factor": 3.0, "original": 40, "fast": 4.0, "slow": 0.5}},
    {"base": 100.0, "dims": 12, "scaling": {"factor": 2.0, "original": 16, "fast": 1.0, "slow": 1.0}},     # a ramp of no width
    {"base": 7000.0, "dims": 24, "scaling": {"factor": 5.0, "original": 100000, "fast": 2.0, "slow": 1.0}},  # every pair fast
])
def test_frequencies_blended_along_a_ramp(rot):
    """The position part's frequencies, magnitude and table of a step against the plain implementation."""
    from rocml_b200 import kernels
    from rocml_b200.config.specs import PositionSpec, _frozen_params
    from rocml_b200.parts import BuildEnv, build_position
    params = {"ramp_scaling": rot["scaling"]} if "scaling" in rot else {}
    enc = build_position(PositionSpec("rope_neox", theta=rot["base"], rot_dim=rot["dims"], params_items=_frozen_params(params)),
                         64, BuildEnv(torch.device(DEV), torch.bfloat16))
    want, mag = P.frequencies(rot)
    assert not enc.interleaved and enc.rot_dim == rot["dims"] and abs(enc.magnitude - mag) < 1e-12
    assert float((enc.inv_freq.cpu().double() - want).abs().max() / want.max()) < 1e-7
    if "scaling" in rot and rot["scaling"]["original"] == 40:
        plain, _ = P.frequencies({"base": rot["base"], "dims": rot["dims"]})
        ratio = (want / plain).tolist()
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 3.0) < 1e-12 and any(1 / 3.0 + 1e-6 < r < 1 - 1e-6 for r in ratio)
        assert mag > 1.05
    pos = torch.tensor([0, 1, 77, 300], dtype=torch.int32, device=DEV)
    table = kernels.rope_table(pos, enc.inv_freq, 4, enc.magnitude).cpu().double()
    ang = pos.cpu().double()[:, None] * want[None, :]
    assert float((table[..., 0] - torch.cos(ang) * mag).abs().max()) < 1e-4
    assert float((table[..., 1] - torch.sin(ang) * mag).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, hd, vd, rot_dims, parts, order", [
    (4, 2, 32, 16, 16, 1, "rotate_then_unit"), (3, 3, 20, 28, 12, 3, "norm_then_rotate"), (8, 1, 64, 48, 64, 2, "rotate_then_unit"),
    (2, 2, 128, 64, 32, 1, "norm_then_rotate"), (5, 1, 16, 16, 0, 1, "rotate_then_unit"), (2, 1, 128, 128, 128, 4, "rotate_then_unit"),
    # heads of 128 on both sides take the kernel with four dimensions a lane: part of a head turns, by 1 to 16 lanes
    (4, 2, 128, 128, 64, 1, "norm_then_rotate"), (3, 1, 128, 128, 40, 2, "rotate_then_unit"), (6, 3, 128, 128, 8, 1, "rotate_then_unit"),
    (5, 5, 128, 128, 120, 8, "norm_then_rotate"), (2, 2, 128, 128, 0, 1, "rotate_then_unit")])
def test_rotation_norms_and_blended_values(dtype, nq, nkv, hd, vd, rot_dims, parts, order):
    """Queries and keys: a weighted per-head norm before the rotation, or a division by the root mean square after
    it; rotate-half over the first rot_dims entries with a magnitude on cosines and sines; value heads of another
    width; every head padded to one width; the values handed on as projected and, in a second call, blended with
    them; from one result and from partial sums."""
    from rocml_b200 import kernels
    torch.manual_seed(nq * hd + vd)
    dt = DT[dtype]
    T, eps = 70, 1e-5
    hdp = -(-max(hd, vd) // 16) * 16
    width = nq * hd + nkv * (hd + vd)
    width_p = -(-(width + 5) // 8) * 8          # more columns follow (a gate's), which the kernel leaves alone
    rows = torch.randn(parts, T, width_p) if parts > 1 else torch.randn(T, width_p).to(dt)
    pos = torch.arange(5, 5 + T, dtype=torch.int32)
    rot = {"base": 10000.0, "dims": rot_dims, "scaling": {"factor": 6.0, "original": 32, "fast": 8.0, "slow": 1.0}}
    inv = mag = None
    if rot_dims:
        f, mag = P.frequencies(rot)
        inv = f.float().to(DEV)
    n_pages = 4
    kc = torch.full((n_pages, nkv, 64, hdp), 7.0, dtype=dt, device=DEV)
    vc = torch.full((n_pages, nkv, 64, hdp), 7.0, dtype=dt, device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, n_pages).contiguous().to(DEV)
    q = torch.full((T, nq * hdp), 7.0, dtype=dt, device=DEV)
    wq = wk = None
    if order == "norm_then_rotate":
        wq, wk = (1 + 0.3 * torch.randn(hd)).to(dt).to(DEV), (1 + 0.3 * torch.randn(hd)).to(dt).to(DEV)
    cs = kernels.rope_table(pos.to(DEV), inv, T, mag) if rot_dims else None
    v_out = torch.full((T, nkv * vd), 9.0, dtype=torch.float32, device=DEV)
    slot = torch.zeros(T, dtype=torch.int32, device=DEV)
    kernels.qk_norm_rope_cache(rows.to(DEV), q, T, nq, nkv, hd, wq, wk, eps, inv, rot_dims, pos.to(DEV), slot, table, kc, vc,
                               cos_sin=cs, v_head_dim=vd, padded_head_dim=hdp, post_norm=order == "rotate_then_unit", v_out=v_out)
    x = (rows.double().sum(0) if parts > 1 else rows.double())
    xq = x[:, :nq * hd].reshape(T, nq, hd)
    xk = x[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    xv = x[:, (nq + nkv) * hd:width].reshape(T, nkv, vd)
    if order == "norm_then_rotate":
        xq, xk = P.rms(xq, eps) * wq.cpu().double(), P.rms(xk, eps) * wk.cpu().double()
    xq, xk = P.rotate_half(xq, pos.tolist(), rot), P.rotate_half(xk, pos.tolist(), rot)
    if order == "rotate_then_unit":
        xq, xk = P.rms(xq, eps), P.rms(xk, eps)
    tol = 1e-2 if dtype == "bfloat16" else 2e-5
    got_q = q.reshape(T, nq, hdp)
    assert close(got_q[:, :, :hd], xq, tol) and float(got_q[:, :, hd:].abs().sum()) == 0
    assert close(v_out.reshape(T, nkv, vd), xv, 1e-6)

    def cached(cache, width_of_head):
        return torch.stack([cache[n_pages - 1 - int(p) // 64, :, int(p) % 64, :width_of_head] for p in pos])
    assert close(cached(kc, hd), xk, tol) and close(cached(vc, vd), xv, tol)
    assert float(cached(kc, hdp)[..., hd:].abs().sum()) == 0 and float(cached(vc, hdp)[..., vd:].abs().sum()) == 0
    # a later layer: its own values blended with the first call's
    lam = torch.tensor([0.37], dtype=torch.float32, device=DEV)
    rows2 = torch.randn(T, width_p).to(dt)
    kernels.qk_norm_rope_cache(rows2.to(DEV), q, T, nq, nkv, hd, wq, wk, eps, inv, rot_dims, pos.to(DEV), slot, table, kc, vc,
                               cos_sin=cs, v_head_dim=vd, padded_head_dim=hdp, v_first=v_out, v_lambda=lam)
    xv2 = rows2.double()[:, (nq + nkv) * hd:width].reshape(T, nkv, vd)
    assert close(cached(vc, vd), P.mix_values(xv2, xv, 0.37), tol)
    assert float(cached(vc, hdp)[..., vd:].abs().sum()) == 0


def _plain_attention(qs, ks, vs, scale, window, keep, sink):
    """Rows of the step's queries: each sequence's last len(q) positions over all its keys; heads grouped."""
    outs = []
    for q, k, v in zip(qs, ks, vs):
        n, ql = k.shape[0], q.shape[0]
        pos = list(range(n))
        seen = P.visible(pos, window or n + 1, keep)[n - ql:]
        H, G = q.shape[1], k.shape[1]
        o = torch.empty(ql, H, v.shape[-1], dtype=torch.float64)
        for h in range(H):
            s = (q[:, h].double() @ k[:, h // (H // G)].double().t()) * scale
            a = P.weights_one_more(s, seen) if sink else P.weights_softmax(s, seen)
            o[:, h] = a @ v[:, h // (H // G)].double()
        outs.append(o)
    return torch.cat(outs, 0)


MASK_CASES = [
    # lens, q_lens, nq, nkv, hd, window, keep, sink
    ([5, 70, 129], [5, 70, 129], 4, 2, 16, 24, 3, True),          # whole prompts; a window and a few kept positions
    ([200, 64, 1], [30, 1, 1], 6, 1, 32, 40, 20, False),          # a piece of a prompt and single tokens
    ([300, 131], [300, 3], 5, 5, 48, 9, 70, True),                # more kept positions than the window is long, over a page border
    ([700], [1], 8, 1, 64, 130, 6, True),                         # one token far into a sequence
    ([700, 333, 150], [1, 1, 1], 8, 2, 64, 64, 64, False),        # a window and kept positions of exactly a page
    ([260, 90], [65, 90], 20, 1, 64, 100, 1, True),               # a group wider than a block's 16 rows
    ([513, 70], [513, 70], 4, 2, 128, 150, 33, True),
    ([400, 200], [137, 200], 2, 2, 128, None, 0, True),           # no window at all: only the extra term
    ([1100, 300], [1, 1], 16, 2, 128, 300, 100, True),
    ([333, 90], [333, 90], 8, 1, 64, 40, 20, True),
]


@pytest.mark.parametrize("case", range(len(MASK_CASES)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_with_kept_first_positions_and_one_more_term(case, dtype):
    """The library's paged attention (whichever kernels it picks for the sizes, and the plain kernel forced) against
    the plain implementation; one far key and one kept key are made to stand out, and a key just outside the window
    is made large so that seeing it would show."""
    from types import SimpleNamespace
    from rocml_b200 import kernels
    from rocml_b200.parts.attention import paged_attention
    from test_kernels_gpu import paged_case
    lens, q_lens, nq, nkv, hd, window, keep, sink = MASK_CASES[case]
    dt = DT[dtype]
    ks, vs, qs, kc, vc, meta = paged_case(100 + case, lens, q_lens, nq, nkv, hd, dt)
    # make the edges matter: the last query of every sequence looks for the key just outside its window, the key
    # just inside, the last kept key and the first key that is not kept
    g = torch.Generator().manual_seed(case)
    for b, n in enumerate(lens):
        if window is None or n <= window + keep + 2:
            continue
        marks = [n - 1 - window, n - window, keep - 1, keep] if keep else [n - 1 - window, n - window]
        for j in marks:
            ks[b][j] = (qs[b][-1][:: nq // nkv] * (1.0 + 0.2 * torch.rand(1, generator=g))).to(dt).float()
            page = int(meta["table"][meta["seq_slot"][b], j // 64])
            kc[page, :, j % 64] = ks[b][j]
    scale = 1.0 / math.sqrt(hd)
    want = _plain_attention(qs, ks, vs, scale, window, keep, sink)
    q = torch.cat(qs, 0).reshape(-1, nq * hd).to(dt).to(DEV)
    d = {k: v.to(DEV) for k, v in meta.items()}
    T = q.shape[0]
    is_decode = max(q_lens) == 1
    positions = torch.cat([torch.arange(n - ql, n) for n, ql in zip(lens, q_lens)]).to(torch.int32).to(DEV)
    slot_of_token = torch.cat([torch.full((ql,), int(meta["seq_slot"][b])) for b, ql in enumerate(q_lens)]).to(torch.int32).to(DEV)
    batch = SimpleNamespace(is_decode=is_decode, n_tokens=T, n_seqs=len(lens), max_q_len=max(q_lens), max_kv_len=max(lens),
                            seq_slot=d["seq_slot"], cu_q=d["cu_q"], kv_len=d["kv_len"], positions=positions,
                            slot_of_token=slot_of_token)
    tol = 2e-2 if dtype == "bfloat16" else 3e-5
    out = torch.full_like(q, float("nan"))
    paged_attention(q, out, batch, kc.to(dt).to(DEV), vc.to(dt).to(DEV), d["table"], nq, nkv, hd, scale, window or 0,
                    keep=keep, sink=0.0 if sink else None)
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < tol, ("library's choice", err)
    if dtype == "bfloat16":
        # a gate for every value, taken by the attention kernel from columns of the projection rows: in one piece, and
        # (single tokens) as partial sums that are added first; the kernels for heads of 64, 128 and 256 take it
        forms = [torch.randn(T, 8 + nq * hd, generator=g).to(dt)] + ([torch.randn(3, T, 8 + nq * hd, generator=g)] if is_decode else [])
        for rows in forms:
            out = torch.full_like(q, float("nan"))
            done = paged_attention(q, out, batch, kc.to(dt).to(DEV), vc.to(dt).to(DEV), d["table"], nq, nkv, hd, scale, window or 0,
                                   keep=keep, sink=0.0 if sink else None, gate=rows.to(DEV)[..., 8:])
            assert done == (hd in (64, 128, 256))
            z = (rows.double().sum(0) if rows.dim() == 3 else rows.double())[:, 8:]
            gated = want * torch.sigmoid(z).reshape(want.shape) if done else want
            err = (out.cpu().double().reshape(want.shape) - gated).abs().max().item()
            assert err < tol, ("gated inside", done, err)
    out = torch.full_like(q, float("nan"))
    kernels.attention_generic(q, out, kc.to(dt).to(DEV), vc.to(dt).to(DEV), d["table"], d["seq_slot"], d["cu_q"], d["kv_len"],
                              len(lens), max(q_lens), nq, nkv, hd, scale, window or 0, keep=keep, sink=0.0 if sink else None)
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < tol, ("plain kernel", err)
    # the marks matter: without the kept positions, or with a window one longer, the plain result moves
    if window is not None and any(n > window + keep + 2 for n in lens):
        assert (_plain_attention(qs, ks, vs, scale, window + 1, keep, sink) - want).abs().max() > 0.1
        if keep:
            assert (_plain_attention(qs, ks, vs, scale, window, keep - 1, sink) - want).abs().max() > 0.1
            assert (_plain_attention(qs, ks, vs, scale, window, keep + 1, sink) - want).abs().max() > 0.1


@pytest.mark.parametrize("lens, nq, nkv, window, keep, sink, rot_dims, order, parts, mix", [
    ([1, 70, 333, 700], 8, 2, 150, 3, True, 32, "rotate_then_unit", 3, "source"),
    ([64, 65, 1100], 4, 4, 300, 100, False, 128, "norm_then_rotate", 8, "mix"),
    ([129, 5], 16, 1, 40, 0, True, 0, "rotate_then_unit", 1, None),
    ([2000, 900, 31, 64, 640], 6, 3, 64, 64, True, 72, "norm_then_rotate", 2, "mix"),
])
def test_single_tokens_made_from_partial_sums_inside_the_attention_kernel(lens, nq, nkv, window, keep, sink, rot_dims, order, parts, mix):
    """Heads of 128, one token a sequence: the decode kernel adds the projection's partial sums, normalises, turns part
    of each head, divides by the root mean square, keeps or blends the new values, writes key and value to their page,
    attends under the window with kept first positions and one more term, and multiplies by the sigmoid of the gate
    columns.  Against the plain implementation; the new key is made to matter (the query looks for it)."""
    from rocml_b200 import kernels
    from test_kernels_gpu import paged_case
    hd, eps, B = 128, 1e-5, len(lens)
    dt = torch.bfloat16
    ks, vs, qs, kc, vc, meta = paged_case(7 + len(lens), lens, [1] * B, nq, nkv, hd, dt)
    g = torch.Generator().manual_seed(nq)
    width = (nq + 2 * nkv) * hd
    total = width + nq * hd + 8                       # heads, gate columns, padding
    x = torch.randn(B, total, generator=g)
    for b in range(B):                                # each sequence's first query head resembles its new key
        x[b, :hd] = x[b, nq * hd:nq * hd + hd] * 1.5
    rows = torch.randn(parts, B, total, generator=g)
    rows[0] += x - rows.sum(0)                        # partial sums whose sum is x up to 32-bit rounding
    x = rows.double().sum(0)
    pos = [n - 1 for n in lens]
    rot = {"base": 10000.0, "dims": rot_dims, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    inv = mag = cs = None
    if rot_dims:
        f, mag = P.frequencies(rot)
        inv = f.float().to(DEV)
        cs = kernels.rope_table(torch.tensor(pos, dtype=torch.int32, device=DEV), inv, B, mag)
    wq = wk = None
    if order == "norm_then_rotate":
        wq, wk = (1 + 0.3 * torch.randn(hd, generator=g)).to(dt).to(DEV), (1 + 0.3 * torch.randn(hd, generator=g)).to(dt).to(DEV)
    xq = x[:, :nq * hd].reshape(B, nq, hd)
    xk = x[:, nq * hd:(nq + nkv) * hd].reshape(B, nkv, hd)
    xv = x[:, (nq + nkv) * hd:width].reshape(B, nkv, hd)
    z = x[:, width:width + nq * hd].reshape(B, nq, hd)
    if order == "norm_then_rotate":
        xq, xk = P.rms(xq, eps) * wq.cpu().double(), P.rms(xk, eps) * wk.cpu().double()
    if rot_dims:
        xq, xk = P.rotate_half(xq, pos, rot), P.rotate_half(xk, pos, rot)
    if order == "rotate_then_unit":
        xq, xk = P.rms(xq, eps), P.rms(xk, eps)
    v_first = lam = v_keep = None
    v_new = xv
    if mix == "mix":
        v_first = torch.randn(B, nkv * hd, generator=g)
        lam = torch.tensor([0.6], dtype=torch.float32)
        v_new = P.mix_values(xv, v_first.double().reshape(B, nkv, hd), 0.6)
    elif mix == "source":
        v_keep = torch.full((B, nkv * hd), 9.0, dtype=torch.float32, device=DEV)
    scale = 0.09
    want = []
    for b in range(B):
        k = torch.cat([ks[b][:-1].double(), xk[b:b + 1].to(dt).double()])
        v = torch.cat([vs[b][:-1].double(), v_new[b:b + 1].to(dt).double()])
        want.append(_plain_attention([xq[b:b + 1]], [k], [v], scale, window, keep, sink))
    want = torch.cat(want, 0) * torch.sigmoid(z)
    d = {k: v.to(DEV) for k, v in meta.items()}
    kc, vc = kc.to(DEV), vc.to(DEV)
    n_pages = (max(lens) + 63) // 64
    out = torch.full((B, nq * hd), float("nan"), dtype=dt, device=DEV)
    for ppb in ([1, 4] if n_pages > 1 else [1]):
        n_blocks = -(-n_pages // ppb)
        acc = torch.empty((B, nq, n_blocks, hd), dtype=torch.float32, device=DEV) if n_blocks > 1 else None
        ml = torch.empty((B, nq, n_blocks, 2), dtype=torch.float32, device=DEV) if n_blocks > 1 else None
        dev_rows = rows.to(DEV) if parts > 1 else rows[0].to(DEV)
        done = kernels.attention_decode_fused(
            dev_rows, out, kc, vc, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"], B, nq, nkv, hd, wq, wk, eps, cs, True,
            scale, window, n_blocks, acc, ml, ppb, keep=keep, sink=0.0 if sink else None, rot_dim=rot_dims,
            post_norm=order == "rotate_then_unit", v_first=None if v_first is None else v_first.to(DEV),
            v_lambda=None if lam is None else lam.to(DEV), v_keep=v_keep, gate=dev_rows[..., width:width + nq * hd])
        assert done
        err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
        assert err < 2e-2, (ppb, err)
        for b in range(B):
            page = int(meta["table"][meta["seq_slot"][b], pos[b] // 64])
            assert close(kc[page, :, pos[b] % 64], xk[b], 1e-2) and close(vc[page, :, pos[b] % 64], v_new[b], 1e-2)
        if v_keep is not None:
            assert close(v_keep.reshape(B, nkv, hd), xv, 1e-6)
    # the new key matters: without it the first head's result moves
    b = max(range(B), key=lambda i: lens[i])
    k = torch.cat([ks[b][:-1].double(), torch.zeros(1, nkv, hd, dtype=torch.float64)])
    v = torch.cat([vs[b][:-1].double(), v_new[b:b + 1].double()])
    other = _plain_attention([xq[b:b + 1]], [k], [v], scale, window, keep, sink) * torch.sigmoid(z[b:b + 1])
    assert (other[:, 0] - want[b:b + 1, 0]).abs().max() > 0.05


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, in_w, out_w, parts", [(3, 32, 28, 1), (8, 64, 48, 2), (2, 128, 128, 1), (5, 16, 13, 3)])
def test_gate_for_every_value(dtype, heads, in_w, out_w, parts):
    """Heads narrowed to the values' width and multiplied by the sigmoid of the projection's gate columns, one a value."""
    from rocml_b200 import kernels
    torch.manual_seed(heads)
    dt = DT[dtype]
    T = 37
    a = torch.randn(T, heads * in_w).to(dt)
    rows = torch.randn(parts, T, 24 + heads * out_w) if parts > 1 else torch.randn(T, 24 + heads * out_w).to(dt)
    raw = rows.to(DEV)[..., 24:]
    o = torch.empty(T, heads * out_w, dtype=dt, device=DEV)
    kernels.head_gate(a.to(DEV), o, None, heads, in_w, out_w, T, raw=raw, per_value=True)
    z = rows.double().sum(0)[:, 24:] if parts > 1 else rows.double()[:, 24:]
    want = a.double().reshape(T, heads, in_w)[:, :, :out_w] * torch.sigmoid(z).reshape(T, heads, out_w)
    assert close(o.reshape(T, heads, out_w), want, 1e-2 if dtype == "bfloat16" else 1e-6)
    gate = torch.sigmoid(z).float().contiguous().to(DEV)
    kernels.head_gate(a.to(DEV), o, gate, heads, in_w, out_w, T, per_value=True)
    assert close(o.reshape(T, heads, out_w), want, 1e-2 if dtype == "bfloat16" else 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, H", [(3, 72), (70, 256), (300, 1024)])
def test_two_norms_of_one_row_with_weights_around_zero(dtype, T, H):
    """x + pending, then rms(x) * (1 + w1) and rms(x) * (1 + w2) from one kernel; the weights are bfloat16 numbers
    near zero whose sum with one is formed in 32-bit."""
    from rocml_b200.config.specs import NormSpec
    from rocml_b200.parts import BuildEnv, build_norm
    torch.manual_seed(T)
    env = BuildEnv(torch.device(DEV), DT[dtype])
    spec = NormSpec("rmsnorm", 2e-5, 1.0)
    n1, n2 = build_norm(spec, H, env), build_norm(spec, H, env)
    w1, w2 = (0.01 * torch.randn(H)).to(torch.bfloat16), (0.3 * torch.randn(H)).to(torch.bfloat16)
    n1.load({"a.weight": w1.to(DEV)}, "a")
    n2.load({"b.weight": w2.to(DEV)}, "b")
    x, pend = torch.randn(T, H), torch.randn(2, T, H)
    resid = x.clone().to(DEV)
    o1, o2 = n1.forward_with(n2, resid, pend.to(DEV), T)
    xs = x.double() + pend.double().sum(0)
    assert close(resid, xs, 1e-6)
    tol = 1e-2 if dtype == "bfloat16" else 1e-6
    assert close(o1, P.norm_one_plus(xs, w1.double(), 2e-5), tol) and close(o2, P.norm_one_plus(xs, w2.double(), 2e-5), tol)
    if dtype == "float32":      # 1 + w in bfloat16 would be off by up to 2^-9: the 32-bit sum is not
        assert close(o1, P.norm_one_plus(xs, w1.double(), 2e-5), 2e-6)


# ---- the engine -------------------------------------------------------------------------------------------------

class Folder:
    """A model folder with its plain implementation (logits kept per prompt)."""

    def __init__(self, folder):
        self.folder = folder
        self.cfg, self.w = P.load(folder)
        self.kept = {}

    def __call__(self, ids):
        key = tuple(ids)
        if key not in self.kept:
            self.kept[key] = P.forward(self.cfg, self.w, list(ids))
        return self.kept[key]


@pytest.fixture(scope="module", params=sorted(SAFESUN))
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"safesun_{name}"))
    write_safesun(folder, SAFESUN[name], seed=70 + ord(name[-1]))
    return name, SAFESUN[name], Folder(folder)


def engine(folder, dtype, **kw):
    from rocml_b200 import Engine
    kw.setdefault("max_tokens", 1024)
    return Engine.from_folder(folder, dtype=dtype, **kw)


def assert_rows(got, want, dtype, what):
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    assert bool(torch.isfinite(got).all()), what
    err = rel_err(got, want)
    assert err < TOL[dtype], f"{what}: off by {err:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype):
    """Lengths around the pages' borders (64) and around every window and count of kept positions of the three
    configurations, every place compared: the first tokens, keys just inside and just outside."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, dtype)
    for n in (1, 2, 3, 6, 10, 37, 38, 43, 63, 64, 65, 71, 80, 91, 128, 129, 131, 261, 302):
        ids = prompt(n, n, cfg["vocab"])
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(n)))])
        eng.release(slot)
        assert_rows(got, plain(ids), dtype, f"{name} {dtype} n={n}")
    eng.cache.check_invariants()


def test_a_window_or_kept_count_one_off_would_show(model):
    """The plain implementation with every window one longer or shorter, or one more or fewer kept position, is far
    from itself by many times the 32-bit tolerance, so the comparisons of this file would see such a fault."""
    name, cfg, plain = model
    ids = prompt(5, 200, cfg["vocab"])
    want = plain(ids)
    for key, least in (("size", 1), ("keep_first", 0)):
        for off in (1, -1):
            other = json.loads(json.dumps(cfg))
            changed = False
            for L in other["layers"]:
                m = L["mixer"].get("mask")
                if m and m[key] + off >= least and m[key] < 150:
                    m[key] += off
                    changed = True
            assert changed
            err = rel_err(P.forward(other, plain.w, ids), want)
            assert err > 30 * TOL["float32"], f"{name} {key} {off:+d}: {err}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_prompt_then_token_by_token(model, dtype, graphs):
    """The last tokens one by one (windows of up to 150 positions pass over decoded tokens; pages begin and end;
    windowed layers give pages back but for those of the kept positions; the blended values come from the step's own
    first layer), against the same positions of the whole prompt."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, dtype, use_graphs=graphs)
    for n, tail in ((150, 80), (81, 80), (330, 200)):
        ids = prompt(300 + n, n, cfg["vocab"])
        want = plain(ids)
        slot = eng.new_sequence()
        head = n - tail
        got = [eng.step([StepEntry(slot, ids[:head], [head - 1])]).clone()]
        for t in range(head, n):
            got.append(eng.step([StepEntry(slot, [ids[t]], [0])]).clone())
        eng.release(slot)
        assert_rows(torch.cat(got, dim=0), want[head - 1:], dtype, f"{name} {dtype} n={n} graphs={graphs}")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_very_first_token(model, dtype):
    """A sequence grown one token at a time from nothing, across page borders, windows, kept positions and the
    graphs' context buckets, every row compared."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    n = 270
    ids = prompt(9, n, cfg["vocab"])
    eng = engine(plain.folder, dtype)
    slot = eng.new_sequence()
    got = [eng.step([StepEntry(slot, [ids[t]], [0])]).clone() for t in range(n)]
    eng.release(slot)
    assert_rows(torch.cat(got, dim=0), plain(ids), dtype, f"{name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("piece", [2, 5, 64, 100])
def test_prompts_in_pieces(model, dtype, piece):
    """Steps cut into pieces of 2 to 100 tokens (the engine's work space is that small): two sequences side by
    side, every place wanted, then a few tokens one by one."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, dtype, max_step_tokens=piece)
    lens = (140, 70) if piece > 2 else (67, 9)
    seqs = [prompt(700 + i, n + 4, cfg["vocab"]) for i, n in enumerate(lens)]
    slots = [eng.new_sequence() for _ in seqs]
    got = eng.step([StepEntry(s, ids[:-4], list(range(len(ids) - 4))) for s, ids in zip(slots, seqs)])
    rows, at = [], 0
    for ids in seqs:
        rows.append([got[at:at + len(ids) - 4].clone()])
        at += len(ids) - 4
    for k in range(4, 0, -1):
        out = eng.step([StepEntry(s, [ids[-k]], [0]) for s, ids in zip(slots, seqs)])
        for i in range(len(seqs)):
            rows[i].append(out[i:i + 1].clone())
    for i, ids in enumerate(seqs):
        assert_rows(torch.cat(rows[i], dim=0), plain(ids), dtype, f"{name} {dtype} piece={piece} seq {i}")
        eng.release(slots[i])
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_against_each_alone_and_reuse(model, dtype):
    """Batches of unequal prompts, then one token each until the shorter ones end; later batches get the slots and
    pages that earlier ones gave back.  Every request is compared with the plain implementation of it alone, and in
    32-bit the batched rows equal the rows of the request stepped alone in the same engine."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, dtype, max_tokens=640)
    batches = [[(5, 8), (70, 3), (130, 12), (1, 5)], [(64, 4), (2, 9), (33, 1)], [(190, 6), (90, 2)]]
    for r, batch in enumerate(batches):
        seqs = []
        for j, (plen, ndec) in enumerate(batch):
            ids = prompt(1000 * r + j, plen + ndec, cfg["vocab"])
            seqs.append({"ids": ids, "plen": plen, "slot": eng.new_sequence(), "got": []})
        out = eng.step([StepEntry(s["slot"], s["ids"][:s["plen"]], [s["plen"] - 1]) for s in seqs])
        for i, s in enumerate(seqs):
            s["got"].append(out[i].clone())
            s["pos"] = s["plen"]
        live = list(seqs)
        while live:
            for s in [s for s in live if s["pos"] >= len(s["ids"])]:
                eng.release(s["slot"])
            live = [s for s in live if s["pos"] < len(s["ids"])]
            if not live:
                break
            out = eng.step([StepEntry(s["slot"], [s["ids"][s["pos"]]], [0]) for s in live])
            for i, s in enumerate(live):
                s["got"].append(out[i].clone())
                s["pos"] += 1
        for j, s in enumerate(seqs):
            got = torch.stack(s["got"])
            assert_rows(got, plain(s["ids"])[s["plen"] - 1:], dtype, f"{name} {dtype} batch {r} seq {j}")
            if dtype == "float32" and j == 2:
                slot = eng.new_sequence()
                alone = [eng.step([StepEntry(slot, s["ids"][:s["plen"]], [s["plen"] - 1])]).clone()]
                for t in range(s["plen"], len(s["ids"])):
                    alone.append(eng.step([StepEntry(slot, [s["ids"][t]], [0])]).clone())
                eng.release(slot)
                assert rel_err(got, torch.cat(alone).cpu()) < 2e-6
        eng.cache.check_invariants()
    assert eng.cache.slots.n_held == 0
    for g in eng.cache.kv_groups:
        assert g.pool.n_held == 0


def test_a_windowed_layer_holds_its_window_and_the_kept_pages(model):
    """A long sequence decoded token by token: a layer with a window holds the pages of its window and those of its
    kept first positions, not the whole sequence."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, "float32", max_tokens=2048)
    slot = eng.new_sequence()
    eng.step([StepEntry(slot, prompt(3, 900, cfg["vocab"]), [])])
    for t in range(30):
        eng.step([StepEntry(slot, [t % cfg["vocab"]], [0])])
    for g in eng.cache.kv_groups:
        held = int((g.table_host[slot] >= 0).sum())
        if g.req.window is None:
            assert held == (930 + 63) // 64
        else:
            assert held <= (g.req.window + 63) // 64 + 1 + g.req.kept_pages, (g.req, held)
            assert all(g.table_host[slot][p] >= 0 for p in range(g.req.kept_pages))
    eng.release(slot)
    eng.cache.check_invariants()


def _one_layer(layer, width=64, vocab=40):
    return {"architecture": "Safesun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [layer]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_keys_that_must_and_must_not_be_seen(tmp_path, dtype, kind):
    """One attention layer, no feed-forward, no rotation, a window of 150 positions that keeps the first 10, in a
    prompt of 460.  The weights are made so that one key stands out: the first 16 entries of a token's row are its
    'key part', the next 16 its 'value part'; queries and keys compare key parts, values come from value parts.
    Tokens 7 and 9 share a key part and nothing else.  Token 7 sits at places 9 and 10 (the last kept place and the
    first that is not) in one variant, at place 155 in another; token 9 sits at places 303 to 306: 303 and 304 still
    see place 155 (149 back, across two page borders), 305 and 306 do not.  Whole, in pieces, and decoding over the edge."""
    from safetensors.torch import load_file, save_file
    from rocml_b200 import StepEntry
    mixer = {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 1.0, "v_mix": False,
             "mask": {"size": 150, "keep_first": 10}, "rot": {"base": 10000.0, "dims": 0}}
    cfg = _one_layer({"type": kind, "mixer": mixer, "mlp": None})
    folder = str(tmp_path / "far")
    write_model(folder, cfg, 3)
    path = folder + "/model.safetensors"
    w = load_file(path)
    g = torch.Generator().manual_seed(1)
    E = torch.zeros(40, 64)
    E[:, :16] = torch.randn(40, 16, generator=g)
    E[:, 16:32] = torch.randn(40, 16, generator=g)
    E[:, 32:] = 0.3 * torch.randn(40, 32, generator=g)
    E[9, :16] = E[7, :16]
    E[9, 16:] *= E[7, 16:].norm() / E[9, 16:].norm()       # rows of equal length: equal keys after the norms
    pick_key = torch.zeros(16, 64)
    pick_key[:, :16] = torch.eye(16)
    pick_val = torch.zeros(16, 64)
    pick_val[:, 16:32] = torch.eye(16)
    zeros = lambda *s: torch.zeros(*s, dtype=torch.bfloat16)
    w["embed"] = E.to(torch.bfloat16)
    w["embed.norm"], w["l0.norm1"], w["final.norm"] = zeros(64), zeros(64), zeros(64)
    w["l0.mix.q"] = torch.cat([pick_key, pick_key]).to(torch.bfloat16)
    w["l0.mix.k"] = pick_key.to(torch.bfloat16)
    w["l0.mix.v"] = pick_val.to(torch.bfloat16)
    if kind == "attention_2":
        w["l0.mix.q.b"], w["l0.mix.k.b"], w["l0.mix.v.b"] = zeros(32), zeros(16), zeros(16)
    else:
        w["l0.mix.q.norm"], w["l0.mix.k.norm"] = torch.ones(16, dtype=torch.bfloat16), torch.ones(16, dtype=torch.bfloat16)
    w["l0.mix.g"] = zeros(32, 64)
    o = torch.zeros(64, 32)
    o[32:64, :] = torch.eye(32) * 4
    w["l0.mix.o"] = o.to(torch.bfloat16)
    save_file(w, path)
    others = [t for t in range(40) if t not in (7, 9)]
    base_ids = [others[i % len(others)] for i in range(460)]
    for p in (303, 304, 305, 306):
        base_ids[p] = 9
    c, wf = P.load(folder)
    tol = TOL[dtype]
    for places in ((155,), (9,), (10,)):
        ids = list(base_ids)
        for p in places:
            ids[p] = 7
        want = P.forward(c, wf, ids)
        # the test is worth something: seeing the place or not moves these rows by far more than the tolerance
        for size, keep in ((149, 10), (151, 10), (150, 9), (150, 11)):
            other = json.loads(json.dumps(c))
            other["layers"][0]["mixer"]["mask"] = {"size": size, "keep_first": keep}
            moved = rel_err(P.forward(other, wf, ids)[303:307], want[303:307])
            expect = (places == (155,) and keep == 10) or (places == (9,) and keep == 9) or (places == (10,) and keep == 11)
            assert (moved > 0.1) == expect, (places, size, keep, moved)
        eng = engine(folder, dtype)
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(460)))])
        eng.release(slot)
        assert rel_err(got, want) < tol, places
        eng = engine(folder, dtype, max_step_tokens=100)        # pieces: 303 to 306 lie in one piece, the far places in others
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(460)))])
        eng.release(slot)
        assert rel_err(got, want) < tol, places
        for graphs in (False, True):
            eng = engine(folder, dtype, use_graphs=graphs)
            slot = eng.new_sequence()
            eng.step([StepEntry(slot, ids[:290], [])])
            rows = [eng.step([StepEntry(slot, [ids[t]], [0])]).clone() for t in range(290, 312)]
            eng.release(slot)
            assert rel_err(torch.cat(rows), want[290:312]) < tol, (places, graphs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model, dtype):
    """A short prompt and 700 tokens one by one under CUDA graphs: every window passes over decoded tokens several
    times, pages come back and are handed out again; the last 40 rows compared."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    ids = prompt(77, 720, cfg["vocab"])
    eng = engine(plain.folder, dtype, max_tokens=1024)
    slot = eng.new_sequence()
    eng.step([StepEntry(slot, ids[:20], [])])
    got = []
    for t in range(20, 720):
        r = eng.step([StepEntry(slot, [ids[t]], [0] if t >= 680 else [])])
        if r is not None:
            got.append(r.clone())
    eng.release(slot)
    assert_rows(torch.cat(got), plain(ids)[680:], dtype, f"{name} {dtype}")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(model, dtype):
    """Engine.generate (its scheduler, sampler and run-ahead loop) against greedy decoding with the plain
    implementation, for prompts of unequal length in one batch; compared until the first step whose two best logits
    are closer than the tolerance."""
    from rocml_b200 import SamplingParams
    name, cfg, plain = model
    eng = engine(plain.folder, dtype)
    prompts = [prompt(50 + i, n, cfg["vocab"]) for i, n in enumerate((3, 70, 35))]
    outs = eng.generate(prompts, max_new_tokens=12, sampling=SamplingParams(temperature=0.0), ignore_eos=True)
    for ids, out in zip(prompts, outs):
        seq = list(ids)
        for tok in out.tokens:
            logits = P.forward(plain.cfg, plain.w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 5 * TOL[dtype] * float(logits.abs().max()):
                break
            assert tok == int(logits.argmax()), f"{name} {dtype}: after {len(seq)} tokens"
            seq.append(tok)
    assert eng.cache.slots.n_held == 0


def test_trace_replay_and_command_line(model, tmp_path):
    """bin/trace_run on a folder of this architecture: a prompt in two steps and two decoded tokens, a second request
    beside it; the logits are the plain implementation's."""
    import os
    import subprocess
    import sys
    import numpy as np
    name, cfg, f = model
    a, b = prompt(1, 40, cfg["vocab"]), prompt(2, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:38], "want": [0, 37]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[38:39], "want": [0]}, {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[39:], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["a", "b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", f.folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = f(a), f(b)
    V = cfg["vocab"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got0, torch.stack([wa[0], wa[37], wb[6]])) < TOL["float32"]
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got1, wa[38:39]) < TOL["float32"]
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got2, torch.stack([wa[39], wb[8]])) < TOL["float32"]
    r = subprocess.run([sys.executable, "-m", "rocml_b200", "generate", "--model", f.folder, "--prompt-ids", "1,2,3", "-n", "5"],
                       capture_output=True, text=True, timeout=600, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]


# ---- configurations drawn at random -----------------------------------------------------------------------------

def random_configuration(seed):
    g = torch.Generator().manual_seed(1000 + seed)

    def pick(*xs):
        return xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    width = pick(48, 64, 96, 136)
    kv, vdim = pick(1, 2, 3), pick(8, 16, 24, 64)          # shared by the layers that blend values
    layers = []
    for i in range(pick(1, 2, 3, 4)):
        kind = pick("attention", "attention_2")
        v_mix = pick(True, True, False)
        g_kv = kv if v_mix else pick(1, 2)
        heads = g_kv * pick(1, 2, 4)
        dim = pick(8, 16, 32, 64, 40)
        vd = vdim if v_mix else pick(8, 32, 48)
        rot_dims = pick(0, dim // 2 - (dim // 2) % 2, dim)
        rot = None if rot_dims == 0 else ((pick(100.0, 10000.0, 1e6), rot_dims) + (
            ((pick(2.0, 8.0), pick(16, 64, 512), pick(4.0, 32.0), pick(0.5, 1.0)),) if pick(True, False) else ()))
        mask = None if pick(True, False, False, False) else (pick(1, 5, 40, 64, 100, 200), pick(0, 1, 6, 64, 70))
        layers.append(_sfn(kind, heads, g_kv, dim, vd, pick(0.1, 0.3, 0.7), mask, rot, v_mix, pick(None, 32, 72)))
    return {"architecture": "Safesun", "vocab": pick(50, 101, 256), "width": width, "norm": {"eps": pick(1e-6, 1e-5)},
            "layers": layers}


def _sfn(kind, heads, kv, dim, vdim, scale, mask, rot, v_mix, ff):
    from tiny_models import _s, _sattn
    return _s(_sattn(kind, heads, kv, dim, vdim, scale, mask, rot, v_mix), ff)


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    """A configuration drawn at random: a whole prompt, the same in pieces of 50 with a tail decoded under graphs, and
    two requests side by side, in 32-bit (sharp) and bfloat16."""
    from rocml_b200 import StepEntry
    cfg = random_configuration(seed)
    folder = str(tmp_path / "m")
    write_safesun(folder, cfg, seed)
    plain = Folder(folder)
    ids, other = prompt(seed, 210, cfg["vocab"]), prompt(seed + 50, 75, cfg["vocab"])
    for dtype in ("float32", "bfloat16"):
        eng = engine(folder, dtype)
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(210)))])
        eng.release(slot)
        assert_rows(got, plain(ids), dtype, f"seed {seed} {dtype} whole: {json.dumps(cfg)}")
        eng = engine(folder, dtype, max_step_tokens=50)
        a, b = eng.new_sequence(), eng.new_sequence()
        got = eng.step([StepEntry(a, ids[:180], [0, 179]), StepEntry(b, other[:60], [59])]).clone()
        assert_rows(got, torch.stack([plain(ids)[0], plain(ids)[179], plain(other)[59]]), dtype, f"seed {seed} {dtype} pieces")
        rows_a, rows_b = [], []
        for t in range(15):
            out = eng.step([StepEntry(a, [ids[180 + t]], [0]), StepEntry(b, [other[60 + t]], [0])])
            rows_a.append(out[0].clone())
            rows_b.append(out[1].clone())
        assert_rows(torch.stack(rows_a), plain(ids)[180:195], dtype, f"seed {seed} {dtype} decoded a")
        assert_rows(torch.stack(rows_b), plain(other)[60:75], dtype, f"seed {seed} {dtype} decoded b")
        eng.release(a)
        eng.release(b)
        eng.cache.check_invariants()
