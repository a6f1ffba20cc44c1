"""Tibenex on the GPU against the plain implementation (tests/plain_tibenex.py): each mechanism alone, then the
engine in every way of cutting and batching, in 32-bit and in bfloat16.

Tolerances are a fraction of the largest |logit| of the row compared.  float32: sums of a few hundred terms in
another order than the plain implementation's float64.  bfloat16: activations are rounded to 8 bits of mantissa
between kernels, a dozen roundings a layer.
"""
import json
import math

import pytest
import torch

import plain_tibenex as P
from tiny_models import TIBENEX, prompt, write_tibenex

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 4e-2}
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


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


# ---- each mechanism alone -------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [20, 64, 100])
def test_blend_with_the_token_before(dtype, H):
    """Sequences side by side, in two steps: the row before a sequence's first comes from its slot (zeros at the start),
    the slot then holds the step's last row; a slot that was used before starts from what it was reset to."""
    from rocml_b200 import kernels
    torch.manual_seed(H)
    lens1, lens2 = [5, 1, 33], [1, 4, 2]
    slots = [2, 0, 3]
    mu = torch.rand(H)
    kept = torch.full((5, H), 9.0, device=DEV)
    kept[slots] = 0.0                                         # what a slot holds when it is handed out
    xs = [torch.randn(a + b, H) for a, b in zip(lens1, lens2)]
    want = [P.token_shift(x.double(), mu.double()) for x in xs]
    for step, lens in enumerate((lens1, lens2)):
        rows = [x[:a] if step == 0 else x[a:] for x, a in zip(xs, lens1)]
        x = torch.cat(rows).to(DEV)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        # a padding sequence (slot -1) at the end is skipped
        out = torch.full((x.shape[0], H), 7.0, dtype=DT[dtype], device=DEV)
        kernels.token_shift(x, mu.to(DEV), kept, i32(slots + [-1]), i32(cu + [cu[-1]]), 4, max(lens), out, x.shape[0])
        ref = torch.cat([w[:a] if step == 0 else w[a:] for w, a in zip(want, lens1)])
        assert close(out, ref, 1e-2 if dtype == "bfloat16" else 1e-6)
        for s, r in zip(slots, rows):
            assert torch.equal(kept[s].cpu(), r[-1])
    assert float(kept[1].min()) == 9.0 and float(kept[4].min()) == 9.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, H, parts, alpha, gain", [(70, 64, 1, 2.5, True), (3, 100, 3, 1.0, True), (9, 322, 8, 0.3, False), (130, 4096, 2, 7.0, True)])
def test_norm_after_the_sum(dtype, T, H, parts, alpha, gain):
    """x <- rmsnorm(alpha x + g * sum of partial sums) * w in place, with and without the vector g, rows of odd width, a padded
    row left alone."""
    from rocml_b200 import kernels
    torch.manual_seed(T + H)
    x, d = torch.randn(T, H), torch.randn(parts, T + 2, H)
    g = (1 + torch.randn(H)) if gain else None
    w = 1 + 0.3 * torch.randn(H)
    resid = x.clone().to(DEV)
    out = torch.full((T, H), 7.0, dtype=DT[dtype], device=DEV)
    slot = torch.zeros(T, dtype=torch.int32)
    slot[T // 2] = -1
    kernels.postln(resid, d.to(DEV), None if g is None else g.to(DEV), w.to(DEV), alpha, 2e-5, out, slot.to(DEV), T)
    s = d.double()[:, :T].sum(0) * (g.double() if gain else 1.0)
    want = P.norm(alpha * x.double() + s, w.double(), 2e-5)
    live = slot >= 0
    assert close(resid[live.to(DEV)], want[live], 2e-6)
    assert close(out[live.to(DEV)], want[live], 1e-2 if dtype == "bfloat16" else 2e-6)
    assert torch.equal(resid[T // 2].cpu(), x[T // 2]) and float(out[T // 2].float().min()) == 7.0
    # without anything to add: x <- rmsnorm(alpha x) * w
    resid = x.clone().to(DEV)
    kernels.postln(resid, None, None, w.to(DEV), alpha, 2e-5, None, None, T)
    assert close(resid, P.norm(alpha * x.double(), w.double(), 2e-5), 2e-6)
    # one token a sequence: the same kernel blends the new rows with the rows the next layer kept, and leaves the new rows there
    if T <= 16:
        slots = torch.randperm(T + 3)[:T].to(torch.int32)
        slots[1] = -1
        kept = torch.randn(T + 3, H)
        mu = torch.rand(H)
        resid, kept_dev = x.clone().to(DEV), kept.clone().to(DEV)
        blended = torch.full((T, H), 7.0, dtype=DT[dtype], device=DEV)
        kernels.postln(resid, d.to(DEV), None if g is None else g.to(DEV), w.to(DEV), alpha, 2e-5, None, slots.to(DEV), T,
                       next_mu=mu.to(DEV), next_kept=kept_dev, next_out=blended)
        for t in range(T):
            if t == 1:
                assert float(blended[t].float().min()) == 7.0 and torch.equal(kept_dev[slots[0]].cpu(), resid[0].cpu())
                continue
            ref = P.token_shift(want[t:t + 1], mu.double(), before=kept[slots[t]].double())
            assert close(blended[t:t + 1], ref, 1e-2 if dtype == "bfloat16" else 2e-6)
            assert torch.equal(kept_dev[slots[t]].cpu(), resid[t].cpu())


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("parts", [1, 3])
def test_short_convolution_with_kept_inputs(taps, parts):
    """Prompts and single tokens in several steps, among them steps shorter than the taps and a prompt longer than a
    block of tokens; the inputs before a step's first token come from the slot."""
    from rocml_b200 import kernels
    torch.manual_seed(taps)
    C, col0, N = 150, 8, 170
    w, b = torch.randn(C, taps), torch.randn(C)
    steps = [[40, 1, 2], [1, 1, 3], [2, 70, 1], [1, 1, 1]]
    slots = [1, 3, 0]
    total = [sum(s[i] for s in steps) for i in range(3)]
    us = [torch.randn(n, N) for n in total]
    want = [P.silu(P.causal_conv(u.double()[:, col0:col0 + C], w.double(), b.double())) for u in us]
    kept = torch.zeros((4, taps - 1, C), device=DEV) if taps > 1 else None
    at = [0, 0, 0]
    for lens in steps:
        rows = torch.cat([u[a:a + n] for u, a, n in zip(us, at, lens)])
        proj = rows.to(DEV) if parts == 1 else torch.stack([rows * 0.5, rows * 0.25, rows * 0.25]).to(DEV)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        out = torch.zeros((rows.shape[0], C), device=DEV)
        kernels.causal_conv(proj, rows.shape[0], col0, C, taps, w.to(DEV), b.to(DEV), "silu", kept, i32(slots), i32(cu), 3,
                            max(lens), out)
        ref = torch.cat([x[a:a + n] for x, a, n in zip(want, at, lens)])
        assert close(out, ref, 1e-5), (taps, lens)
        at = [a + n for a, n in zip(at, lens)]


@pytest.mark.parametrize("heads, groups, n, p", [(4, 2, 8, 16), (1, 1, 5, 36), (6, 6, 64, 64), (3, 1, 128, 100), (8, 2, 16, 4)])
@pytest.mark.parametrize("parts", [1, 2])
@pytest.mark.parametrize("by_blocks", [False, True])
def test_recurrence_with_a_step_size_per_token(heads, groups, n, p, parts, by_blocks):
    """Prompts, pieces and single tokens through the recurrence, the state carried in the slot from step to step; decays near
    one, so that the first tokens still count hundreds of tokens later (the plain result without them is far away)."""
    from rocml_b200 import kernels
    torch.manual_seed(heads * n + p)
    inner, gn = heads * p, groups * n
    lens_by_step = [[150, 3], [1, 1], [60, 1], [1, 200]]
    slots = [2, 0]
    total = [sum(s[i] for s in lens_by_step) for i in range(2)]
    a_log = torch.randn(heads) - 4.0
    dt_bias, skip = torch.randn(heads) - 1.0, torch.randn(heads)
    us = [torch.randn(T, inner + 2 * gn) for T in total]
    raws = [torch.randn(T, heads + 3) for T in total]

    def plain(u, raw, skip_first=0):
        T = u.shape[0]
        x, B, C = u[:, :inner].reshape(T, heads, p), u[:, inner:inner + gn].reshape(T, groups, n), u[:, inner + gn:].reshape(T, groups, n)
        dt = P.softplus(raw[:, 3:] + dt_bias.double())
        dec = torch.exp(-torch.exp(a_log.double()) * dt)
        S = torch.zeros(heads, n, p, dtype=torch.float64)
        y = torch.zeros(T, heads, p, dtype=torch.float64)
        of = torch.arange(heads) // (heads // groups)
        for t in range(T):
            S = dec[t][:, None, None] * S
            if t >= skip_first:
                S = S + dt[t][:, None, None] * B[t, of][:, :, None] * x[t][:, None, :]
            y[t] = torch.einsum("hnp,hn->hp", S, C[t, of]) + skip.double()[:, None] * x[t]
        return y.reshape(T, inner), S
    want = [plain(u.double(), r.double()) for u, r in zip(us, raws)]
    # the state must remember: without the first ten tokens the last rows differ
    forgot, _ = plain(us[0].double(), raws[0].double(), skip_first=10)
    assert float((forgot[-1] - want[0][0][-1]).abs().max()) > 1e-3 * float(want[0][0][-1].abs().max())
    state = torch.full((3, heads, n, p), 5.0, device=DEV)
    state[slots] = 0.0
    at = [0, 0]
    for lens in lens_by_step:
        u = torch.cat([x[a:a + k] for x, a, k in zip(us, at, lens)]).to(DEV)
        raw = torch.cat([x[a:a + k] for x, a, k in zip(raws, at, lens)])
        proj = raw.to(DEV) if parts == 1 else torch.stack([raw * 0.75, raw * 0.25]).to(DEV)
        cu = [0, lens[0], lens[0] + lens[1]]
        out = torch.zeros((u.shape[0], inner), device=DEV)
        if by_blocks and max(lens) > 1:       # prompts: blocks of 64 tokens side by side
            blocks = u.shape[0] // 64 + 2
            work = torch.full((blocks, heads, n, p), float("nan"), device=DEV)
            decay = torch.full((blocks, heads), float("nan"), device=DEV)
            cb = torch.full((blocks, groups, 64, 64), float("nan"), device=DEV)
            kernels.ssm_scan_blocks(u, u.shape[0], 0, inner, inner + gn, proj, 3, dt_bias.to(DEV), a_log.to(DEV), skip.to(DEV), heads,
                                    groups, n, p, state, i32(slots), i32(cu), 2, out, work, decay, cb)
        else:         # single tokens: the state through registers when told so (by_blocks), through shared memory otherwise
            kernels.ssm_scan(u, u.shape[0], 0, inner, inner + gn, proj, 3, dt_bias.to(DEV), a_log.to(DEV), skip.to(DEV), heads, groups,
                             n, p, state, i32(slots), i32(cu), 2, out, one_token_each=by_blocks and max(lens) == 1)
        ref = torch.cat([w[0][a:a + k] for w, a, k in zip(want, at, lens)])
        assert close(out, ref, 3e-5), lens
        at = [a + k for a, k in zip(at, lens)]
    for s, w in zip(slots, want):
        assert close(state[s], w[1], 3e-5)
    assert float(state[1].min()) == 5.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W, groups, parts", [(64, 2, 1), (36, 3, 2), (512, 8, 1), (240, 24, 3), (100, 1, 1)])
def test_gate_then_norm_in_parts(dtype, W, groups, parts):
    from rocml_b200 import kernels
    torch.manual_seed(W)
    T, z_off = 37, 4
    y = torch.randn(T, W)
    rows = torch.randn(parts, T, W + 9) if parts > 1 else torch.randn(T, W + 9).to(DT[dtype])
    w = 1 + 0.3 * torch.randn(W)
    out = torch.zeros((T, W), dtype=DT[dtype], device=DEV)
    kernels.gate_group_norm(y.to(DEV), rows.to(DEV), z_off, w.to(DEV), 1e-5, groups, "silu", out, torch.zeros(T, dtype=torch.int32, device=DEV), T)
    z = (rows.double().sum(0) if parts > 1 else rows.double())[:, z_off:z_off + W]
    g = y.double() * P.silu(z)
    want = P.rms(g.reshape(T, groups, W // groups), 1e-5).reshape(T, W) * w.double()
    assert close(out, want, 1e-2 if dtype == "bfloat16" else 2e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, rot, rank, q_rank, parts", [(4, 16, 8, 24, 40, 1), (3, 20, 0, 20, 12, 2), (5, 4, 12, 36, 100, 3), (8, 32, 32, 96, 64, 1)])
def test_latents_and_the_rotated_key_part(dtype, heads, dim, rot, rank, q_rank, parts):
    """The query latent normalised; the latent normalised and the shared key part turned into the cached row, zeros behind
    them; gates; then the queries' rotated parts turned and placed behind the folded part."""
    from rocml_b200 import kernels
    torch.manual_seed(heads + rank)
    dt = DT[dtype]
    T, eps = 70, 1e-5
    dp = rank if not rot else -(-(rank + rot) // 16) * 16
    width = q_rank + rank + rot + heads
    rows = torch.randn(parts, T, width + 3) if parts > 1 else torch.randn(T, width + 3).to(dt)
    if dtype == "bfloat16" and parts > 1:
        rows = rows.to(dt).float()
    pos = torch.arange(5, 5 + T, dtype=torch.int32)
    rotc = {"base": 1000.0, "dims": rot, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    cs = None
    if rot:
        f, mag = P.frequencies(rotc)
        cs = kernels.rope_table(pos.to(DEV), f.float().to(DEV), T, mag)
    wq, wc = 1 + 0.3 * torch.randn(q_rank), 1 + 0.3 * torch.randn(rank)
    cache = torch.full((3, 1, 64, dp), 7.0, dtype=dt, device=DEV)
    table = i32([[2, 0, 1]])
    cq = torch.zeros((T, q_rank), dtype=dt, device=DEV)
    gates = torch.zeros((T, heads), device=DEV)
    slot = torch.zeros(T, dtype=torch.int32, device=DEV)
    kernels.latent_rot_prep(rows.to(DEV), T, q_rank, rank, rot, heads, wq.to(DEV), wc.to(DEV), eps, cq, gates, cache, cs, pos.to(DEV),
                            slot, table)
    x = rows.double().sum(0) if parts > 1 else rows.double()
    tol = 1e-2 if dtype == "bfloat16" else 2e-6
    assert close(cq, P.norm(x[:, :q_rank], wq.double(), eps), tol)
    c = P.norm(x[:, q_rank:q_rank + rank], wc.double(), eps)
    kr = P.rotate(x[:, None, q_rank + rank:q_rank + rank + rot], pos.tolist(), rotc, "half")[:, 0] if rot else x[:, :0]
    got = torch.stack([cache[[2, 0, 1][int(p) // 64], 0, int(p) % 64] for p in pos])
    assert close(got[:, :rank], c, tol) and (not rot or close(got[:, rank:rank + rot], kr, tol))
    assert float(got[:, rank + rot:].float().abs().sum()) == 0
    assert close(gates, torch.sigmoid(x[:, q_rank + rank + rot:width]), 1e-5)
    if rot:
        q = torch.randn(T, heads * (dim + rot)).to(dt)
        folded = torch.full((T, heads * dp), 7.0, dtype=dt, device=DEV)
        kernels.latent_q_rot(q.to(DEV), heads, dim, rot, rank, cs, folded, slot, T)
        qr = P.rotate(q.double().reshape(T, heads, dim + rot)[..., dim:], pos.tolist(), rotc, "half")
        f3 = folded.reshape(T, heads, dp)
        assert close(f3[..., rank:rank + rot], qr, tol) and float(f3[..., rank + rot:].float().abs().sum()) == 0
        assert float(f3[..., :rank].float().min()) == 7.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, hd, vd, rot, pairs, parts", [(4, 2, 16, 16, 8, "neighbours", 1), (9, 3, 12, 20, 4, "neighbours", 2),
                                                                (8, 1, 64, 64, 64, "neighbours", 1), (6, 6, 32, 48, 0, "neighbours", 3),
                                                                (2, 2, 24, 8, 12, "half", 1)])
def test_norm_over_whole_projections_rotation_and_temperature(dtype, nq, nkv, hd, vd, rot, pairs, parts):
    from rocml_b200 import kernels
    torch.manual_seed(nq * hd + vd)
    dt = DT[dtype]
    T, eps = 70, 1e-5
    hdp = -(-max(hd, vd) // 16) * 16
    width = (nq + nkv) * hd + nkv * vd
    rows = torch.randn(parts, T, width + 5) if parts > 1 else torch.randn(T, width + 5).to(dt)
    pos = torch.arange(3, 3 + T, dtype=torch.int32)
    rotc = {"base": 300.0, "dims": rot}
    cs = None
    if rot:
        f, mag = P.frequencies(rotc)
        cs = kernels.rope_table(pos.to(DEV), f.float().to(DEV), T, mag)
    wq, wk, temp = 1 + 0.3 * torch.randn(nq * hd), 1 + 0.3 * torch.randn(nkv * hd), 1 + 0.5 * torch.randn(nq)
    kc = torch.full((2, nkv, 64, hdp), 7.0, dtype=dt, device=DEV)
    vc = torch.full((2, nkv, 64, hdp), 7.0, dtype=dt, device=DEV)
    q = torch.full((T, nq * hdp), 7.0, dtype=dt, device=DEV)
    kernels.wide_norm_rope_cache(rows.to(DEV), q, T, nq, nkv, hd, vd, hdp, wq.to(DEV), wk.to(DEV), eps, temp.to(DEV), cs, rot,
                                 pairs == "neighbours", pos.to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV), i32([[1, 0]]), kc, vc)
    x = rows.double().sum(0) if parts > 1 else rows.double()
    xq = P.norm(x[:, :nq * hd], wq.double(), eps).reshape(T, nq, hd)
    xk = P.norm(x[:, nq * hd:(nq + nkv) * hd], wk.double(), eps).reshape(T, nkv, hd)
    xv = x[:, (nq + nkv) * hd:width].reshape(T, nkv, vd)
    if rot:
        xq, xk = P.rotate(xq, pos.tolist(), rotc, pairs), P.rotate(xk, pos.tolist(), rotc, pairs)
    xq = xq * temp.double()[None, :, None]
    tol = 1e-2 if dtype == "bfloat16" else 2e-6
    q3 = q.reshape(T, nq, hdp)
    assert close(q3[..., :hd], xq, tol) and float(q3[..., hd:].float().abs().sum()) == 0

    def cached(cache):
        return torch.stack([cache[[1, 0][int(p) // 64], :, int(p) % 64] for p in pos])
    assert close(cached(kc)[..., :hd], xk, tol) and close(cached(vc)[..., :vd], xv, tol)
    assert float(cached(kc)[..., hd:].float().abs().sum()) == 0 and float(cached(vc)[..., vd:].float().abs().sum()) == 0


PAIR_CASES = [
    # lens, q_lens, nq, nkv, hd
    ([5, 70, 129], [5, 70, 129], 4, 2, 16),
    ([200, 64, 1], [30, 1, 1], 6, 3, 32),
    ([700, 333, 150], [1, 1, 1], 8, 4, 64),
    ([300], [300], 9, 3, 48),
    ([1100, 65], [1, 1], 4, 4, 16),
    ([300, 70], [300, 70], 8, 2, 128),          # head sizes that the tensor-memory kernel takes
    ([513], [200], 4, 4, 64),
    ([900, 200, 64], [1, 1, 1], 16, 4, 128),
]


@pytest.mark.parametrize("case", range(len(PAIR_CASES)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_mixed_after_the_softmax(case, dtype):
    """Every query head's weights on every stored head's values, then the sums over heads, against weights mixed and then
    applied; prompts, pieces and single tokens over pages in any order.  One key hundreds of positions back is made to
    stand out for one head only, and the mix carries it to the others."""
    from types import SimpleNamespace
    from rocml_b200 import kernels
    from rocml_b200.parts.attention import paged_attention
    from test_kernels_gpu import paged_case
    lens, q_lens, nq, nkv, hd = PAIR_CASES[case]
    dt = DT[dtype]
    ks, vs, qs, kc, vc, meta = paged_case(300 + case, lens, q_lens, nq, nkv, hd, dt)
    gs = nq // nkv
    for b, n in enumerate(lens):
        if n > 40:      # the far key: head 0's last query looks for key 3
            ks[b][3, 0] = (qs[b][-1, 0] * 3.0).to(dt).float()
            page = int(meta["table"][meta["seq_slot"][b], 0])
            kc[page, 0, 3] = ks[b][3, 0]
    torch.manual_seed(case)
    talk = torch.eye(nq) * 0.6 + 0.4 * torch.randn(nq, nq)
    scale = 1.0 / math.sqrt(hd)
    want = []
    for q, k, v in zip(qs, ks, vs):
        n, ql = k.shape[0], q.shape[0]
        pos = list(range(n))
        kv_of = torch.arange(nq) // gs
        s = torch.einsum("ihd,jhd->hij", q.double(), k.double()[:, kv_of]) * scale
        seen = (torch.arange(n)[None, :] <= torch.arange(n - ql, n)[:, None])
        a = torch.softmax(s.masked_fill(~seen[None], float("-inf")), dim=-1)
        if n > 40:
            assert float(a[0, -1, 3]) > 0.5
        a = torch.einsum("hg,gij->hij", talk.double(), a)
        want.append(torch.einsum("hij,jhd->ihd", a, v.double()[:, kv_of]))
    want = torch.cat(want, 0)
    q = torch.cat(qs, 0).reshape(-1, nq * hd).to(dt).to(DEV)
    d = {k: v.to(DEV) for k, v in meta.items()}
    T = q.shape[0]
    positions = torch.cat([torch.arange(n - ql, n) for n, ql in zip(lens, q_lens)]).to(torch.int32).to(DEV)
    slot_of_token = torch.cat([torch.full((ql,), int(meta["seq_slot"][b])) for b, ql in enumerate(q_lens)]).to(torch.int32).to(DEV)
    batch = SimpleNamespace(is_decode=max(q_lens) == 1, n_tokens=T, n_seqs=len(lens), max_q_len=max(q_lens), max_kv_len=max(lens),
                            seq_slot=d["seq_slot"], cu_q=d["cu_q"], kv_len=d["kv_len"], positions=positions, slot_of_token=slot_of_token)
    wide = torch.full((T, nq * nkv * hd), float("nan"), dtype=dt, device=DEV)
    paged_attention(q, wide, batch, kc.to(dt).to(DEV), vc.to(dt).to(DEV), d["table"], nq * nkv, nkv * nkv, hd, scale, 0, cross=nkv)
    out = torch.full((T, nq * hd), float("nan"), dtype=dt, device=DEV)
    kernels.talk_mix(wide, talk.to(DEV), out, nq, nkv, hd, hd, slot_of_token, T)
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < (3e-2 if dtype == "bfloat16" else 3e-5), err


# ---- the engine -------------------------------------------------------------------------------------------------

class Folder:
    """A model folder with its plain implementation (logits kept per prompt)."""

    def __init__(self, folder):
        self.folder = folder
        self.cfg, self.w = P.load_folder(folder)
        self.kept = {}

    def __call__(self, ids):
        key = tuple(ids)
        if key not in self.kept:
            self.kept[key] = P.forward(self.cfg, self.w, list(ids))
        return self.kept[key]


@pytest.fixture(scope="module", params=sorted(TIBENEX))
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"tibenex_{name}"))
    write_tibenex(folder, TIBENEX[name], seed=40 + ord(name[-1]))
    return name, TIBENEX[name], Folder(folder)


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
    """Lengths around the pages' borders (64), the convolutions' taps and the scan's blocks of tokens, every place compared,
    the first tokens among them."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, dtype)
    for n in (1, 2, 3, 4, 7, 8, 9, 33, 63, 64, 65, 128, 129, 131, 257):
        ids = prompt(n, n, cfg["vocab"])
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(n)))])
        eng.release(slot)
        assert_rows(got, plain(ids), dtype, f"{name} {dtype} n={n}")
    eng.cache.check_invariants()


def test_every_mechanism_matters(model):
    """The plain implementation with one mechanism taken out is far from itself by many times the 32-bit tolerance, so the
    comparisons of this file would see it missing."""
    name, cfg, plain = model
    ids = prompt(5, 90, cfg["vocab"])
    want = plain(ids)

    def differs(w=None, c=None):
        return rel_err(P.forward(c or plain.cfg, w or plain.w, ids), want) > 30 * TOL["float32"]
    for suffix, value in ((".shift", 0.0), (".ls1", 1.0), (".ls2", 1.0), (".temp", 1.0), (".D", 0.0), (".conv.b", 0.0)):
        w = {k: (torch.full_like(v, value) if k.endswith(suffix) else v) for k, v in plain.w.items()}
        if any(k.endswith(suffix) for k in w):
            assert differs(w), suffix
    w = {k: (torch.eye(v.shape[0], dtype=v.dtype) if k.endswith(".talk") else v) for k, v in plain.w.items()}
    assert differs(w), "talk"
    other = json.loads(json.dumps(plain.cfg))
    other["postln_alpha"] += 0.5
    assert differs(c=other), "alpha"
    other = json.loads(json.dumps(plain.cfg))
    other["embedding"]["scale"] *= 2
    assert differs(c=other), "embedding scale"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_prompt_then_token_by_token(model, dtype, graphs):
    """The last tokens one by one (state, kept inputs and the row of the token before pass from the prompt's step to the
    single tokens; pages begin and end), against the same positions of the whole prompt."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    eng = engine(plain.folder, dtype, use_graphs=graphs)
    for n, tail in ((150, 80), (41, 40), (200, 3)):
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
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    n = 200
    ids = prompt(9, n, cfg["vocab"])
    eng = engine(plain.folder, dtype)
    slot = eng.new_sequence()
    got = [eng.step([StepEntry(slot, [ids[t]], [0])]).clone() for t in range(n)]
    eng.release(slot)
    assert_rows(torch.cat(got, dim=0), plain(ids), dtype, f"{name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("piece", [2, 5, 64, 100])
def test_prompts_in_pieces(model, dtype, piece):
    """Steps cut into pieces of 2 to 100 tokens (the engine's work space is that small; 2 is fewer than the taps of a
    convolution): two sequences side by side, every place wanted, then a few tokens one by one."""
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
    """Batches of unequal prompts, then one token each until the shorter ones end; later batches get the slots, pages and
    states that earlier ones gave back.  Every request is compared with the plain implementation of it alone, and in 32-bit
    the batched rows equal the rows of the request stepped alone in the same engine."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_that_remembers_hundreds_of_tokens(tmp_path, dtype):
    """Decays close to one: the first three tokens still move the logits 500 tokens later (shown on the plain implementation), in a
    slot that another request used before; whole, and with the tail decoded."""
    from rocml_b200 import StepEntry
    cfg = TIBENEX["TA"]
    folder = write_tibenex(str(tmp_path / "m"), cfg, seed=3, slow_decay=True)
    plain = Folder(folder)
    ids = prompt(21, 520, cfg["vocab"])
    want = plain(ids)
    other = plain([(t + 1) % cfg["vocab"] for t in ids[:3]] + ids[3:])
    assert rel_err(other[-1:], want[-1:]) > 10 * TOL["float32"]
    eng = engine(folder, dtype)
    slot = eng.new_sequence()
    eng.step([StepEntry(slot, prompt(22, 300, cfg["vocab"]), [])])
    eng.release(slot)
    slot = eng.new_sequence()
    got = [eng.step([StepEntry(slot, ids[:480], [479])]).clone()]
    for t in range(480, 520):
        got.append(eng.step([StepEntry(slot, [ids[t]], [0])]).clone())
    eng.release(slot)
    assert_rows(torch.cat(got), want[479:], dtype, f"{dtype} decoded tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model, dtype):
    """A short prompt and 500 tokens one by one under CUDA graphs; the last 40 rows compared."""
    from rocml_b200 import StepEntry
    name, cfg, plain = model
    ids = prompt(77, 520, cfg["vocab"])
    eng = engine(plain.folder, dtype, max_tokens=1024)
    slot = eng.new_sequence()
    eng.step([StepEntry(slot, ids[:20], [])])
    got = []
    for t in range(20, 520):
        r = eng.step([StepEntry(slot, [ids[t]], [0] if t >= 480 else [])])
        if r is not None:
            got.append(r.clone())
    eng.release(slot)
    assert_rows(torch.cat(got), plain(ids)[480:], dtype, f"{name} {dtype}")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(model, dtype):
    """Engine.generate (its scheduler, sampler and run-ahead loop) against greedy decoding with the plain implementation,
    for prompts of unequal length in one batch; compared until the first step whose two best logits are closer than the
    tolerance."""
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
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got2, torch.stack([wa[39], wb[8]])) < TOL["float32"]
    r = subprocess.run([sys.executable, "-m", "rocml_b200", "generate", "--model", f.folder, "--prompt-ids", "1,2,3", "-n", "5"],
                       capture_output=True, text=True, timeout=600, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]


# ---- configurations drawn at random -----------------------------------------------------------------------------

def random_configuration(seed):
    from tiny_models import _ssm, _t, _tattn, _tlat
    g = torch.Generator().manual_seed(2000 + seed)

    def pick(*xs):
        return xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    layers = []
    for i in range(pick(1, 2, 3, 4)):
        kind = pick("mamba2", "mamba2", "attention", "latent_attention")
        if kind == "mamba2":
            groups = pick(1, 2, 3)
            heads = groups * pick(1, 2, 4)
            vdim = pick(4, 8, 24, 64)
            parts = pick(1, 2, heads)
            mixer = _ssm(heads, vdim, pick(4, 16, 40, 128), groups, pick(1, 2, 3, 4, 5), parts)
        elif kind == "attention":
            kv = pick(1, 2, 3)
            dim = pick(8, 16, 32, 64, 40)
            rot_dims = pick(0, dim // 2 - (dim // 2) % 2, dim)
            mixer = _tattn(kv * pick(1, 2, 4), kv, dim, pick(8, 32, 48), pick(0.1, 0.3, 0.7), None if not rot_dims else (pick(100.0, 1e4, 1e6), rot_dims))
        else:
            rot_dim = pick(0, 4, 16, 32)
            rot = None if not rot_dim else ((pick(100.0, 1e4, 5e5),) + (((pick(2.0, 8.0), pick(16, 64, 512), pick(4.0, 32.0), pick(0.5, 1.0)),) if pick(True, False) else ()))
            mixer = _tlat(pick(1, 3, 8), pick(8, 16, 48), rot_dim, pick(8, 24, 64), pick(16, 40, 96), pick(8, 24, 72), pick(0.1, 0.3), rot)
        layers.append(_t(kind, mixer, pick(None, 32, 72)))
    return {"architecture": "Tibenex", "vocab": pick(50, 101, 256), "width": pick(48, 64, 96, 136), "norm": {"eps": pick(1e-6, 1e-5)},
            "postln_alpha": pick(0.5, 1.0, 2.0, 3.5), "embedding": {"scale": pick(1.0, 4.0, 11.0)}, "layers": layers}


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    """A configuration drawn at random: a whole prompt, the same in pieces of 50 with a tail decoded under graphs, and two
    requests side by side, in 32-bit (sharp) and bfloat16."""
    from rocml_b200 import StepEntry
    cfg = random_configuration(seed)
    folder = str(tmp_path / "m")
    write_tibenex(folder, cfg, seed)
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
