"""The tests' own small configurations and helpers to write them as model folders.

A and B are the two tiny Qwen3 configurations that differ in every size and option (heads and
groups, head size, sizes that are no power of two, layers, vocabulary, eps, theta, tying,
biases); C adds what A and B lack: no grouping (as many key/value heads as query heads), a
head size of 48, and a sliding window on two of its four layers.
"""
import json
import os

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256,
    "max_position_embeddings": 128, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu", "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 96, "intermediate_size": 208, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 311,
    "max_position_embeddings": 256, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": True, "hidden_act": "silu", "eos_token_id": [5, 9],
}
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 4,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "vocab_size": 199,
    "max_position_embeddings": 320, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
}
# D has the head size (64) and group size (4) that the bfloat16 attention kernels take, so that the
# engine tests run them and not only the plain kernels.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 128, "intermediate_size": 320, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 500,
    "max_position_embeddings": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "attention_bias": False, "hidden_act": "silu",
}
# E has a head size of 128, which the tensor-memory attention kernel takes, and a window on one layer.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 192, "intermediate_size": 256, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 389,
    "max_position_embeddings": 640, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 150, "layer_types": ["full_attention", "sliding_attention"],
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def write_model(folder, cfg_dict, seed, std=None):
    """A model folder with random weights (the library's random-weights mode).  ``std``
    rescales the matrices so that the layers matter more than at N(0, 0.02)."""
    from rocml_b200.config import config_from_dict
    from rocml_b200.weights import write_random_model

    cfg = config_from_dict(cfg_dict)
    write_random_model(folder, cfg, seed)
    if std is not None:
        from safetensors.torch import load_file, save_file
        path = os.path.join(folder, "model.safetensors")
        w = load_file(path)
        for k in w:
            if w[k].dim() == 2:
                w[k] = (w[k].float() * (std / 0.02)).to(torch.bfloat16)
        save_file(w, path)
    return folder


def prompt(seed, n, vocab):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---- Pipilix: small configurations that differ in every size, option and constant ---------------------------------
def _latent(heads, dim, vdim, rank, window, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "mask": {"size": window}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# PA: a loop from the first layer that runs three times, a layer without a feed-forward, unequal layers
PIPILIX_A = {
    "architecture": "Pipilix", "vocab": 200, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6},
    "logit_scale": 0.5, "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [_layer(_latent(4, 16, 8, 32, 9, 0.3), _dense(96)),
               _layer(_latent(2, 24, 40, 24, 70, 0.2), _moe(40, 0.7, 5, 2)),
               _layer(_latent(4, 16, 16, 48, 200, 0.25), None)],
}
# PB: no loop; latents of 64 and 128 (the sizes the bfloat16 attention kernels take), one expert a token of sixteen,
# a window of exactly one page
PIPILIX_B = {
    "architecture": "Pipilix", "vocab": 333, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
    "logit_scale": 1.0,
    "layers": [_layer(_latent(8, 32, 32, 64, 100, 0.18), _moe(64, 2.0, 16, 1)),
               _layer(_latent(3, 64, 48, 128, 64, 0.125), _dense(160)),
               _layer(_latent(9, 16, 24, 64, 300, 0.25), _moe(48, 1.5, 4, 3))],
}
# PC: sizes that are multiples of four only, every expert chosen, a window of one token, a loop that runs once
PIPILIX_C = {
    "architecture": "Pipilix", "vocab": 97, "width": 72, "embedding": {"scale": 7.5}, "norm": {"eps": 3e-5},
    "logit_scale": 3.0, "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [_layer(_latent(3, 12, 20, 20, 1, 0.5), _moe(28, 0.4, 3, 3)),
               _layer(_latent(5, 8, 4, 36, 17, 0.35), _dense(52)),
               _layer(_latent(1, 40, 12, 28, 33, 0.15), _moe(20, 1.0, 7, 2))],
}
# PD: a width that is a multiple of four only, more heads than one block of the decode kernel takes (20 and 17 on
# latents of 64 and 128), a single expert, a window that ends inside the second page, and a layer whose sizes are all odd
PIPILIX_D = {
    "architecture": "Pipilix", "vocab": 150, "width": 100, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "logit_scale": 1.5, "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [_layer(_latent(20, 8, 8, 64, 50, 0.4), _moe(32, 0.9, 1, 1)),
               _layer(_latent(17, 16, 8, 128, 90, 0.3), _dense(64)),
               _layer(_latent(3, 7, 5, 37, 31, 0.45), _moe(9, 1.2, 3, 2))],
}
PIPILIX = {"PA": PIPILIX_A, "PB": PIPILIX_B, "PC": PIPILIX_C, "PD": PIPILIX_D}


def write_pipilix(folder, cfg_dict, seed, std=0.05, sharp=1.0, bias_std=0.5, router_gain=3.0):
    """A Pipilix model folder with random weights.  ``std``: the matrices' standard deviation; ``sharp``
    multiplies the query and key-unfolding matrices, so that the softmax picks few keys and a key wrongly
    seen or missed moves the result; ``bias_std``: the routers' choice biases (large enough to change
    choices); ``router_gain`` multiplies the routers, which spreads the scores (fewer near ties)."""
    from safetensors.torch import load_file, save_file
    write_model(folder, cfg_dict, seed)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    for k in w:
        if w[k].dim() == 2:
            f = std / 0.02
            if k.endswith(".mix.q") or k.endswith(".mix.uk"):
                f *= sharp
            if k.endswith(".mlp.router"):
                f *= router_gain
            w[k] = (w[k].float() * f).to(torch.bfloat16)
        elif k.endswith(".correction"):
            w[k] = (w[k].float() * (bias_std / 0.02)).to(torch.bfloat16)
    save_file(w, path)
    return folder


# ---- Zokelorn: small configurations that differ in every size, option and constant --------------------------------
def _zattn(heads, kv, dim, vdim, block, scale, rot_dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                                          "mask": {"size": block}, "rot": rot}}


def _zdecay(kind, heads, dim, vdim, decay):
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _zmoe(ff, experts, top, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    d = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def _z(layer, mlp):
    return {**layer, "mlp": mlp}


# ZA: a loop from the first layer that runs three times; value heads wider and narrower than key heads; a rotation of
# half of every head with stretched long waves; blocks of 37 positions; groups of experts; a layer without feed-forward
ZOKELORN_A = {
    "architecture": "Zokelorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [_z(_zdecay("lightning", 3, 16, 24, (0.5, 0.9, 0.99)), _dense(96)),
               _z(_zattn(4, 2, 32, 16, 37, 0.3, 16, 10000.0, (4.0, 1.0, 2.0, 64)), _zmoe(24, 6, 2, (3, 2), 40)),
               _z(_zdecay("retention", 2, 24, 8, (0.97, 0.75)), None)],
}
# ZB: no loop; head sizes 64 and 128 (which the bfloat16 attention kernels take), one key/value head for eight query
# heads, blocks of exactly one page, one expert a token of sixteen without groups or a shared expert
ZOKELORN_B = {
    "architecture": "Zokelorn", "vocab": 333, "width": 128, "norm": {"eps": 1e-5},
    "layers": [_z(_zattn(8, 1, 64, 64, 64, 0.125, 64, 1000000.0), _zmoe(64, 16, 1)),
               _z(_zdecay("lightning", 4, 64, 64, (0.999, 0.9, 0.8, 0.95)), _dense(160)),
               _z(_zdecay("retention", 5, 8, 40, (0.9, 0.99, 0.999, 0.5, 0.7)), _zmoe(48, 4, 3, None, 32)),
               _z(_zattn(2, 2, 128, 128, 300, 0.09, 32, 500.0, (8.0, 1.0, 4.0, 256)), _dense(96))],
}
# ZC: sizes that are multiples of four only, head sizes that are no multiple of 16, every expert chosen, every group
# kept, blocks of one position, a loop that runs once, decays of 0 and 1
ZOKELORN_C = {
    "architecture": "Zokelorn", "vocab": 97, "width": 72, "norm": {"eps": 3e-5}, "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [_z(_zattn(3, 3, 20, 28, 1, 0.5, 12, 100.0), _zmoe(28, 4, 4, (2, 2), 16)),
               _z(_zdecay("retention", 1, 40, 12, (1.0,)), _dense(52)),
               _z(_zdecay("lightning", 7, 4, 4, (0.0, 0.3, 0.6, 0.9, 0.95, 0.99, 1.0)), _zmoe(20, 9, 2, (3, 1)))],
}
# ZD: a width that is a multiple of four only, more query heads a key/value head than one block of the decode kernel
# takes, a single expert, key heads of 128 with value heads of 64, no rotation at all, a block that ends inside the
# second page
ZOKELORN_D = {
    "architecture": "Zokelorn", "vocab": 150, "width": 100, "norm": {"eps": 1e-6}, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [_z(_zattn(20, 1, 16, 16, 90, 0.4, 0), _zmoe(32, 1, 1, None, 24)),
               _z(_zattn(6, 2, 128, 64, 130, 0.2, 128, 30000.0, (2.0, 0.5, 3.0, 32)), _dense(64)),
               _z(_zdecay("lightning", 2, 72, 136, (0.98, 0.6)), _zmoe(12, 8, 3, (4, 2), 20))],
}
ZOKELORN = {"ZA": ZOKELORN_A, "ZB": ZOKELORN_B, "ZC": ZOKELORN_C, "ZD": ZOKELORN_D}


def write_zokelorn(folder, cfg_dict, seed, std=0.05, sharp=1.0, router_gain=3.0, fixed_routes=False):
    """A Zokelorn model folder with random weights.  ``std``: the matrices' standard deviation; ``sharp`` multiplies
    the attention layers' query matrices, so that the softmax picks few keys and a key wrongly seen or missed
    moves the result; ``router_gain`` multiplies the routers, which spreads the scores (fewer near ties).
    ``fixed_routes``: every token makes the same choices, by a wide margin: entry 0 of the stream is the same
    large number for every token and stays so (no layer writes to it), and a router's row for expert e is
    c_e times the unit vector 0, the c_e far enough apart that no rounding changes an order."""
    from safetensors.torch import load_file, save_file
    write_model(folder, cfg_dict, seed)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    g = torch.Generator().manual_seed(seed)
    for k in sorted(w):
        if w[k].dim() != 2:
            continue
        f = std / 0.02
        if k.endswith(".mix.q") and cfg_dict["layers"][int(k.split(".")[0][1:])]["type"] == "attention":
            f *= sharp
        if k.endswith(".mlp.router"):
            f *= router_gain
        t = w[k].float() * f
        if fixed_routes:
            if k == "embed":
                t[:, 0] = 4.0 * std         # a few times the other entries: the norm's output there is about 3
            elif k.endswith(".o") or k.endswith(".down"):
                t[0, :] = 0.0
            elif k.endswith(".mlp.router"):
                E = t.shape[0]
                order = torch.randperm(E, generator=g).float()
                t = torch.zeros_like(t)
                t[:, 0] = (order - (E - 1) / 2.0) * min(0.25, 2.0 / E)
        w[k] = t.to(torch.bfloat16)
    save_file(w, path)
    return folder


# ---- Safesun: small configurations that differ in every size, option and constant -------------------------------
def _sattn(kind, heads, kv, dim, vdim, scale, mask, rot, v_mix):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return {"type": kind, "mixer": m}


def _s(layer, ff):
    return {**layer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# SA: value heads narrower and wider than key heads, two key/value heads, rotation of half, a third and all of a head,
# frequencies blended along a ramp, a window shorter than the kept first positions (which cross a page border), a layer
# without feed-forward, a layer that takes no part in the blending of values between two that do
SAFESUN_A = {
    "architecture": "Safesun", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [_s(_sattn("attention_2", 4, 2, 32, 16, 0.3, (37, 5), (10000.0, 16), True), 96),
               _s(_sattn("attention", 4, 2, 16, 16, 0.6, (70, 0), (1000.0, 16, (4.0, 64, 8.0, 1.0)), True), None),
               _s(_sattn("attention", 3, 1, 24, 40, 0.45, (9, 70), (200.0, 8), False), 52),
               _s(_sattn("attention_2", 2, 2, 16, 16, 0.7, (300, 1), (50000.0, 16, (2.5, 32, 4.0, 0.5)), True), 40)],
}
# SB: head sizes 64 and 128 (which the bfloat16 attention kernels take), eight query heads a key/value head, a window
# and kept positions of exactly one page, a window of one position, kept positions as long as the window
SAFESUN_B = {
    "architecture": "Safesun", "vocab": 333, "width": 128, "norm": {"eps": 1e-5},
    "layers": [_s(_sattn("attention", 8, 1, 64, 64, 0.2, (64, 64), (1000000.0, 64), False), 160),
               _s(_sattn("attention_2", 4, 2, 128, 128, 0.08, (150, 3), (30000.0, 32, (8.0, 128, 16.0, 2.0)), True), 64),
               _s(_sattn("attention_2", 8, 2, 64, 128, 0.15, (1, 0), (500.0, 64), True), None),
               _s(_sattn("attention", 2, 2, 128, 128, 0.1, (130, 130), (7000.0, 128, (3.0, 200, 20.0, 1.5)), True), 96)],
}
# SC: sizes that are multiples of four only, head sizes that are no multiple of 16, as many key/value heads as query
# heads, no rotation, a layer that sees every earlier key, a single layer that would blend values (so none does),
# more query heads a key/value head than one block of the decode kernel takes
SAFESUN_C = {
    "architecture": "Safesun", "vocab": 97, "width": 72, "norm": {"eps": 3e-5},
    "layers": [_s(_sattn("attention", 3, 3, 20, 28, 0.5, (1, 1), None, False), None),
               _s(_sattn("attention_2", 6, 1, 12, 12, 0.9, None, (100.0, 12), True), 52),
               _s(_sattn("attention_2", 20, 1, 16, 16, 0.55, (90, 33), (10000.0, 4), False), 28)],
}
SAFESUN = {"SA": SAFESUN_A, "SB": SAFESUN_B, "SC": SAFESUN_C}


def write_safesun(folder, cfg_dict, seed, std=0.06):
    """A Safesun model folder with random weights: matrices of standard deviation ``std``, the stream's norm weights
    around zero (they act as 1 + w), the per-head norm weights around one, biases large enough to matter, the blend's
    shares between a quarter and three quarters."""
    from safetensors.torch import load_file, save_file
    write_model(folder, cfg_dict, seed)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    for k in sorted(w):
        t = w[k].float()
        if t.dim() == 2:
            t = t * (std / 0.02)
        elif k.endswith((".norm1", ".norm2")) or k in ("embed.norm", "final.norm"):
            t = (t - 1.0) * 2.0
        elif k.endswith(".b"):
            t = t * 10.0
        w[k] = t.to(torch.bfloat16)
    save_file(w, path)
    return folder


# ---- Tibenex: layers that normalise after the sum; a state-space mixer, latent attention with a rotated part, attention
# whose heads' weights are mixed -------------------------------------------------------------------------------------------
def _t(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _tlat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot_dim}
        if len(rot) > 1:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[1]))
    return m


def _tattn(heads, kv_heads, dim, vdim, scale, rot):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


# TA: every mixer once and the state-space mixer twice with different sizes; a layer without feed-forward
TIBENEX_A = {
    "architecture": "Tibenex", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 1.7, "embedding": {"scale": 3.0},
    "layers": [_t("mamba2", _ssm(4, 16, 8, 2, 4, 2), 96),
               _t("attention", _tattn(4, 2, 16, 16, 0.3, (10000.0, 8)), None),
               _t("latent_attention", _tlat(4, 16, 8, 24, 24, 40, 0.25, (1000.0, (4.0, 64, 8.0, 1.0))), 52),
               _t("mamba2", _ssm(3, 20, 12, 1, 2, 1), 40)],
}
# TB: head sizes that the bfloat16 attention kernels take (a cached row of 96 + 32 = 128; heads of 64), one key/value head
# (nothing to cross), as many key/value heads as query heads with value heads wider than key heads, a rotation of the whole
# head and none at all, as many groups as heads, alpha 1
TIBENEX_B = {
    "architecture": "Tibenex", "vocab": 333, "width": 128, "norm": {"eps": 1e-5}, "postln_alpha": 1.0, "embedding": {"scale": 1.0},
    "layers": [_t("latent_attention", _tlat(8, 32, 32, 64, 96, 64, 0.1, (500000.0,)), 160),
               _t("attention", _tattn(8, 1, 64, 64, 0.12, (1000000.0, 64)), 64),
               _t("mamba2", _ssm(8, 64, 64, 8, 3, 8), None),
               _t("attention", _tattn(6, 6, 32, 48, 0.2, None), 96)],
}
# TC: sizes that are multiples of four only; one head; a convolution of one tap (nothing to keep); a latent without a
# rotated part; a tiny plain part beside a larger rotated one; three query heads a key/value head; a large alpha
TIBENEX_C = {
    "architecture": "Tibenex", "vocab": 97, "width": 72, "norm": {"eps": 3e-5}, "postln_alpha": 4.0, "embedding": {"scale": 0.5},
    "layers": [_t("mamba2", _ssm(1, 36, 5, 1, 1, 3), 28),
               _t("latent_attention", _tlat(3, 20, 0, 12, 20, 12, 0.4, None), None),
               _t("attention", _tattn(9, 3, 12, 20, 0.5, (300.0, 4)), 52),
               _t("latent_attention", _tlat(5, 4, 12, 8, 36, 100, 0.3, (50.0, (3.0, 32, 4.0, 0.5))), 20),
               _t("mamba2", _ssm(6, 4, 40, 3, 7, 6), None)],
}
TIBENEX = {"TA": TIBENEX_A, "TB": TIBENEX_B, "TC": TIBENEX_C}


def write_tibenex(folder, cfg_dict, seed, std=0.06, slow_decay=False):
    """A Tibenex model folder with random weights: matrices of standard deviation ``std``; norm weights, layer scales and
    temperatures around one; the blend with the token before between 0 and 1; mixing matrices far from the identity; step
    sizes and decays such that the state remembers tens of tokens (``slow_decay``: hundreds)."""
    from safetensors.torch import load_file, save_file
    write_model(folder, cfg_dict, seed)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    g = torch.Generator().manual_seed(seed)
    for k in sorted(w):
        t = w[k].float()
        if k.endswith(".talk"):
            t = torch.eye(t.shape[0]) * 0.7 + 0.3 * torch.randn(t.shape, generator=g)
        elif k.endswith(".conv"):
            t = t * 15.0
        elif t.dim() == 2:
            t = t * (std / 0.02)
        elif k.endswith(".shift"):
            t = torch.rand(t.shape, generator=g)
        elif k.endswith((".ls1", ".ls2", ".temp", ".D")):
            t = 1.0 + 3.0 * (t - 1.0)
        elif k.endswith(".A_log"):
            t = (t - 1.0) * 5.0 - (5.0 if slow_decay else 1.5)
        elif k.endswith(".dt_bias"):
            t = (t - 1.0) * 5.0 - 1.0
        elif k.endswith(".conv.b"):
            t = t * 5.0
        w[k] = t.to(torch.bfloat16)
    save_file(w, path)
    return folder
