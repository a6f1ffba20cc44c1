"""Safesun without a GPU: the configuration, the parts it is spelled as, the tensors it declares, the cache it
asks for, and the plain implementation's own mechanisms."""
import json
import math

import pytest
import torch

import plain_safesun as P
from tiny_models import SAFESUN, prompt, write_safesun


def spec_of(cfg):
    from rocml_b200.config import config_from_dict
    return config_from_dict(cfg).to_model_spec()


@pytest.mark.parametrize("name", sorted(SAFESUN))
def test_config_round_trip(name):
    from rocml_b200.config import SafesunConfig, config_from_dict
    cfg = config_from_dict(SAFESUN[name])
    assert isinstance(cfg, SafesunConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert len(cfg.layers) == len(SAFESUN[name]["layers"])


@pytest.mark.parametrize("broken, needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", -1), "keep_first"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("v_mix", 1), "v_mix"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("vdim", 24), "v_mix"),          # blended values of two widths
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].__setitem__("factor", 0), "factor"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_faults_are_named(broken, needle):
    from rocml_b200.config import config_from_dict
    from rocml_b200.errors import ConfigError
    cfg = json.loads(json.dumps(SAFESUN["SA"]))
    broken(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg).to_model_spec()
    assert needle in str(e.value)


def test_the_architecture_as_parts():
    """Layer by layer: the arrangement, both norms with weights around zero, and what tells the two mixers apart."""
    spec = spec_of(SAFESUN["SA"])
    assert spec.tie_embeddings and spec.embedding_norm is not None and spec.embedding_norm.weight_offset == 1.0
    assert spec.final_norm.weight_offset == 1.0 and spec.weight_suffix == "" and spec.bias_suffix == ".b"
    assert all(L.arrangement == "parallel_two_norms" and L.mixer_norm.weight_offset == 1.0 for L in spec.layers)
    first, second, third, fourth = (L.mixer.params for L in spec.layers)
    assert first["bias"] == ("q", "k", "v") and first["qk_unit_norm"] and not first["qk_norm"] and first["sink"] == 0.0
    assert second["bias"] is False and second["qk_norm"] and not second["qk_unit_norm"] and second["sink"] is None
    assert (first["window"], first["keep_first"]) == (37, 5) and (third["window"], third["keep_first"]) == (9, 70)
    assert [p["value_mix"] for p in (first, second, third, fourth)] == ["source", "mix", None, "mix"]
    assert all(p["gated"] == "per_value" for p in (first, second, third, fourth))
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.params["activation"] == "silu"
    assert dict(spec.layers[1].mixer.position.params["ramp_scaling"])["fast"] == 8.0 and spec.layers[0].mixer.position.params == {}
    # a layer without a mask sees every earlier key; one without a rotation has no position part
    c = spec_of(SAFESUN["SC"])
    assert c.layers[1].mixer.params["window"] is None and c.layers[1].mixer.params["keep_first"] == 0
    assert c.layers[0].mixer.position.kind == "none"
    assert [L.mixer.params["value_mix"] for L in c.layers] == [None, "source", None]


@pytest.mark.parametrize("name", sorted(SAFESUN))
def test_declared_tensors_are_the_files(name, tmp_path):
    """The random-weights folder holds exactly the declared tensors under the design's names, and the loader's check
    accepts a folder that also carries the blend's number of a layer that does not blend."""
    from safetensors.torch import load_file, save_file
    from rocml_b200.engine.model import Model, declared_tensors
    from rocml_b200.parts import BuildEnv
    from rocml_b200.weights.loader import check_against
    cfg = SAFESUN[name]
    folder = write_safesun(str(tmp_path / "m"), cfg, 1)
    w = load_file(folder + "/model.safetensors")
    decls = declared_tensors(spec_of(cfg))
    assert sorted(w) == sorted(d.name for d in decls)
    assert "embed" in w and "embed.norm" in w and "final.norm" in w and "head" not in w
    for i, L in enumerate(cfg["layers"]):
        two = L["type"] == "attention_2"
        assert (f"l{i}.mix.q.b" in w) == two and (f"l{i}.mix.q.norm" in w) == (not two)
        assert (f"l{i}.norm2" in w) == (L["mlp"] is not None)
        m = L["mixer"]
        assert tuple(w[f"l{i}.mix.g"].shape) == (m["heads"] * m["vdim"], cfg["width"])
        assert tuple(w[f"l{i}.mix.o"].shape) == (cfg["width"], m["heads"] * m["vdim"])
    mixing = [i for i, L in enumerate(cfg["layers"]) if L["mixer"]["v_mix"]]
    for i in range(len(cfg["layers"])):
        assert (f"l{i}.mix.vmix" in w) == (i in mixing[1:])
        if i in mixing[1:]:
            assert tuple(w[f"l{i}.mix.vmix"].shape) == ()
    model = Model(spec_of(cfg), BuildEnv(torch.device("cpu"), torch.bfloat16))
    names = set(w) | {f"l{i}.mix.vmix" for i in range(len(cfg["layers"]))}
    check_against(model.declare(), names, lambda n: tuple(w[n].shape) if n in w else (), model.ignorable(), strict=True)


def test_frequencies_along_a_ramp_by_hand():
    """The ramp form of frequency scaling against numbers worked out by hand, in the part and in the plain implementation."""
    from rocml_b200.parts.position import blend_along_ramp
    base, dims, sc = 100.0, 8, {"factor": 4.0, "original": 40, "fast": 4.0, "slow": 0.5}
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)

    def at(t):
        return dims * math.log(40 / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(at(4.0)), 0), min(math.ceil(at(0.5)), dims - 1)
    assert (lo, hi) == (0, 3)
    ramp = [min(max((i - lo) / (hi - lo), 0.0), 1.0) for i in range(4)]
    want = torch.tensor([f / 4.0 * r + f * (1 - r) for f, r in zip(inv.tolist(), ramp)], dtype=torch.float64)
    got, mag = blend_along_ramp(inv, base, 4.0, 40, 4.0, 0.5)
    assert torch.allclose(got, want, rtol=1e-14) and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-15
    mine, mag2 = P.frequencies({"base": base, "dims": dims, "scaling": sc})
    assert torch.allclose(mine, want, rtol=1e-14) and mag2 == mag
    assert float(got[0]) == 1.0 and abs(float(got[3]) - float(inv[3]) / 4.0) < 1e-15
    # a ramp of no width: every pair from lo on is slow
    got, _ = blend_along_ramp(inv, base, 2.0, 16, 1.0, 1.0)
    lo = max(math.floor(dims * math.log(16 / (2 * math.pi)) / (2 * math.log(base))), 0)
    assert [round(float(a / b), 12) for a, b in zip(got, inv)] == [1.0 if i <= lo else 0.5 for i in range(4)]


def test_the_weights_with_one_more_term():
    s = torch.tensor([[0.3, -1.0, 2.0], [5.0, 0.0, -4.0]], dtype=torch.float64)
    seen = torch.tensor([[True, True, False], [True, True, True]])
    a = P.weights_one_more(s, seen)
    e = torch.exp(s) * seen
    assert torch.allclose(a, e / (1.0 + e.sum(-1, keepdim=True)), rtol=1e-14)
    assert float(a[0, 2]) == 0.0 and float(a.sum(-1).max()) < 1.0
    far = P.weights_one_more(torch.full((1, 3), -80.0, dtype=torch.float64), torch.ones(1, 3, dtype=torch.bool))
    assert float(far.sum()) < 1e-30            # every key far below the extra term: almost nothing is read


def test_the_mask():
    seen = P.visible(list(range(12)), 3, 2)
    for i in range(12):
        for j in range(12):
            assert bool(seen[i, j]) == (j <= i and (i - j < 3 or j < 2))
    assert bool(seen[11, 1]) and not bool(seen[11, 2]) and bool(seen[11, 9]) and not bool(seen[11, 8])


def test_blended_values_reach_later_queries(tmp_path):
    """In the plain implementation itself: a later layer reads (1 - lambda) v + lambda v_first for every key, so
    changing the first blending layer's value projection moves a model whose later layers have lambda near one, and
    a layer that does not say v_mix is untouched by the blend."""
    cfg = SAFESUN["SA"]
    folder = write_safesun(str(tmp_path / "m"), cfg, 4)
    c, w = P.load(folder)
    ids = prompt(3, 50, cfg["vocab"])
    x = P.norm_one_plus(w["embed"][torch.as_tensor(ids)], w["embed.norm"], 1e-6)
    y0, v0 = P.attention(x, w, "l0.mix.", "attention_2", c["layers"][0]["mixer"], 1e-6)
    y1, v1 = P.attention(x, w, "l1.mix.", "attention", c["layers"][1]["mixer"], 1e-6, v_first=v0)
    y1_alone, _ = P.attention(x, w, "l1.mix.", "attention", c["layers"][1]["mixer"], 1e-6)
    assert float((y1 - y1_alone).abs().max()) > 1e-3
    w2 = dict(w)
    w2["l1.mix.vmix"] = torch.tensor(1.0, dtype=torch.float64)
    w2["l1.mix.v"] = torch.zeros_like(w["l1.mix.v"])
    y1_first, _ = P.attention(x, w2, "l1.mix.", "attention", c["layers"][1]["mixer"], 1e-6, v_first=v0)
    w2["l1.mix.vmix"] = torch.tensor(0.0, dtype=torch.float64)
    y1_none, _ = P.attention(x, w2, "l1.mix.", "attention", c["layers"][1]["mixer"], 1e-6, v_first=v0)
    assert float(y1_none.abs().max()) == 0.0 and float(y1_first.abs().max()) > 1e-3


def test_the_cache_keeps_the_pages_of_the_kept_positions():
    """A windowed group with kept first positions: the pages that hold any kept position are never given back, the
    pages between them and the window are, growth and the plan agree, and a freed slot's pages all return."""
    from rocml_b200.cache import SequenceCache
    from rocml_b200.cache.requirements import KVRequirement
    req = KVRequirement(2, 16, window=100, keep_first=70)          # kept: pages 0 and 1
    assert req.kept_pages == 2 and KVRequirement(2, 16, window=100).kept_pages == 0
    cache = SequenceCache([req, KVRequirement(2, 16)], [None, None], 4096, 4, 4096, torch.float32, "cpu", max_step_tokens=256)
    g = cache.kv_groups[0]
    s = cache.alloc_slot()
    total = 0
    for n in (30, 200, 1, 1, 500, 64, 1, 700):
        before = g.pool.n_free
        cache.plan([[(s, n)]])
        cache.grow(s, n)
        cache.commit(s, n)
        total += n
        row = g.table_host[s]
        held = [p for p in range(len(row)) if row[p] >= 0]
        first_needed = max(0, total - 100 + 1) // 64
        assert held == sorted(set(range(min(2, (total + 63) // 64))) | set(range(first_needed, (total + 63) // 64))), (total, held)
        cache.check_invariants()
    # a step cut into pieces: the plan counts what growth then takes, piece by piece
    t = cache.alloc_slot()
    pieces = [[(t, 256)], [(t, 256)], [(t, 256)], [(t, 100)]]
    cache.plan(pieces)
    low = g.pool.n_free
    for piece in pieces:
        for slot, n in piece:
            cache.grow(slot, n)
        low = min(low, g.pool.n_free)
        for slot, n in piece:
            cache.commit(slot, n)
    row = g.table_host[t]
    assert [p for p in range(len(row)) if row[p] >= 0] == [0, 1] + list(range((868 - 99) // 64, (868 + 63) // 64))
    cache.free_slot(s)
    cache.free_slot(t)
    assert g.pool.n_held == 0
    cache.check_invariants()
    # a group sized for a window and a step: the kept pages are part of what a sequence may hold
    small = SequenceCache([req], [None], 100000, 2, 100000, torch.float32, "cpu", max_step_tokens=128)
    assert small.kv_groups[0].n_pages == 2 * ((100 + 128 + 63) // 64 + 1 + 2)
