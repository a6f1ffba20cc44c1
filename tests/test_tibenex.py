"""Tibenex without a GPU: the configuration, the parts it is spelled as, the tensors it declares, the cache it asks
for, and the plain implementation's own mechanisms."""
import json

import pytest
import torch

import plain_tibenex as P
from tiny_models import TIBENEX, prompt, write_tibenex


def spec_of(cfg):
    from rocml_b200.config import config_from_dict
    return config_from_dict(cfg).to_model_spec()


@pytest.mark.parametrize("name", sorted(TIBENEX))
def test_config_round_trip(name):
    from rocml_b200.config import TibenexConfig, config_from_dict
    cfg = config_from_dict(TIBENEX[name])
    assert isinstance(cfg, TibenexConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert len(cfg.layers) == len(TIBENEX[name]["layers"])


@pytest.mark.parametrize("broken, needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("norm_groups", 5), "norm_groups"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("rot_dim", 7), "rot_dim"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].__setitem__("factor", 0), "factor"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_faults_are_named(broken, needle):
    from rocml_b200.config import config_from_dict
    from rocml_b200.errors import ConfigError
    cfg = json.loads(json.dumps(TIBENEX["TA"]))
    broken(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg).to_model_spec()
    assert needle in str(e.value)


def test_the_architecture_as_parts():
    spec = spec_of(TIBENEX["TA"])
    assert not spec.tie_embeddings and spec.embedding_scale == 3.0 and spec.weight_suffix == "" and spec.bias_suffix == ".b"
    assert all(L.arrangement == "post_norm" for L in spec.layers)
    p = spec.layers[0].arrangement_params
    assert p["alpha"] == 1.7 and p["layer_scale"] and p["token_shift"] and p["names"]["shift"] == "shift"
    kinds = [L.mixer.kind for L in spec.layers]
    assert kinds == ["state_space", "attention", "latent_attention", "state_space"]
    a = spec.layers[1].mixer
    assert a.params["qk_norm"] == "whole" and a.params["talking_heads"] and a.params["head_temperature"]
    assert a.position.kind == "rope_pairs" and a.position.rot_dim == 8
    la = spec.layers[2].mixer
    assert la.params["q_rank"] == 40 and la.params["rot_head_dim"] == 8 and la.position.kind == "rope_neox"
    assert dict(la.position.params["ramp_scaling"])["factor"] == 4.0
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.params["intermediate"] == 96


def test_declared_tensors_and_a_folder(tmp_path):
    from rocml_b200.engine.model import declared_tensors
    from safetensors import safe_open
    cfg = TIBENEX["TC"]
    folder = write_tibenex(str(tmp_path / "m"), cfg, 1)
    decl = {d.name: tuple(d.shape) for d in declared_tensors(spec_of(cfg))}
    with safe_open(f"{folder}/model.safetensors", "pt") as f:
        have = {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()}
    assert have == decl
    assert decl["l0.mix.in"] == (2 * 36 + 2 * 5 + 1, 72) and decl["l0.mix.conv"] == (36 + 10, 1) and decl["l0.mix.conv.b"] == (46,)
    assert decl["l2.mix.talk"] == (9, 9) and decl["l2.mix.temp"] == (9,) and decl["l2.mix.q.norm"] == (108,) and decl["l2.mix.k.norm"] == (36,)
    assert decl["l3.mix.dkv"] == (36 + 12, 72) and decl["l3.mix.uq"] == (5 * 16, 100) and decl["l3.mix.dq.norm"] == (100,)
    assert "l1.norm2" not in decl and "l1.ls2" not in decl and decl["l1.shift"] == (72,) and decl["head"] == (97, 72)


def test_what_the_cache_keeps():
    """Every layer keeps the row of the token before; a state-space layer its state and the convolution's last inputs (none
    with one tap); a latent layer one row a token that holds the latent and the rotated key part."""
    from rocml_b200.cache import SequenceCache
    from rocml_b200.cache.requirements import BundleRequirement, KVRequirement, StateRequirement
    from rocml_b200.engine.model import Model
    from rocml_b200.parts import BuildEnv
    model = Model(spec_of(TIBENEX["TC"]), BuildEnv(torch.device("cpu"), torch.bfloat16))
    reqs = model.cache_requirements()
    assert all(isinstance(r, BundleRequirement) and dict(r.extras)["shift"] == StateRequirement((72,), torch.float32) for r in reqs)
    assert reqs[0].main == StateRequirement((1, 5, 36), torch.float32) and [n for n, _ in reqs[0].extras] == ["shift"]
    assert reqs[4].main == StateRequirement((6, 40, 4), torch.float32) and dict(reqs[4].extras)["conv"] == StateRequirement((6, 24 + 240), torch.float32)
    assert reqs[1].main == KVRequirement(1, 20, None, shared_values=True)
    assert reqs[3].main == KVRequirement(1, 48, None, shared_values=True)
    assert reqs[2].main == KVRequirement(3, 32, None)
    cache = SequenceCache(reqs, model.reads_cache_of(), 256, 4, 1024, torch.bfloat16, "cpu")
    assert [v.kind for v in cache.views] == ["state", "kv", "kv", "kv", "state"]
    assert all(v.extras["shift"].state.shape == (4, 72) for v in cache.views)
    assert cache.views[4].extras["conv"].state.shape == (4, 6, 264) and "conv" not in cache.views[0].extras
    # the five layers' rows of the token before share one group, each with a place of its own
    assert len({v.extras["shift"].index for v in cache.views}) == 5
    s = cache.alloc_slot()
    cache.views[0].state[s].fill_(3.0)
    cache.views[2].extras["shift"].state[s].fill_(3.0)
    cache.free_slot(s)
    assert cache.alloc_slot() == s
    assert float(cache.views[0].state[s].abs().sum()) == 0 and float(cache.views[2].extras["shift"].state[s].abs().sum()) == 0


def test_plain_recurrence_in_pieces_is_the_whole():
    torch.manual_seed(0)
    m = {"heads": 4, "vdim": 6, "state": 5, "groups": 2, "conv": 3, "norm_groups": 2}
    D, inner, gn = 16, 24, 10
    w = {"in": torch.randn(2 * inner + 2 * gn + 4, D).double() * 0.3, "conv": torch.randn(inner + 2 * gn, 3).double(),
         "conv.b": torch.randn(inner + 2 * gn).double(), "dt_bias": torch.randn(4).double(), "A_log": torch.randn(4).double() - 2,
         "D": torch.randn(4).double(), "norm": torch.randn(inner).double(), "o": torch.randn(D, inner).double()}
    h = torch.randn(30, D).double()
    whole = P.mamba2(h, m, w, 1e-6)
    a, S, kept = P.mamba2(h[:11], m, w, 1e-6, return_state=True)
    b, S, kept = P.mamba2(h[11:12], m, w, 1e-6, state=S, conv_before=kept, return_state=True)
    c = P.mamba2(h[12:], m, w, 1e-6, state=S, conv_before=kept)
    assert float((torch.cat([a, b, c]) - whole).abs().max()) < 1e-12


def test_mixing_weights_or_mixing_results():
    """sum_g M[h, g] a_g applied to head h's values equals sum_g M[h, g] (a_g applied to those values)."""
    torch.manual_seed(1)
    H, G, T, d = 6, 3, 9, 4
    a = torch.softmax(torch.randn(H, T, T).double(), dim=-1)
    v = torch.randn(T, G, d).double()
    M = torch.randn(H, H).double()
    kv_of = torch.arange(H) // (H // G)
    first = torch.einsum("hij,jhd->ihd", torch.einsum("hg,gij->hij", M, a), v[:, kv_of])
    every = torch.einsum("gij,jmd->igmd", a, v)                         # head g's weights on stored head m's values
    second = torch.stack([sum(M[h, g] * every[:, g, kv_of[h]] for g in range(H)) for h in range(H)], dim=1)
    assert float((first - second).abs().max()) < 1e-12


def test_token_shift_and_first_token():
    x = torch.arange(12, dtype=torch.float64).reshape(4, 3)
    mu = torch.tensor([0.0, 1.0, 0.5], dtype=torch.float64)
    h = P.token_shift(x, mu)
    assert h[0].tolist() == [0.0, 0.0, 1.0] and h[2].tolist() == [6.0, 4.0, 6.5]
    again = torch.cat([P.token_shift(x[:1], mu), P.token_shift(x[1:], mu, before=x[0])])
    assert torch.equal(again, h)
