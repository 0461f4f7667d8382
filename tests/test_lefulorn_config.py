"""Lefulorn on the host: configuration, registry, tensor names, the loader's checks, and the
plain implementation's own mechanisms against closed forms."""
import json
import math

import pytest
import torch

from lgml_b200.config import ConfigError, LefulornConfig, config_from_dict, load_config
from lgml_b200.models import build_model
from lgml_b200.weights import WeightError, check_index, index_folder
from tests import lefulorn_helpers as L
from tests.plain import lefulorn_plain as P


def test_registry_reads_the_architecture_key_and_every_layer():
    cfg = config_from_dict(L.MIXED)
    assert isinstance(cfg, LefulornConfig) and cfg.architecture == "Lefulorn"
    assert cfg.vocab_size == 97 and cfg.hidden_size == 64 and cfg.num_hidden_layers == 6
    model = build_model(cfg)
    kinds = [type(b.mixer).__name__ for b in model.blocks]
    assert kinds == ["ChannelDelta", "SinkAttention", "SinkAttention", "ChannelDelta", "SinkAttention", "SinkAttention"]
    # the value-mixing chain: the first such layer keeps, the later ones mix, the others do neither
    assert [getattr(b.mixer, "v_mix", None) for b in model.blocks] == [None, None, "keep", None, "mix", "mix"]
    assert [b.ffn is not None for b in model.blocks] == [True, False, True, False, True, False]
    att = model.blocks[1].mixer
    assert (att.window, att.temp_coef, att.temp_every, att.scale) == (20, 0.3, 8, 0.2)
    assert model.blocks[4].mixer.window is None
    assert model.logit_scale == 0.5


@pytest.mark.parametrize("name", sorted(L.CONFIGS))
def test_folder_gives_ranks_and_its_tensors_fit(tmp_path, name):
    cfg_d, ranks = L.CONFIGS[name]
    w = L.random_weights(cfg_d, ranks, seed=1)
    folder = L.write_folder(tmp_path / name, cfg_d, w)
    cfg = load_config(folder)
    for i, (ra, rg) in ranks.items():
        assert (cfg.layers[i]["mixer"]["rank_a"], cfg.layers[i]["mixer"]["rank_g"]) == (ra, rg)
    specs = build_model(cfg).tensor_specs()
    check_index(index_folder(folder), specs)            # nothing missing, unexpected or misshaped
    assert {s.name for s in specs if not s.optional} <= set(w)
    # a config built from its own dictionary is the same model
    again = config_from_dict(cfg.to_dict())
    assert again.layers == cfg.layers and again.norm_eps == cfg.norm_eps and again.logit_scale == cfg.logit_scale


def test_loader_names_what_does_not_fit(tmp_path):
    cfg_d, ranks = L.CONFIGS["only_delta"]
    w = L.random_weights(cfg_d, ranks, seed=2)
    del w["l0.mix.dt_bias"]
    w["l1.mix.extra"] = torch.zeros(3)
    w["l1.mix.A_log"] = torch.zeros(5)
    folder = L.write_folder(tmp_path / "bad", cfg_d, w)
    with pytest.raises(WeightError) as e:
        check_index(index_folder(folder), build_model(load_config(folder)).tensor_specs())
    assert e.value.missing == ["l0.mix.dt_bias"] and e.value.unexpected == ["l1.mix.extra"]
    assert [n for n, _, _ in e.value.wrong_shape] == ["l1.mix.A_log"]


def test_sizes_a_mixer_leaves_out():
    d = json.loads(json.dumps(L.ONLY_ATTENTION))
    del d["layers"][1]["mixer"]["kv_heads"], d["layers"][1]["mixer"]["vdim"], d["logit_scale"]
    cfg = config_from_dict(d)
    att = build_model(cfg).blocks[1].mixer
    assert (att.n_kv_heads, att.v_head_dim) == (2, 32) and build_model(cfg).logit_scale is None


def test_config_errors_name_the_key():
    def broken(edit):
        d = json.loads(json.dumps(L.MIXED))
        edit(d)
        return d

    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.heads"):
        config_from_dict(broken(lambda d: d["layers"][1]["mixer"].update(heads=5)))
    with pytest.raises(ConfigError, match=r"layers\[0\]\.type"):
        config_from_dict(broken(lambda d: d["layers"][0].update(type="conv")))
    with pytest.raises(ConfigError, match="scale"):
        config_from_dict(broken(lambda d: d["layers"][1]["mixer"].pop("scale")))
    with pytest.raises(ConfigError, match="first one's"):
        config_from_dict(broken(lambda d: d["layers"][4]["mixer"].update(vdim=16)))
    with pytest.raises(ConfigError, match=r"mask\.size"):
        config_from_dict(broken(lambda d: d["layers"][1]["mixer"].update(mask={"size": 0})))
    with pytest.raises(ConfigError, match="conv"):
        config_from_dict(broken(lambda d: d["layers"][0]["mixer"].pop("conv")))
    with pytest.raises(ConfigError, match="norm"):
        config_from_dict(broken(lambda d: d.pop("norm")))


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from lgml_b200.weights import write_random_model

    d = json.loads(json.dumps(L.ODD))
    d["layers"][1]["mixer"].update(rank_a=6, rank_g=10)
    folder = write_random_model(tmp_path / "rnd", config_from_dict(d), 3)
    cfg = load_config(folder)
    assert cfg.layers[1]["mixer"]["rank_g"] == 10 and cfg.layers[3]["mixer"]["rank_a"] == cfg.default_rank
    check_index(index_folder(folder), build_model(cfg).tensor_specs())


# ---- the plain implementation against closed forms -------------------------------------------

def test_plain_attention_reduces_to_softmax_without_its_extras():
    torch.manual_seed(0)
    T, H, D, Dv = 9, 2, 6, 4
    q, k, v = (torch.randn(T, H, n, dtype=torch.float64) for n in (D, D, Dv))
    out = P.sink_attention(q, k, v, torch.full((H,), -1e9, dtype=torch.float64), 0.5, None, torch.zeros(H, dtype=torch.float64))
    for h in range(H):
        s = (q[:, h] @ k[:, h].T) * 0.5
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        assert torch.allclose(out[:, h], torch.softmax(s, -1) @ v[:, h], atol=1e-12)


def test_plain_sink_and_window_and_slopes():
    # equal scores, sink 0: each of n keys weighs 1 / (n + 1); the window caps n
    T = 7
    q = torch.zeros(T, 1, 3, dtype=torch.float64)
    k = torch.zeros(T, 1, 3, dtype=torch.float64)
    v = torch.ones(T, 1, 1, dtype=torch.float64)
    out = P.sink_attention(q, k, v, torch.zeros(1, dtype=torch.float64), 1.0, 4, torch.zeros(1, dtype=torch.float64))
    want = [min(i + 1, 4) / (min(i + 1, 4) + 1) for i in range(T)]
    assert torch.allclose(out[:, 0, 0], torch.tensor(want, dtype=torch.float64))
    assert torch.allclose(P.distance_slopes(4), torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    # a slope takes slope * distance off the score: with v_j = j the output leans to the near keys
    vj = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    near = P.sink_attention(q, k, vj, torch.full((1,), -1e9, dtype=torch.float64), 1.0, None, torch.tensor([2.0], dtype=torch.float64))
    e = torch.exp(-2.0 * torch.arange(T - 1, -1, -1, dtype=torch.float64))
    assert torch.allclose(near[T - 1, 0, 0], (e * torch.arange(T, dtype=torch.float64)).sum() / e.sum())


def test_plain_temperature_steps():
    t = P.query_temperature(torch.arange(0, 20), 0.5, 8)
    assert float(t[6]) == 1.0 and math.isclose(float(t[7]), 1 + 0.5 * math.log(2)) and math.isclose(float(t[15]), 1 + 0.5 * math.log(3))


def test_plain_delta_rule_stores_and_recalls():
    # no decay, beta 1, orthonormal keys: the state stores every value, and reading with a key gives its value back
    D, Dv = 4, 3
    k = torch.eye(D, dtype=torch.float64)
    v = torch.randn(D, Dv, dtype=torch.float64)
    o = P.gated_delta_rule(k.clone(), k, v, torch.ones(D, dtype=torch.float64), torch.ones(D, D, dtype=torch.float64))
    assert torch.allclose(o, v)
    # writing the same key again with another value replaces the first (the delta), and a decay of
    # one half on the key's channel halves what is recalled before the write corrects it
    k2 = torch.stack([k[0], k[0]])
    v2 = torch.randn(2, Dv, dtype=torch.float64)
    o2 = P.gated_delta_rule(k2.clone(), k2, v2, torch.ones(2, dtype=torch.float64), torch.ones(2, D, dtype=torch.float64))
    assert torch.allclose(o2[1], v2[1])
    half = torch.ones(2, D, dtype=torch.float64)
    half[1, 0] = 0.5
    o3 = P.gated_delta_rule(k2.clone(), k2, v2, torch.tensor([1.0, 0.0], dtype=torch.float64), half)
    assert torch.allclose(o3[1], 0.5 * v2[0])


def test_plain_convolution_is_causal_and_ends_on_the_current_token():
    x = torch.zeros(6, 1, dtype=torch.float64)
    x[2] = 1.0
    taps = torch.tensor([[0.1, 0.2, 0.7]], dtype=torch.float64)
    y = P.causal_conv_silu(x, taps)
    pre = torch.tensor([0, 0, 0.7, 0.2, 0.1, 0], dtype=torch.float64)
    assert torch.allclose(y[:, 0], pre * torch.sigmoid(pre))
