"""Gotulorn on the host: the registry, the configuration's keys and errors, which cache each layer gets,
the loader's report, a random-weights folder, and the plain functions against closed forms."""
import copy
import json

import numpy as np
import pytest
import torch

from lgml_b200.cache import PagedKV
from lgml_b200.config import ConfigError, GotulornConfig, architectures, config_from_dict, load_config
from lgml_b200.models import build_model
from lgml_b200.weights import WeightError, index_folder, write_random_model
from lgml_b200.weights.loader import check_index
from tests import gotulorn_helpers as L
from tests.plain import gotulorn_plain as P


def test_registered_and_read_from_its_own_keys():
    assert "Gotulorn" in architectures()
    cfg = config_from_dict(copy.deepcopy(L.MIXED))
    assert isinstance(cfg, GotulornConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers, cfg.embedding_scale) == (97, 64, 6, 6.0)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("edit,word", [
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][0].update(type="conv"), "layers[0].type"),
    (lambda d: d["layers"][0]["mixer"].update(heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=4), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda d: d["layers"][5]["mixer"].update(kv_from=2), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=8), "vdim"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda d: d["layers"][0]["mlp"].update(kind="sparse"), "kind"),
])
def test_errors_name_the_key(edit, word):
    d = copy.deepcopy(L.MIXED)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_a_cache_keeps_what_the_widest_mask_among_its_readers_needs():
    model = build_model(config_from_dict(copy.deepcopy(L.MIXED)))
    layout = model.cache_layout()
    assert sorted(layout) == [0, 1, 3, 4]                    # layers 2 and 5 read the caches of 0 and 3
    assert [c.cache for c in model.schedule] == [None, None, 0, None, None, 3]
    # layer 0: own window 20 / 3 kept; its reader: 70 / 5.  Layer 3: 3 / 0; its reader: 2 / 70
    assert layout[0] == PagedKV(4, 16, 70, 24, keep_first=5, v_heads=2)
    assert layout[3] == PagedKV(6, 8, 3, 8, keep_first=70, v_heads=3)
    assert layout[1] == PagedKV(1, 32, None, 24, v_in_k=True)
    assert model.blocks[0].mixer.window == 20 and model.blocks[2].mixer.window == 70 and model.blocks[5].mixer.keep_first == 70
    free = build_model(config_from_dict(copy.deepcopy(L.NO_WINDOW))).cache_layout()
    assert free[0].window is None and free[0].keep_first == 0


def test_folder_of_random_weights_and_the_loaders_report(tmp_path):
    cfg = config_from_dict(copy.deepcopy(L.ODD))
    folder = write_random_model(tmp_path / "m", cfg, seed=3)
    loaded = load_config(folder)
    assert loaded.to_dict() == cfg.to_dict()
    specs = build_model(loaded).tensor_specs()
    index = index_folder(folder)
    check_index(index, specs)
    names = set(index)
    assert {"embed", "embed.norm", "embed.norm.b", "embed.norm.alpha", "final.norm.alpha", "head", "l0.mix.dkv.norm", "l0.mlp.e0.down",
            "l0.mlp.router.b", "l1.mix.lq1", "l2.mix.k", "l3.mlp.gate"} <= names
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and "l2.norm2" not in names      # a reader projects no keys; no feed-forward, no norm
    assert tuple(index["embed.norm.alpha"].shape) == ()
    index.pop("l1.mix.lk2")
    with pytest.raises(WeightError) as e:
        check_index(index, specs)
    assert "l1.mix.lk2" in e.value.missing


def test_plain_functions_against_closed_forms():
    # dynamic tanh: saturates at +-w + b, linear near 0
    x = np.array([[0.0, 1e-4, 50.0, -50.0]])
    y = P.dyt(x, np.full(4, 2.0), np.full(4, 0.5), 0.3)
    assert np.allclose(y, [[0.5, 0.5 + 2.0 * 0.3e-4, 2.5, -1.5]], atol=1e-9)
    # the mask: position 10 with a window of 3 and 2 kept tokens sees 0, 1, 8, 9, 10
    see = P.window_with_first(12, 3, 2)
    assert list(np.nonzero(see[10])[0]) == [0, 1, 8, 9, 10]
    assert list(np.nonzero(see[2])[0]) == [0, 1, 2] and list(np.nonzero(P.window_with_first(5, 1, 0)[4])[0]) == [4]
    # rotation: a pair at position p turns by p * base^(-2i / dims); entries past dims pass
    v = np.zeros((3, 6)); v[:, 0] = 1.0; v[:, 2] = 1.0; v[:, 4] = 7.0
    r = P.rotate_interleaved(v, 100.0, 4, [0, 1, 2])
    assert np.allclose(r[2], [np.cos(2.0), np.sin(2.0), np.cos(0.2), np.sin(0.2), 7.0, 0.0])
    # equal maps and lambda 1 would cancel; with diff alone the output is the normed (1 - diff) a
    W = {"m.q": np.zeros((8, 4)), "m.k": np.zeros((8, 4)), "m.v": np.eye(4)[:3], "m.o": np.eye(3),
         "m.lq1": np.zeros(4), "m.lk1": np.zeros(4), "m.lq2": np.zeros(4), "m.lk2": np.zeros(4)}
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 1.0, "diff": 0.25}
    h = np.array([[3.0, 0.0, 0.0, 0.0], [0.0, 3.0, 0.0, 0.0]])
    out, _ = P.differential_attention(h, W, "m", m, 0.0)
    a = np.array([[3.0, 0, 0], [1.5, 1.5, 0]])               # uniform maps: running means of v; lambda = 1 - 1 + 0.25
    o = a - 0.25 * a
    assert np.allclose(out, o / np.sqrt((o ** 2).mean(1, keepdims=True)) * 0.75)
    # the router: top 2 of logits (1, 3, 2) are experts 1 and 2 with weights softmax(3, 2)
    Wf = {"f.router": np.array([[1.0], [3.0], [2.0]]), "f.router.b": np.zeros(3)}
    for e in range(3):
        Wf[f"f.e{e}.gate"], Wf[f"f.e{e}.up"], Wf[f"f.e{e}.down"] = np.array([[1.0]]), np.array([[1.0]]), np.array([[float(10 ** e)]])
    y = P.routed_ff(np.array([[1.0]]), Wf, "f", {"router": {"experts": 3, "top": 2}})
    silu = 1.0 / (1.0 + np.exp(-1.0))
    w1, w2 = np.exp(3.0) / (np.exp(3.0) + np.exp(2.0)), np.exp(2.0) / (np.exp(3.0) + np.exp(2.0))
    assert np.allclose(y, [[silu * (w1 * 10.0 + w2 * 100.0)]])
    # the clamped gate: g = min(5, 2) = 2, u = clamp(-9, -2, 2) = -2: 2 sigmoid(3.404) (-2 + 1)
    Wd = {"d.gate": np.array([[5.0]]), "d.up": np.array([[-9.0]]), "d.down": np.array([[1.0]])}
    assert np.allclose(P.dense_ff(np.array([[1.0]]), Wd, "d", {"limit": 2.0}), [[-2.0 / (1.0 + np.exp(-3.404))]])
