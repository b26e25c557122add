"""CPU: the Luzosun configuration reader, its model as data, the cache manager's handling of masks of blocks of
positions and of shared caches, and the plain implementation's own pieces."""
import numpy as np
import pytest
import torch

from mashbox_b200.cache.manager import CacheManager, CacheNeed
from mashbox_b200.config.luzosun import LuzosunConfig
from mashbox_b200.config.registry import read_config
from mashbox_b200.errors import ConfigError
from mashbox_b200.models.model import Model
from tests import luzosun_helpers as L
from tests.plain import luzosun as plain


@pytest.mark.parametrize("name", list(L.CONFIGS))
def test_config_round_trip_and_tensor_table(name):
    cfg = L.CONFIGS[name][0]
    entry, back = read_config(cfg.to_hf())
    assert back == cfg and entry.name == "Luzosun"
    model = Model(entry.model_spec(cfg), cfg)
    wants = {w.name: tuple(w.shape) for w in model.wants()}
    stored = {n: tuple(s) for n, (s, _) in entry.stored_tensors(cfg).items()}
    assert wants == stored
    canonical = entry.canonical_names(cfg)
    assert canonical("embed") == ("embed", None)
    with pytest.raises(KeyError):
        canonical("l0.mix.nothing")
    assert model.graph_safe


def test_schedule_caches_and_state():
    cfg = L.LUZ_P
    entry, _ = read_config(cfg.to_hf())
    model = Model(entry.model_spec(cfg), cfg)
    runs = model.schedule
    assert [(r.cache, r.write, r.state_id) for r in runs] == [(0, True, 0), (0, False, 1), (2, True, 2), (2, False, 3)]
    needs, states = model.cache_needs()
    # layer 1 reads layer 0's cache with blocks of 40 where layer 0 has 20: the cache keeps the larger block
    assert needs[0] == CacheNeed("chunk", ((2, 32), (2, 40)), 40)
    assert needs[2] == CacheNeed("chunk", ((2, 48), (2, 24)), 48)
    D = cfg.width
    # state: (canon taps - 1) rows of the width, then (conv taps - 1) rows of the projections the layer has
    assert states[0].shape == (1 * D + 2 * (6 * 32 + 2 * 32 + 2 * 40),)
    assert states[1].shape == (1 * D + 1 * (6 * 32),)
    assert states[3].shape == (1 * D + 4 * (2 * 48),)


def test_filters_of_one_tap_and_no_filters():
    """a convolution of one tap exists (its tensor is read) and keeps no state; an absent one has no tensor"""
    cfg = L.LUZ_S
    entry, back = read_config(cfg.to_hf())
    assert back == cfg and "conv" not in cfg.to_hf()["layers"][0]["mixer"] and cfg.to_hf()["canon"] == {"taps": 1}
    model = Model(entry.model_spec(cfg), cfg)
    wants = {w.name: tuple(w.shape) for w in model.wants()}
    assert wants["l0.canon1"] == (40, 1) and "l0.mix.q.conv" not in wants and wants["l1.mix.q.conv"] == (2 * 2 * 8, 2)
    needs, states = model.cache_needs()
    assert 0 not in states and states[1].shape == (1 * 2 * 2 * 8,)          # layer 0 carries nothing, layer 1 its q rows
    assert needs[0].kind == "full"                                           # blocks of 3 and of 7: every position is kept
    q = L.LUZ_Q
    entry, back = read_config(q.to_hf())
    assert back == q and back.layers[2].mixer.conv == 1 and back.layers[2].mixer.mask_size == 1 and back.layers[2].mixer.diff == 0.0
    assert back.layers[0].mixer.conv is None and back.canon_taps == 0


def test_config_refusals():
    good = L.LUZ_P.to_hf()
    for change, word in ((lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
                         (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
                         (lambda c: c["layers"][1]["mixer"].update(vdim=8), "other sizes"),
                         (lambda c: c["layers"][0].update(type="recurrent"), "type"),
                         (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
                         (lambda c: c.pop("width"), "width")):
        import copy
        c = copy.deepcopy(good)
        change(c)
        with pytest.raises(ConfigError, match=word):
            LuzosunConfig.from_hf(c)


def test_merged_needs():
    t = ((2, 32), (2, 40))
    a, b = CacheNeed("chunk", t, 64), CacheNeed("chunk", t, 128)
    assert a.merged(b) == b.merged(a) == b
    assert a.merged(CacheNeed("chunk", t, 96)) == CacheNeed("full", t, None)
    assert a.merged(CacheNeed("full", t, None)) == CacheNeed("full", t, None)
    assert a.merged(CacheNeed("chunk", ((2, 32), (2, 32)), 64)) is None


def test_chunk_group_gives_pages_back_when_a_block_is_left():
    need = CacheNeed("chunk", ((1, 8), (1, 8)), 20)           # blocks of 20 positions, pages of 8
    m = CacheManager({0: need}, {}, page_size=8, num_pages=8, max_requests=2, max_context=400)
    m.admit("a")
    held = []
    for step in range(60):                                     # 60 single tokens: three blocks
        m.extend("a", 1)
        m.commit("a", 1)
        length = m.length("a")
        first = (length // 20 * 20) // 8                       # the page the current block starts in
        row = m.groups[0].table[m.get("a").row]
        assert all(row[b] < 0 for b in range(first)) and all(row[b] >= 0 for b in range(first, -(-length // 8)))
        held.append(m.pages_held("a")[0])
        m.check()
    assert max(held) <= 4 and m.pages_to_hold(400, 1) == [min(50, -(-(19 + 1) // 8) + 1)]
    # a portion that crosses two block borders at once
    m.admit("b")
    m.extend("b", 17)
    m.commit("b", 17)
    m.extend("b", 30)                                          # positions 17 .. 46: needs pages 2 .. 5
    m.commit("b", 30)
    assert m.length("b") == 47 and m.pages_held("b") == [1]    # block 40 .. 59 starts in page 5
    m.release("a")
    m.release("b")
    assert m.free_pages() == [8]
    m.check()


def test_plain_block_mask_and_convolution():
    m = plain.block_mask(7, 3)
    want = [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0],
            [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]]
    assert m.int().tolist() == want
    assert plain.block_mask(4, None).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    assert plain.causal_conv(u, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def test_plain_activation_and_rotation():
    z = torch.tensor([-2.0, 0.0, 1.5], dtype=torch.float64)
    sp = lambda t: np.log1p(np.exp(t))
    got = plain.xielu(z, 0.3, -0.2)
    want = [(0.5 + sp(-0.2)) * (np.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, sp(0.3) * 2.25 + 0.75]
    assert np.allclose(got.numpy(), want, rtol=1e-12)
    f = plain.rotary_frequencies(100.0, 4, 2.0)
    assert np.allclose(f, [0.5, 0.05], rtol=1e-6)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)
    y = plain.rotate_halves(x, [3], f)[0, 0]
    a0, a1 = 1.5, 3 * float(f[1])
    want = [np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + np.sin(a0),
            4 * np.cos(a1) + 2 * np.sin(a1), 5.0]
    assert np.allclose(y.numpy(), want, rtol=1e-6)


def test_rotary_part_divides_by_the_factor():
    from mashbox_b200.parts.position import RotaryEncoding
    for base, dims, factor in ((30000.0, 40, 2.0), (10000.0, 8, 3.0), (500.0, 64, None)):
        part = RotaryEncoding(head_dim=dims + 8, rotary_dim=dims, theta=base, pairing="halves",
                              scaling=("divide", factor) if factor else None)
        assert np.allclose(part.frequencies(), plain.rotary_frequencies(base, dims, factor), rtol=3e-7, atol=0)


def test_random_folder_loads_and_one_error_lists_everything_wrong(tmp_path):
    """the command line's random-weights mode writes a folder the loader reads back; a tensor too many, one too few
    and one of the wrong shape come out in ONE error"""
    import json
    import math
    import os

    from mashbox_b200.cli import main as cli
    from mashbox_b200.engine.loading import build_model, read_config_file
    from mashbox_b200.errors import WeightError
    from mashbox_b200.weights.safetensors_io import DictSource, SafetensorsSource
    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(L.LUZ_P.to_hf()))
    folder = str(tmp_path / "model")
    assert cli(["random", folder, "--config", str(cfg_path), "--seed", "3", "--store", "float32"]) == 0
    source = SafetensorsSource(folder)
    model = build_model(read_config_file(folder), source, "float32", "cpu")
    mixer = model.layers[1].mixer
    assert mixer.shares_kv and mixer.w.shape == (6 * 32, 64) and mixer.wconv.shape == (2, 6 * 32)
    t = {n: source.get(n).double() for n in ("l1.mix.lq1", "l1.mix.lk1", "l1.mix.lq2", "l1.mix.lk2")}
    lam = math.exp(float((t["l1.mix.lq1"] * t["l1.mix.lk1"]).sum())) - math.exp(float((t["l1.mix.lq2"] * t["l1.mix.lk2"]).sum())) + 0.1
    assert abs(mixer.lam - lam) < 1e-12
    assert model.layers[1].ffn is None and model.layers[1].norm2 is None
    tensors = {n: source.get(n) for n in source.names()}
    source.close()
    tensors["l1.mix.k"] = torch.zeros(64, 64)                  # a borrowing layer has no key projection
    del tensors["l2.canon1"]
    tensors["l0.mlp.act"] = torch.zeros(3)
    with pytest.raises(WeightError) as e:
        build_model(L.LUZ_P.to_hf(), DictSource(tensors), "float32", "cpu")
    msg = str(e.value)
    assert "l2.canon1" in msg and "l1.mix.k" in msg and "l0.mlp.act" in msg
