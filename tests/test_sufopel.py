"""CPU: the Sufopel decoder's configuration, the model as data, its loader, and the plain implementation's pieces on
inputs whose answers are known."""
import json
import math

import numpy as np
import pytest
import torch

from mashbox_b200.config.registry import read_config
from mashbox_b200.config.sufopel import SufopelConfig
from mashbox_b200.errors import ConfigError, WeightError
from mashbox_b200.models.model import Model
from tests import sufopel_helpers as S
from tests.plain import sufopel as plain


@pytest.mark.parametrize("name", list(S.CONFIGS))
def test_configuration_round_trip(name):
    cfg = S.CONFIGS[name][0]
    entry, back = read_config(json.loads(json.dumps(cfg.to_hf())))
    assert entry.name == "Sufopel" and back == cfg


def test_configuration_refusals():
    good = S.SUF_T.to_hf()

    def broken(change):
        c = json.loads(json.dumps(good))
        change(c)
        return c
    for change, word in ((lambda c: c["layers"][0].update(type="other"), "type"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_rank=48), "another size"),
                         (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
                         (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "router"),
                         (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=5), "router"),
                         (lambda c: c["layers"][1]["mlp"].update(kind="other"), "kind"),
                         (lambda c: c.pop("max_positions"), "max_positions"),
                         (lambda c: c.pop("norm"), "eps")):
        with pytest.raises(ConfigError, match=word):
            SufopelConfig.from_hf(broken(change))


def test_absent_keys_mean_absent_parts():
    c = S.SUF_U.to_hf()
    assert "token_side" not in c and "conv" not in c["layers"][1]["mixer"] and c["layers"][2]["mlp"] is None
    cfg = SufopelConfig.from_hf(c)
    names = read_config(c)[0].stored_tensors(cfg)
    assert "side.embed" not in names and "l1.mix.q.conv" not in names and "l2.mix.q.conv" in names
    assert "l2.norm2" not in names and "l2.ls2" not in names and "l3.mix.dkv" not in names and "l0.mix.dkv" in names
    del c["layers"][1]["mlp"]["router"]["groups"]           # no groups: every expert may be chosen
    assert SufopelConfig.from_hf(c).layers[1].mlp.groups == 1


def test_model_as_data():
    cfg = S.SUF_T
    entry, _ = read_config(cfg.to_hf())
    model = Model(entry.model_spec(cfg), cfg)
    runs = model.schedule
    assert [(r.layer, r.cache, r.write, r.state_id) for r in runs] == [(0, None, False, 0), (1, 1, True, 1),
                                                                      (2, None, False, 2), (3, 1, False, 1)]
    needs, states = model.cache_needs()
    assert list(needs) == [1] and needs[1].kind == "full" and needs[1].tensors == ((1, 40),)
    # a delta layer keeps the last taps - 1 rows of its q/k/v product and a (dim, vdim) matrix per head
    assert states[0].shape == (3 * (2 * 2 * 16 + 4 * 24) + 4 * 16 * 24,)
    assert states[2].shape == (1 * (2 * 2 * 24 + 2 * 16) + 2 * 24 * 16,)
    assert 1 not in states and 3 not in states
    assert model.graph_safe and model.context_limit() == cfg.max_positions and model.portion_alignment() == 1
    wanted = {w.name for w in model.wants()}
    stored = set(entry.stored_tensors(cfg))
    canon = entry.canonical_names(cfg)
    assert {canon(n)[0] for n in stored} == wanted


def test_loader_reads_inner_widths_from_the_tensors(tmp_path):
    """the inner widths of a delta layer's low-rank products are in no key of config.json"""
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.weights.safetensors_io import SafetensorsSource
    folder = S.make_folder(tmp_path, "T")
    c = json.load(open(folder + "/config.json"))
    for layer in c["layers"]:
        layer["mixer"].pop("a_rank", None)
        layer["mixer"].pop("g_rank", None)
    src = SafetensorsSource(folder)
    model = build_model(c, src, "float32", "cpu")
    mixer = model.layers[0].mixer
    assert mixer.w_low.shape == (4 + 8 + 12, 64) and mixer.w_wide.shape == (4 * 16 + 4 * 24, 4 + 8 + 12)
    assert torch.equal(mixer.w_wide[:64, :4], torch.zeros(64, 4)) and torch.equal(mixer.w_wide[64:, 4:12], torch.zeros(96, 8))
    c["layers"][0]["mixer"]["heads"] = 8
    with pytest.raises(WeightError, match="wrong shape"):
        build_model(c, src, "float32", "cpu")
    src.close()


# ------------------------------------------------------------------------------------------------ the plain pieces
def test_plain_delta_rule_on_known_cases():
    dim, vdim = 3, 2
    e = torch.eye(dim, dtype=torch.float64)
    one = torch.ones(dim, dtype=torch.float64)
    # write v under key e0 with beta 1, read it back with the same key: the read-out sees the token's own write
    v = torch.tensor([[2.0, -1.0]], dtype=torch.float64)
    o = plain.delta_rule(e[:1], e[:1], v, one[None], torch.ones(1, dtype=torch.float64))
    assert torch.allclose(o, v)
    # a second write under the same key replaces the first (u = v - S^T k), another key does not disturb it
    q = torch.stack([e[0], e[1], e[0], e[0]])
    k = torch.stack([e[0], e[1], e[0], e[1]])
    v = torch.tensor([[1.0, 1.0], [5.0, 5.0], [3.0, 4.0], [7.0, 7.0]], dtype=torch.float64)
    o = plain.delta_rule(q, k, v, one.expand(4, dim), torch.ones(4, dtype=torch.float64))
    assert torch.allclose(o, torch.tensor([[1.0, 1.0], [5.0, 5.0], [3.0, 4.0], [3.0, 4.0]], dtype=torch.float64))
    # the decay acts per key channel, before the token's write: channel 0 halves each step, channel 1 stays
    g = torch.tensor([[0.5, 1.0, 1.0]], dtype=torch.float64).expand(3, dim)
    k = torch.stack([e[0] + e[1], torch.zeros(dim, dtype=torch.float64), torch.zeros(dim, dtype=torch.float64)])
    v = torch.tensor([[1.0, 0.0], [0.0, 0.0], [0.0, 0.0]], dtype=torch.float64)
    o = plain.delta_rule(torch.stack([e[0], e[0], e[1]]), k, v, g, torch.ones(3, dtype=torch.float64) * 0.5)
    assert torch.allclose(o[:, 0], torch.tensor([0.5, 0.25, 0.5], dtype=torch.float64))


def test_plain_routing_on_known_cases():
    W = {"l.mlp.router": torch.eye(6, dtype=torch.float64) * 4.0,
         "l.mlp.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.9, -3.0, -3.0, 0.8, -3.0]], dtype=torch.float64)
    r = dict(experts=6, top=2, groups=dict(count=2, keep=1))
    chosen, weight = plain.route(W, "l.", r, h)
    assert sorted(chosen[0].tolist()) == [0, 1]                    # group 0 (two strong) beats group 1 (one strong)
    assert torch.allclose(weight[0].sort().values, torch.sigmoid(torch.tensor([3.6, 4.0], dtype=torch.float64)))
    # the correction moves the choice, not the weights
    W["l.mlp.correction"] = torch.tensor([0.0, 0.0, 0.0, 2.0, 0.0, 2.0], dtype=torch.float64)
    chosen, weight = plain.route(W, "l.", r, h)
    assert sorted(chosen[0].tolist()) == [3, 5]
    assert torch.allclose(weight[0], torch.sigmoid(torch.tensor([-12.0, -12.0], dtype=torch.float64)))
    # negative choice scores: an expert outside the kept group counts as minus infinity, not as 0
    W["l.mlp.correction"] = torch.full((6,), -3.0, dtype=torch.float64)
    chosen, _ = plain.route(W, "l.", r, h)
    assert sorted(chosen[0].tolist()) == [0, 1]
    chosen, _ = plain.route(W, "l.", dict(experts=6, top=3, groups=dict(count=3, keep=2)), h)
    assert sorted(chosen[0].tolist()) == [0, 1, 4]                 # groups {0,1} and {4,5}; 4 beats 5


def test_plain_expert_clamps():
    W = {"l.mlp.e0.gate": torch.tensor([[1.0], [1.0]], dtype=torch.float64),
         "l.mlp.e0.up": torch.tensor([[1.0], [-1.0]], dtype=torch.float64),
         "l.mlp.e0.down": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)}
    y = plain.expert(W, "l.", 0, torch.tensor([[5.0]], dtype=torch.float64), 2.0)[0]
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y, torch.tensor([g * 3.0, g * -1.0], dtype=torch.float64))
    y = plain.expert(W, "l.", 0, torch.tensor([[-5.0]], dtype=torch.float64), 2.0)[0]     # the gate has no lower clamp
    g = -5.0 / (1.0 + math.exp(1.702 * 5.0))
    assert torch.allclose(y, torch.tensor([g * -1.0, g * 3.0], dtype=torch.float64))


def test_plain_latent_attention_is_causal_and_needs_only_the_latents():
    cfg, tmp_seed = S.SUF_T, 3
    g = torch.Generator().manual_seed(tmp_seed)
    m = dict(heads=3, dim=16, vdim=24, scale=0.3)
    W = {"l.mix." + n: torch.randn(*s, generator=g, dtype=torch.float64) * 0.2 for n, s in
         dict(dq=(40, 64), uq=(48, 40), uk=(48, 40), uv=(72, 40), g=(72, 64), o=(64, 72)).items()}
    W["l.mix.dq.norm"] = torch.ones(40, dtype=torch.float64)
    h = torch.randn(9, 64, generator=g, dtype=torch.float64)
    c = torch.randn(9, 40, generator=g, dtype=torch.float64)
    full = plain.latent_attention(W, "l.", m, h, c, 1e-5)
    c2 = c.clone()
    c2[6:] += 1.0                                                  # later latents do not reach earlier positions
    assert torch.allclose(plain.latent_attention(W, "l.", m, h, c2, 1e-5)[:6], full[:6])
    assert not torch.allclose(plain.latent_attention(W, "l.", m, h, c2, 1e-5)[6:], full[6:])


def test_plain_model_runs_and_side_input_matters(tmp_path):
    folder = S.make_folder(tmp_path, "T")
    (p,) = S.prompts_for("T", (30,))
    lg = S.plain_logits(folder, p)
    assert lg.shape == (30, 131) and np.isfinite(lg).all()
    cfg, W = S._model(folder)
    W2 = dict(W)
    W2["side.embed"] = W["side.embed"] * 0.0
    assert np.abs(plain.forward(cfg, W2, p).numpy() - lg).max() > 1e-3
