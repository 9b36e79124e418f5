"""Mivorax without a GPU: configuration (keys, errors, round trip), the model as a specification (shared weights,
layers without a feed-forward, the embedder's state), checkpoint names and shapes, and the plain implementation's
own consistency (a recurrence cut in two equals the whole)."""
import copy
import json
import os

import pytest
import torch

import mivorax_configs as mc
import plain_mivorax as pm
from llm_steadyinfer_b200.config import ConfigError, config_from_dict, load_config
from llm_steadyinfer_b200.models import Model
from llm_steadyinfer_b200.weights import WeightError
from llm_steadyinfer_b200.weights.loader import load_weights_into


def test_configuration_round_trip_and_spec():
    cfg = config_from_dict(mc.MIXED_A)
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.order == [0, 1, 2, 3, 4, 1, 2] and len(spec.layers) == 5
    assert [l.mixer.kind for l in spec.layers] == ["state_space", "attention", "latent_attention", "attention", "state_space"]
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.kind == "dense_mlp"
    assert spec.embedder.kind == "table_pair" and spec.embedder.params["buckets"] == 211
    assert config_from_dict(mc.ONLY_SSM).model_spec().embedder is None


@pytest.mark.parametrize("edit,word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][1]["mixer"].pop("bias_max"), "bias_max"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][5].update(weights_of=5), "weights_of"),
    (lambda d: d["layers"][5].update(weights_of=6), "weights of its own"),
    (lambda d: d["layers"][5]["mixer"].update(dim=64), "differs"),
    (lambda d: d["layers"][0]["mlp"].update(kind="gated"), "kind"),
])
def test_configuration_errors_name_the_key(edit, word):
    d = copy.deepcopy(mc.MIXED_A)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_checkpoint_names_shapes_and_state(tmp_path):
    folder = mc.write_folder(str(tmp_path / "m"), mc.MIXED_A, 3, drop_bias_buckets=True)
    model = Model(load_config(folder), torch.float32, "cpu")
    shapes = model.weight_shapes()
    assert shapes["l1.mix.rel"] == (-1, 4)                 # the checkpoint decides the table's rows
    assert not any(n.startswith(("l5.", "l6.")) for n in shapes)
    assert "l1.norm2" not in shapes and "l0.norm2" in shapes and shapes["bigram"] == (212, 96)
    load_weights_into(model, folder)
    assert model.blocks[1].mixer.dist_bias.shape == (101, 4)
    needs, states = model.cache_places()
    assert len(needs) == 8 and needs[-1] is None and states[-1].dtype == torch.int32
    assert needs[2].value_dim == 0 and needs[2].head_dim == 128 and needs[1].v_dim == 16
    assert states[0].shape == (4 * 16 * 24 + 3 * (96 + 64),) and states[1] is None      # a state of 16 rows needs no padding
    from llm_steadyinfer_b200.csrc import ops
    assert [ops.ssm_padded_state(n, p) for n, p in ((16, 24), (128, 64), (5, 8), (48, 48), (64, 32), (8, 32))] == [16, 128, 8, 64, 64, 8]
    # a table with other rows than the configuration says is refused
    bad = copy.deepcopy(mc.MIXED_A)
    bad["layers"][1]["mixer"]["bias_buckets"] = 20
    bad["layers"][5]["mixer"]["bias_buckets"] = 20
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(bad, f)
    with pytest.raises(WeightError) as e:
        load_weights_into(Model(load_config(folder), torch.float32, "cpu"), folder)
    assert "l1.mix.rel" in str(e.value)


def test_plain_recurrence_and_convolution_compose():
    """The plain scan over a whole sequence equals the scan over its halves with the state handed on (which the
    plain code has no notion of: checked through the linearity of the recurrence)."""
    torch.manual_seed(0)
    T, heads, P, N = 12, 2, 3, 4
    x, B, C = torch.randn(T, heads * P, dtype=pm.F64), torch.randn(T, N, dtype=pm.F64), torch.randn(T, N, dtype=pm.F64)
    dt, a_log, D = torch.rand(T, heads, dtype=pm.F64), torch.randn(heads, dtype=pm.F64), torch.zeros(heads, dtype=pm.F64)
    y = pm.state_space_scan(x, B, C, dt, a_log, D, heads, 1)
    # direct sum: y_t = sum_{s<=t} exp(-rate sum_{s<r<=t} dt_r) dt_s (C_t . B_s) x_s
    for h in range(heads):
        for t in range(T):
            acc = torch.zeros(P, dtype=pm.F64)
            for s in range(t + 1):
                decay = torch.exp(-torch.exp(a_log[h]) * dt[s + 1:t + 1, h].sum())
                acc += decay * dt[s, h] * (C[t] @ B[s]) * x[s, h * P:(h + 1) * P]
            assert torch.allclose(acc, y[t, h * P:(h + 1) * P], atol=1e-12)
    assert pm.distance_bucket(5, 12, 300.0) == 5 and pm.distance_bucket(6, 12, 300.0) == 6
    assert pm.distance_bucket(299, 12, 300.0) == 11 and pm.distance_bucket(10 ** 6, 12, 300.0) == 11
