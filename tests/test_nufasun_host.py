"""Nufasun without a GPU: configuration (keys, errors, round trip), the model as a specification (the run order of a
looped span, a cache or state per pass, what the stream gains before each pass, norms behind the sublayers),
checkpoint names and shapes, and the plain implementation's own consistency."""
import copy

import pytest
import torch

import nufasun_configs as nc
import plain_nufasun as pn
from llm_steadyinfer_b200.config import ConfigError, config_from_dict, load_config
from llm_steadyinfer_b200.models import Model
from llm_steadyinfer_b200.weights import WeightError
from llm_steadyinfer_b200.weights.loader import load_weights_into


def test_configuration_round_trip_and_spec():
    cfg = config_from_dict(nc.MIXED_A)
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.order == [0, 1, 2, 3, 1, 2, 3, 4] and len(spec.layers) == 5
    assert [l.mixer.kind for l in spec.layers] == ["gated_delta", "diff_attention", "gated_delta", "diff_attention", "diff_attention"]
    assert all(l.arrangement == "sandwich" and l.mixer_post_norm is not None for l in spec.layers)
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_post_norm is None
    assert spec.layers[0].feed_forward.kind == "gated_mlp_limited" and spec.layers[0].feed_forward.params["limit"] == 1.5
    assert [(a.place, a.embedding, a.vector_name, a.row) for a in spec.stream_adds] == [(1, False, "loop.step", 0), (4, True, "loop.step", 1)]
    assert spec.logit_softcap == 12.0 and spec.embedder.params["scale"] == 5.0
    assert spec.layers[4].mixer.params["window"] is None and spec.layers[4].mixer.params["softcap"] == 0.0
    assert spec.layers[3].mixer.position.params == {"head_dim": 16, "rot_dim": 4, "theta": 10000.0}
    # a loop from the first layer, three passes; no loop at all
    b = config_from_dict(nc.MIXED_B).model_spec()
    assert b.order == [0, 1, 0, 1, 0, 1, 2, 3] and [a.place for a in b.stream_adds] == [0, 2, 4]
    assert [a.embedding for a in b.stream_adds] == [False, True, True]
    odd = config_from_dict(nc.ODD).model_spec()
    assert odd.order == [0, 1, 2, 3] and odd.stream_adds == () and odd.stream_vector_shapes is None and odd.logit_softcap == 0.0
    assert [pn.run_order(nc.MIXED_A)[i][0] for i in range(8)] == spec.order


@pytest.mark.parametrize("edit,word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][3]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda d: d["layers"][3]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][0]["mlp"].update(kind="gated"), "kind"),
    (lambda d: d["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda d: d["loop"].update(stop=6), "loop"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_configuration_errors_name_the_key(edit, word):
    d = copy.deepcopy(nc.MIXED_A)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_checkpoint_names_shapes_cache_and_state(tmp_path):
    folder = nc.write_folder(str(tmp_path / "m"), nc.MIXED_A, 3)
    model = Model(load_config(folder), torch.float32, "cpu")
    shapes = model.weight_shapes()
    assert shapes["loop.step"] == (2, 96) and shapes["l1.mix.q"] == (4 * 2 * 32, 96) and shapes["l1.mix.k"] == (2 * 2 * 32, 96)
    assert shapes["l1.mix.v"] == (2 * 16, 96) and shapes["l1.mix.g"] == (4, 96) and shapes["l1.mix.lq2"] == (32,)
    assert shapes["l0.mix.q.conv"] == (2 * 24, 4) and shapes["l0.mix.v.conv"] == (4 * 16, 4) and shapes["l0.mix.norm"] == (16,)
    assert shapes["l0.mlp.gate.b"] == (160,) and shapes["l0.mlp.down.b"] == (96,) and shapes["l0.norm2b"] == (96,)
    assert "l1.norm2" not in shapes and "l1.norm2b" not in shapes and "l1.norm1b" in shapes
    assert set(shapes) == set(nc._tensors(nc.MIXED_A, 0))
    load_weights_into(model, folder)
    needs, states = model.cache_places()
    assert len(needs) == 9 and needs[-1] is None and states[-1] is None      # eight runs and the embedder's place
    # a pass of its own for each run of a looped layer; both maps' keys, one value head for the two
    assert needs[1] == needs[4] and needs[1].num_kv_heads == 4 and needs[1].v_heads == 2 and needs[1].window == 21
    assert needs[1].head_dim == 32 and needs[1].v_dim == 16 and needs[7].window is None
    from llm_steadyinfer_b200.csrc import ops
    assert ops.delta_state_floats(24, 16) == 32 * 16 and ops.delta_state_floats(128, 128) == 128 * 128   # 24 rows: 8 parts of 4 rows; 128: 16 parts of 8
    assert states[0].shape == (4 * 4 * 128 + 3 * (2 * 2 * 24 + 4 * 16),) and states[2] == states[5] and states[1] is None
    lam = model.blocks[1].mixer.lam
    cfg, w = pn.read_model_folder(folder)
    want = (torch.exp((w["l1.mix.lq1"] * w["l1.mix.lk1"]).sum()) - torch.exp((w["l1.mix.lq2"] * w["l1.mix.lk2"]).sum())).item() + 0.2
    assert abs(lam - want) < 1e-5
    # a tensor of another size is refused by name
    bad = copy.deepcopy(nc.MIXED_A)
    bad["layers"][0]["mixer"]["conv"] = 3
    with pytest.raises(WeightError) as e:
        load_weights_into(Model(config_from_dict(bad), torch.float32, "cpu"), folder)
    assert "l0.mix.q.conv" in str(e.value)


def test_plain_delta_rule_against_its_closed_form():
    """With beta = 1 and no decay a key that was written once is read back exactly, and writing it again changes
    nothing; with decay g the stored value fades by g a token."""
    torch.manual_seed(0)
    dk, dv = 6, 4
    k = pn.unit(torch.randn(1, dk, dtype=pn.F64))[0]
    other = torch.randn(dk, dtype=pn.F64)
    other = pn.unit((other - (other @ k) * k)[None])[0]                  # orthogonal to k
    v1, v2 = torch.randn(dv, dtype=pn.F64), torch.randn(dv, dtype=pn.F64)
    keys = torch.stack([k, other, k])
    vals = torch.stack([v1, v2, v1])
    ones = torch.ones(3, dtype=pn.F64)
    o = pn.delta_rule_head(keys, keys, vals, ones, ones)
    assert torch.allclose(o[0], v1 * (1 - 1e-6), atol=1e-5) and torch.allclose(o[1], v2, atol=1e-5) and torch.allclose(o[2], v1, atol=1e-5)
    g = torch.full((3,), 0.5, dtype=pn.F64)
    o = pn.delta_rule_head(torch.stack([k, other, k]), keys, vals, torch.tensor([1.0, 0.0, 0.0], dtype=pn.F64), g)
    assert torch.allclose(o[2], v1 * 0.25, atol=1e-5)                    # written once, faded twice, nothing added since


def test_plain_window_and_rotation():
    torch.manual_seed(1)
    T, dk, dv = 9, 8, 3
    q, k, v = torch.randn(T, dk, dtype=pn.F64), torch.randn(T, dk, dtype=pn.F64), torch.randn(T, dv, dtype=pn.F64)
    one = pn.windowed_softmax_attention(q, k, v, 0.3, 5.0, 1)
    assert torch.allclose(one, v)                                        # a window of one token sees itself only
    full, wide = pn.windowed_softmax_attention(q, k, v, 0.3, 0.0, None), pn.windowed_softmax_attention(q, k, v, 0.3, None, T)
    assert torch.allclose(full, wide)
    # rotation keeps the norm of each pair and the score depends on the distance alone
    pos = torch.arange(T)
    rq, rk = pn.rotate_pairs(q[:, None], pos, 100.0, 4)[:, 0], pn.rotate_pairs(k[:, None], pos, 100.0, 4)[:, 0]
    assert torch.allclose(rq[:, 4:], q[:, 4:]) and torch.allclose(rq[:, :2].norm(dim=-1), q[:, :2].norm(dim=-1))
    shifted = pn.rotate_pairs(q[:1].repeat(T, 1)[:, None], pos + 3, 100.0, 4)[:, 0]
    kk = pn.rotate_pairs(k[:1].repeat(T, 1)[:, None], pos, 100.0, 4)[:, 0]
    s = (shifted * kk).sum(-1)
    assert torch.allclose(s, s[0].expand(T))
