"""The Metulix configuration reader and its layout as parts (no GPU needed), and the plain
implementation's mechanisms against closed forms."""

import copy
import math

import pytest
import torch

import metulix_models as mm
import plain_metulix as plain
from from_scratch_inference_engine_b200.config import ConfigError, config_from_dict
from from_scratch_inference_engine_b200.parts import DecoderModel, tensor_specs


def test_every_size_and_constant_comes_from_the_file():
    config = config_from_dict(mm.CONFIGS["hybrid"])
    spec = config.build_spec()
    assert (spec.architecture, spec.hidden_size, spec.vocab_size) == ("Metulix", 64, 131)
    assert [layer.mixer.kind for layer in spec.layers] == [
        "lightning_attention", "talking_window_attention", "lightning_attention",
        "talking_window_attention", "talking_window_attention"]
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.params["bias"]
    reader = spec.layers[3].mixer.params
    assert (reader["window"], reader["keep_first"], reader["own_keys"]) == (25, 18, False)
    assert spec.resolved_schedule()[3] == (3, 1, False)
    assert config_from_dict(config.to_dict()) == config
    names = {s.name: tuple(s.shape) for s in tensor_specs(spec)}
    assert names["l1.mix.k.conv"] == (64, 4) and names["l1.mix.talk"] == (4, 4)
    assert names["l4.mix.q.norm"] == (64,) and names["l0.mlp.gate.b"] == (96,)
    assert "l3.mix.k" not in names and "l3.mix.v.conv" not in names and "l2.norm2" not in names
    assert names["l2.mix.norm"] == (40,) and names["final.norm"] == (64,)


def test_a_reader_widens_what_the_cache_entry_keeps():
    model = DecoderModel(config_from_dict(mm.CONFIGS["hybrid"]).build_spec())
    needs = model.cache_needs()
    assert needs[0] is None and needs[3] is None
    assert (needs[1].window, needs[1].keep_first, needs[1].v_dim) == (25, 18, 8)
    assert (needs[4].kv_heads, needs[4].window, needs[4].keep_first) == (1, 33, 2)
    states = model.state_needs()
    assert states[0].shape == (2, 16, 8) and states[1].shape == (3, 64 + 64 + 32)
    assert states[3] is None and states[4].shape == (1, 64 + 8 + 8)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "attention layer"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "differs from layer 1"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "one factor per head"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_config_that_cannot_run_is_refused(change, message):
    data = copy.deepcopy(mm.CONFIGS["hybrid"])
    change(data)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(data)


def test_plain_lightning_recurrence_is_the_decayed_sum():
    g = torch.Generator().manual_seed(3)
    q, k = torch.randn(6, 2, 4, generator=g).double(), torch.randn(6, 2, 4, generator=g).double()
    v = torch.randn(6, 2, 5, generator=g).double()
    decay = [0.5, 1.0]
    out, _ = plain.lightning_recurrence(q, k, v, decay)
    for h in range(2):
        for t in range(6):
            want = sum(decay[h] ** (t - s) * float(q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert (out[t, h] - want).abs().max() < 1e-12


def test_plain_convolution_rotation_and_mask():
    u = torch.arange(12, dtype=torch.float64).view(4, 3)
    w = torch.tensor([[1.0, 10.0], [2.0, 20.0], [0.0, 1.0]], dtype=torch.float64)
    y = plain.causal_conv(u, w)
    assert y[0].tolist() == [0.0, 20.0, 2.0]                     # nothing before the first token
    assert y[2].tolist() == [3.0 + 60.0, 2 * 4.0 + 20 * 7.0, 8.0]
    x = torch.tensor([[1.0, 0.0, 5.0, 6.0, 0.0, 2.0, 7.0, 8.0]], dtype=torch.float64)
    r = plain.rotate_interleaved(x, 2, 4, 2, 100.0, [3])
    assert r[0, 2:4].tolist() == [5.0, 6.0] and r[0, 6:8].tolist() == [7.0, 8.0]
    assert abs(r[0, 0] - math.cos(3.0)) < 1e-12 and abs(r[0, 1] - math.sin(3.0)) < 1e-12
    assert abs(r[0, 4] + 2 * math.sin(3.0)) < 1e-12 and abs(r[0, 5] - 2 * math.cos(3.0)) < 1e-12
    assert [j for j in range(12) if plain.visible(10, j, 4, 2)] == [0, 1, 7, 8, 9, 10]
    assert [j for j in range(5) if plain.visible(2, j, 4, 2)] == [0, 1, 2]
