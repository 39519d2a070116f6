"""The Zadepel configuration reader and its layout as parts (no GPU needed)."""

import copy

import pytest

import zadepel_models as zm
from from_scratch_inference_engine_b200.config import ConfigError, config_from_dict, load_config
from from_scratch_inference_engine_b200.parts import DecoderModel, tensor_specs


def test_every_size_and_constant_comes_from_the_file():
    config = config_from_dict(zm.CONFIGS["hybrid"])
    spec = config.build_spec()
    assert (spec.architecture, spec.hidden_size, spec.vocab_size) == ("Zadepel", 64, 131)
    assert spec.head_name is None                         # the head is the embedding
    assert [layer.mixer.kind for layer in spec.layers] == [
        "mingru", "scaled_gqa_attention", "latent_attention", "scaled_gqa_attention", "mingru",
        "latent_attention", "scaled_gqa_attention"]
    assert all(layer.arrangement == "sandwich" for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_out_norm is None
    assert spec.layers[0].feed_forward.params["activation"] == "gelu_tanh"
    # the first blending layer is the source, the later ones blend
    assert [spec.layers[i].mixer.params["value_mix"] for i in (1, 3, 6)] == ["source", "mix", "mix"]
    latent = spec.layers[2].mixer.params
    assert (latent["window"], latent["rank"], latent["rope_dim"], latent["scale"]) == (25, 24, 8, 0.5)
    assert spec.layers[5].mixer.params["window"] == 0
    assert spec.layers[2].mixer.params["position"].params["pairing"] == "interleaved"
    assert spec.layers[1].mixer.params["position"].params == {
        "theta": 250000.0, "rotary_dim": 16, "max_position": 0, "pairing": "half"}
    assert config_from_dict(config.to_dict()) == config
    names = {s.name: tuple(s.shape) for s in tensor_specs(spec) if not s.optional}
    assert names["embed"] == (131, 64) and "head" not in names
    assert names["l0.mix.z.b"] == (40,) and names["l0.mix.g"] == (40, 64) and "l0.mix.g.b" not in names
    assert names["l1.mix.q.b"] == (64,) and names["l1.mix.v"] == (24, 64) and names["l1.mix.temp"] == (4,)
    assert names["l1.mix.vmix"] == () and names["l3.mix.vmix"] == ()
    assert names["l2.mix.dkv"] == (32, 64) and names["l2.mix.dkv.norm"] == (24,)
    assert names["l2.mix.uk"] == (32, 24) and names["l2.mix.uv"] == (24, 24) and names["l2.mix.q"] == (48, 64)
    assert names["l2.norm1b"] == (64,) and "l2.norm2" not in names and names["l3.norm2b"] == (64,)
    assert names["l0.mlp.down"] == (64, 96) and names["final.norm"] == (64,)


def test_cache_and_state_needs_follow_the_layers():
    model = DecoderModel(config_from_dict(zm.CONFIGS["hybrid"]).build_spec())
    needs = model.cache_needs()
    assert needs[0] is None and needs[4] is None
    assert (needs[1].kv_heads, needs[1].head_dim, needs[1].v_dim, needs[1].window) == (1, 16, 24, 0)
    assert (needs[2].kv_heads, needs[2].head_dim, needs[2].v_dim, needs[2].window) == (1, 32, 24, 25)
    assert needs[2].values_in_keys and needs[2].stored_value_dim == 0 and not needs[1].values_in_keys
    assert needs[5].window == 0 and needs[5].head_dim == 44
    states = model.state_needs()
    assert states[0].shape == (40,) and states[4].shape == (72,) and states[1] is None


def test_a_model_without_blending_layers_and_one_with_a_single_one():
    data = copy.deepcopy(zm.CONFIGS["attention"])
    for layer in data["layers"]:
        layer["mixer"]["v_mix"] = False
    spec = config_from_dict(data).build_spec()
    assert [layer.mixer.params["value_mix"] for layer in spec.layers] == ["none"] * 3
    assert not any(s.name.endswith("vmix") for s in tensor_specs(spec))
    data["layers"][1]["mixer"]["v_mix"] = True
    spec = config_from_dict(data).build_spec()
    assert [layer.mixer.params["value_mix"] for layer in spec.layers] == ["none", "source", "none"]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "blends its values"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "even and at most 16"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "even and at most 8"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "lacks 'kv_rank'"),
    (lambda c: c["layers"][0].update(type="lstm"), "not a mixer of this design"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "must be 'dense'"),
    (lambda c: c["layers"][0]["mixer"].update(width=0), "at least 1"),
    (lambda c: c.pop("norm"), "'norm' must be an object"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_what_cannot_run_is_refused_with_its_place(change, message):
    data = copy.deepcopy(zm.CONFIGS["hybrid"])
    change(data)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(data)


def test_random_weights_mode_writes_a_folder_the_loader_reads(tmp_path):
    from from_scratch_inference_engine_b200.weights import load_file
    folder = zm.write_model(tmp_path, "odd")
    assert type(load_config(folder)).__name__ == "ZadepelConfig"
    tensors = load_file(folder / "model.safetensors")
    assert tensors["l1.mix.vmix"].shape == () if "l1.mix.vmix" in tensors else True
    assert tensors["l0.mix.dkv"].shape == (5 + 2, 36) and tensors["l2.mix.o"].shape == (36, 19)
