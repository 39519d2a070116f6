"""Small Zadepel configurations for the tests, and folders of random weights for them.

The configurations differ from one another in every size and option: key and value widths that
differ or agree, a rotation over part of a head, over all of it or over nothing, groups of one and
of several query heads per key/value head, windows that end inside a page and layers without one,
layers without a feed-forward, value blending over two and three layers beside a layer that takes
no part in it, one head, widths that are no multiple of eight, a latent rank below and above the
head size, a rope part that is only partly rotated.
"""

from __future__ import annotations

from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, rank, size, scale=None, base=10000.0, rot_dims=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if size is not None:
        mixer["mask"] = {"size": size}
    return {"type": "latent_attention", "mixer": mixer}


def attention(heads, kv_heads, dim, vdim, rot_dims, scale=None, base=10000.0, v_mix=False):
    return {"type": "attention", "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
        "scale": dim ** -0.5 if scale is None else scale, "rot": {"base": base, "dims": rot_dims},
        "v_mix": v_mix}}


def mingru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def with_mlp(layer, ff):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


def model(vocab, width, eps, layers):
    return {"architecture": "Zadepel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


CONFIGS = {
    # latent attention alone: a window that ends inside a page, a rope part of which only four
    # columns turn, a sharp softmax (large scale) so that one key too many or too few at the
    # window's edge changes the result
    "latent": model(97, 40, 1e-5, [
        with_mlp(latent(3, 10, 6, 14, 20, 11, scale=2.0, rot_dims=4), None)]),
    # grouped-query attention alone, three layers: the first gives its values, the second takes
    # no part, the third blends; part of a head rotated; values wider than keys
    "attention": model(83, 48, 1e-6, [
        with_mlp(attention(4, 2, 12, 20, 8, scale=1.5, v_mix=True), None),
        with_mlp(attention(2, 2, 8, 8, 8, scale=1.0, base=500.0), 40),
        with_mlp(attention(6, 2, 16, 20, 4, scale=0.9, v_mix=True), None)]),
    # the recurrence alone
    "mingru": model(71, 24, 1e-6, [with_mlp(mingru(52), 64)]),
    # every mixer, in an order of its own: recurrence first, blending over three layers with a
    # latent layer and another recurrence between them, a latent layer without a window, a
    # layer without feed-forward
    "hybrid": model(131, 64, 1e-6, [
        with_mlp(mingru(40), 96),
        with_mlp(attention(4, 1, 16, 24, 16, scale=0.6, base=250000.0, v_mix=True), 80),
        with_mlp(latent(2, 16, 8, 12, 24, 25, scale=0.5), None),
        with_mlp(attention(2, 1, 8, 24, 0, scale=0.8, v_mix=True), 72),
        with_mlp(mingru(72), 48),
        with_mlp(latent(4, 8, 4, 8, 40, None, scale=0.7, base=100.0), 64),
        with_mlp(attention(3, 1, 32, 24, 32, scale=0.4, v_mix=True), 56)]),
    # sizes that are no multiple of eight, single heads, a window of one key, a rank below the
    # head size
    "odd": model(61, 36, 1e-5, [
        with_mlp(latent(1, 6, 2, 10, 5, 1, scale=0.7), 50),
        with_mlp(attention(1, 1, 6, 10, 6, scale=0.7), 44),
        with_mlp(mingru(19), 30)]),
    # head sizes of real models in small: a window longer than a tile of keys, 8 heads over one
    # latent row, rank 64
    "wide": model(150, 128, 1e-6, [
        with_mlp(latent(8, 32, 16, 32, 64, 70), 160),
        with_mlp(attention(4, 2, 64, 64, 32, v_mix=True), 96),
        with_mlp(mingru(160), None),
        with_mlp(attention(4, 2, 64, 64, 64, v_mix=True), 96)]),
}


def write_model(root, name, seed=0, std=0.08, sharpen=True) -> Path:
    """A folder with config.json and random weights for CONFIGS[name].  With `sharpen` the query
    and key projections are drawn three times as wide, so that scores spread and single keys
    stand out, the temperatures differ from head to head, and the blending weights lie well
    inside (0, 1)."""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import load_file, save_file, write_random_model

    folder = write_random_model(Path(root) / f"zadepel_{name}", config_from_dict(CONFIGS[name]),
                                seed, std, torch.bfloat16)
    tensors = load_file(folder / "model.safetensors")
    generator = torch.Generator().manual_seed(seed + 1000)
    for key in list(tensors):
        if key.endswith(".temp"):
            heads = tensors[key].shape[0]
            tensors[key] = (0.6 + torch.rand(heads, generator=generator)).to(torch.bfloat16)
        elif key.endswith(".vmix"):
            tensors[key] = (0.2 + 0.6 * torch.rand((), generator=generator)).to(torch.bfloat16)
        elif sharpen and key.split(".")[-1] in ("q", "k", "dkv", "uk") and ".mix." in key:
            tensors[key] = (tensors[key].float() * 3.0).to(torch.bfloat16)
    save_file(tensors, folder / "model.safetensors")
    return folder
