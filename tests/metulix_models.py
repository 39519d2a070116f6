"""Small Metulix configurations for the tests, and folders of random weights for them.

The configurations differ from one another in every size and option: key and value widths that
differ, a rotation over part of a head, one to four taps, groups of one and of several query
heads per key/value head, windows that end inside a page, kept first tokens that fill more than
a page or none at all, layers without a feed-forward, a layer that reads another layer's keys
under a mask of its own, a layer that rotates nothing, decays of exactly one, widths that are
no multiple of eight.
"""

from __future__ import annotations

from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, taps, rot_dims, size, keep_first, scale=None,
              base=10000.0, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps,
             "scale": dim ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": rot_dims},
             "mask": {"size": size, "keep_first": keep_first}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                           "decay": list(decay)}}


def with_mlp(layer, ff):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


def model(vocab, width, eps, layers):
    return {"architecture": "Metulix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


CONFIGS = {
    # attention alone: values wider than keys, part of a head rotated, a window that ends inside
    # a page, kept first tokens; a sharp softmax (large scale) so that one key too many or too
    # few at the window's edge changes the result
    "attention": model(97, 40, 1e-5, [
        with_mlp(attention(4, 2, 12, 20, 3, 8, 11, 3, scale=2.5), None)]),
    # lightning alone: a decay of one beside fast and slow ones, key size no multiple of four
    "lightning": model(83, 48, 1e-6, [
        with_mlp(lightning(3, 10, 24, (1.0, 0.5, 0.97)), None)]),
    # both kinds, a layer without feed-forward, a reader of layer 1's keys with a wider window
    # and more kept tokens than layer 1 itself has, one tap and four taps
    "hybrid": model(131, 64, 1e-6, [
        with_mlp(lightning(2, 16, 8, (0.9, 0.999)), 96),
        with_mlp(attention(4, 4, 16, 8, 4, 16, 9, 0, scale=1.5), 80),
        with_mlp(lightning(1, 8, 40, (0.75,)), None),
        with_mlp(attention(4, 4, 16, 8, 1, 16, 25, 18, scale=1.0, kv_from=1), 72),
        with_mlp(attention(8, 1, 8, 8, 2, 0, 33, 2), 64)]),
    # head sizes that the tensor-core form of the attention takes in bfloat16 (prompt portions),
    # a reader of layer 0's keys with a wider window
    "wide": model(150, 128, 1e-6, [
        with_mlp(attention(4, 2, 64, 64, 3, 32, 40, 5), 160),
        with_mlp(lightning(2, 16, 32, (0.9, 0.99)), None),
        with_mlp(attention(4, 2, 64, 64, 2, 32, 70, 3, kv_from=0), 96)]),
    # sizes that are no multiple of eight, a single head, a window of one key
    "odd": model(61, 36, 1e-5, [
        with_mlp(attention(1, 1, 6, 10, 2, 6, 1, 2, scale=0.7), 50),
        with_mlp(lightning(1, 6, 5, (0.8,)), 44)]),
}


def write_model(root, name, seed=0, std=0.08, sharpen=True) -> Path:
    """A folder with config.json and random weights for CONFIGS[name].  With `sharpen` the
    matrices that mix heads are drawn wide (every head's weights reach every other head's
    output) and the embedding is scaled up, so that scores spread and single keys stand out."""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import load_file, save_file, write_random_model

    folder = write_random_model(Path(root) / f"metulix_{name}", config_from_dict(CONFIGS[name]),
                                seed, std, torch.bfloat16)
    if sharpen:
        tensors = load_file(folder / "model.safetensors")
        generator = torch.Generator().manual_seed(seed + 1000)
        for key in list(tensors):
            if key.endswith(".talk"):
                heads = tensors[key].shape[0]
                tensors[key] = (torch.eye(heads) * 0.6 + 0.5 * torch.randn(
                    heads, heads, generator=generator)).to(torch.bfloat16)
            elif key == "embed":
                tensors[key] = (tensors[key].float() * 12.0).to(torch.bfloat16)
        save_file(tensors, folder / "model.safetensors")
    return folder
