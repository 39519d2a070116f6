"""Plain, slow implementation of the Zadepel decoder for the tests.

Whole sequences, no cache, one function per mechanism, torch on the CPU in 64-bit.  It shares
no code with the package under test: it reads config.json and the safetensors file with its
own few lines and computes every layer with dense masks or token by token.

The design in this file's notation (h: input of a sublayer, rows are tokens, p: position):

    layer      x <- x + N1b(mixer(N1(x)));  x <- x + N2b(ff(N2(x)))     N = h / sqrt(mean h^2 + eps) * w
    latent     q = W_q h, per head [nope | rope];  d = W_dkv h = [lat | kr];  c = N(lat) * w_c
               k_nope[head] = W_uk[head] c,  v[head] = W_uv[head] c;  kr is rotated and shared by
               all heads;  s = (q_nope . k_nope + rot(q_rope) . rot(kr)) * scale  over the keys
               j in (i - size, i];  softmax;  out = W_o concat(heads)
               rot here: interleaved pairs (2i, 2i+1), angle p * base^(-2i/dims)
    attention  q, k, v = W h + b;  rot: pairs (i, i + dims/2) of the first `dims` of a head;
               s = (q . k) * scale * temp[head] over j <= i;  softmax;  head h reads key/value
               head h // (heads / kv_heads);  in every value-mixing layer but the first,
               v <- (1 - m) v + m v_src, v_src being what the first of those layers computed as v
               for the same token
    mingru     z = sigmoid(W_z h + b_z);  u = W_x h + b_x;  cand = u + 1/2 (u >= 0), sigmoid(u) (u < 0)
               S_p = (1 - z) S_{p-1} + z cand  (S_{-1} = 0);  out = W_o(S_p * silu(W_g h))
    ff         W_down(gelu_tanh(W_gate h) * (W_up h))
    output     logits = E N_final(x)   with E the embedding table
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- loading
def read_tensors(path):
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        chunk = raw[8 + n + b:8 + n + e]
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(chunk, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(chunk, dtype="<f4").copy())
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(chunk, dtype="<i4").copy())
        else:
            raise ValueError(meta["dtype"])
        out[name] = t.reshape(meta["shape"]).to(F64)
    return out


def load(model_dir):
    model_dir = Path(model_dir)
    return (json.loads((model_dir / "config.json").read_text()),
            read_tensors(model_dir / "model.safetensors"))


# ---------------------------------------------------------------------------- mechanisms
def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def angles(positions, base, dims):
    """[tokens, dims / 2]: position * base^(-2i / dims)."""
    i = torch.arange(dims // 2, dtype=F64)
    return positions.to(F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)[None, :]


def rotate_interleaved(x, positions, base, dims):
    """x [tokens, ..., width]: pairs (2i, 2i + 1) of the first `dims` turn by the angle."""
    if dims == 0:
        return x
    a = angles(positions, base, dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def rotate_half(x, positions, base, dims):
    """x [tokens, ..., width]: pairs (i, i + dims / 2) of the first `dims` turn by the angle."""
    if dims == 0:
        return x
    a = angles(positions, base, dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def masked_softmax(scores, visible):
    """scores [heads, i, j], visible [i, j] bool: softmax over the visible j of every row."""
    scores = scores.masked_fill(~visible[None], float("-inf"))
    return torch.softmax(scores, dim=-1)


def windowed_attention(q, k, v, head_scale, q_pos, k_pos, window=0):
    """q [n, heads, dk], k [m, groups, dk], v [m, groups, dv]; query at position p sees the keys at
    positions j with 0 <= p - j (< window, if one is given); head h reads group h // (heads / groups);
    scores times head_scale[h]."""
    heads, groups = q.shape[1], k.shape[1]
    kk = k.repeat_interleave(heads // groups, dim=1)
    vv = v.repeat_interleave(heads // groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * torch.as_tensor(head_scale, dtype=F64).reshape(-1, 1, 1)
    gap = torch.as_tensor(q_pos)[:, None] - torch.as_tensor(k_pos)[None, :]
    visible = gap >= 0
    if window:
        visible = visible & (gap < window)
    return torch.einsum("hij,jhd->ihd", masked_softmax(scores, visible), vv)


def mingru_states(a, u, start=None):
    """a, u [tokens, width]: the states after every token, from `start` (zeros)."""
    z = torch.sigmoid(a)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    state = torch.zeros(a.shape[1], dtype=F64) if start is None else start.to(F64)
    states = []
    for p in range(a.shape[0]):
        state = (1.0 - z[p]) * state + z[p] * cand[p]
        states.append(state)
    return torch.stack(states)


def latent_attention(h, t, prefix, m, eps, positions):
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    q = (h @ t[prefix + "q"].T).reshape(n, heads, dim + rot_dim)
    q_nope, q_rope = q[..., :dim], q[..., dim:]
    d = h @ t[prefix + "dkv"].T
    c = rms_norm(d[:, :rank], t[prefix + "dkv.norm"], eps)
    k_rope = d[:, rank:]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rope = rotate_interleaved(q_rope, positions, base, dims)
    k_rope = rotate_interleaved(k_rope, positions, base, dims)
    k_nope = (c @ t[prefix + "uk"].T).reshape(n, heads, dim)
    v = (c @ t[prefix + "uv"].T).reshape(n, heads, vdim)
    # every head's keys are its own unrotated part and the shared rotated part side by side
    q_full = torch.cat([q_nope, q_rope], dim=-1)
    k_full = torch.cat([k_nope, k_rope[:, None, :].expand(n, heads, rot_dim)], dim=-1)
    size = (m.get("mask") or {}).get("size", 0)
    o = windowed_attention(q_full, k_full, v, [m["scale"]] * heads, positions, positions, size)
    return o.reshape(n, heads * vdim) @ t[prefix + "o"].T


def attention(h, t, prefix, m, positions, shared):
    """`shared` carries the first value-mixing layer's values through the model."""
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = (h @ t[prefix + "q"].T + t[prefix + "q.b"]).reshape(n, heads, dim)
    k = (h @ t[prefix + "k"].T + t[prefix + "k.b"]).reshape(n, kv_heads, dim)
    v = (h @ t[prefix + "v"].T + t[prefix + "v.b"]).reshape(n, kv_heads, vdim)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q = rotate_half(q, positions, base, dims)
    k = rotate_half(k, positions, base, dims)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = t[prefix + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    o = windowed_attention(q, k, v, m["scale"] * t[prefix + "temp"], positions, positions)
    return o.reshape(n, heads * vdim) @ t[prefix + "o"].T


def mingru(h, t, prefix):
    s = mingru_states(h @ t[prefix + "z"].T + t[prefix + "z.b"], h @ t[prefix + "x"].T + t[prefix + "x.b"])
    return (s * silu(h @ t[prefix + "g"].T)) @ t[prefix + "o"].T


def feed_forward(h, t, prefix):
    return (gelu_tanh(h @ t[prefix + "gate"].T) * (h @ t[prefix + "up"].T)) @ t[prefix + "down"].T


# --------------------------------------------------------------------------------- model
def forward(config, t, tokens, return_layers=False):
    """Logits [tokens, vocab] of one whole sequence (64-bit); with return_layers also the
    residual stream after every layer."""
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    x = t["embed"][ids]
    shared, after = {}, []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = rms_norm(x, t[p + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "latent_attention":
            y = latent_attention(h, t, p + "mix.", m, eps, positions)
        elif kind == "attention":
            y = attention(h, t, p + "mix.", m, positions, shared)
        elif kind == "mingru":
            y = mingru(h, t, p + "mix.")
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, t[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(rms_norm(x, t[p + "norm2"], eps), t, p + "mlp.")
            x = x + rms_norm(y, t[p + "norm2b"], eps)
        after.append(x)
    logits = rms_norm(x, t["final.norm"], eps) @ t["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits


def logits_of(model_dir, tokens):
    config, t = load(model_dir)
    return forward(config, t, tokens)


def greedy(config, t, prompt, new_tokens):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(torch.argmax(forward(config, t, tokens)[-1])))
    return tokens[len(prompt):]
