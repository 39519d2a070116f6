"""Plain, slow implementation of the Metulix decoder for the tests.

Whole sequences, no cache, one function per mechanism, torch on the CPU in 64-bit.  It shares
no code with the package under test: it reads config.json and the safetensors file with its
own few lines and computes every layer token by token or with dense masks.

The design in this file's notation (h: input of a sublayer, rows are tokens):

    layer       x <- x + LN1(mixer(x));  x <- x + LN2(ff(x))      (norm on the sublayer's OUTPUT)
    LN          (h - mean) / sqrt(var + eps) * w                  (no bias, biased variance)
    lightning   q, k = silu(W_q h), silu(W_k h)  [heads, dim];  v = silu(W_v h)  [heads, vdim]
                S_t = decay_head * S_{t-1} + k_t v_t^T;  o_t = S_t^T q_t
                out = W_o( rms(concat heads of o) * w_norm * sigmoid(W_g h) )
    attention   q, k, v = W h, each then a causal depthwise convolution over time (taps from the
                tensor's shape), q and k then RMS-normed over the WHOLE projection with a weight,
                then rotated in interleaved pairs (2i, 2i+1) on the first rot.dims of each head;
                v divided by its per-head root mean square;  scores (q.k) * scale under the
                mask  j <= i and (i - j < size or j < keep_first);  softmax;  the softmax
                weights of the heads are mixed by T (w'_h = sum_g T[h, g] w_g);  head h applies
                w'_h to the values of its own key/value head;  out = W_o(concat heads).
                A layer with kv_from = j reuses layer j's keys and values.
    ff          W_down( silu(W_gate h + b) * (W_up h + b) ) + b
    output      logits = head LN_final(x)
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
def layer_norm(x, w, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_{t - taps + 1 + j}, zeros before t = 0."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotate_interleaved(x, heads, dim, rot_dims, base, positions):
    """x [T, heads * dim]: pairs (2i, 2i + 1) of the first rot_dims of each head turn by
    position * base^(-2i / rot_dims)."""
    T = len(positions)
    out = x.clone().view(T, heads, dim)
    src = x.view(T, heads, dim)
    pos = torch.tensor(positions, dtype=F64)
    for i in range(rot_dims // 2):
        angle = pos * float(base) ** (-2.0 * i / rot_dims)
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        a, b = src[:, :, 2 * i], src[:, :, 2 * i + 1]
        out[:, :, 2 * i] = a * c - b * s
        out[:, :, 2 * i + 1] = b * c + a * s
    return out.reshape(T, heads * dim)


def visible(i, j, size, keep_first):
    """Whether query position i sees key position j (size 0: no window, every earlier key)."""
    return j <= i and (size <= 0 or i - j < size or j < keep_first)


def lightning_recurrence(q, k, v, decay):
    """q, k [T, heads, dim], v [T, heads, vdim] -> o [T, heads, vdim], and the final state."""
    T, heads, dim = q.shape
    vdim = v.shape[2]
    state = torch.zeros(heads, dim, vdim, dtype=F64)
    out = torch.zeros(T, heads, vdim, dtype=F64)
    for t in range(T):
        for h in range(heads):
            state[h] = decay[h] * state[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = state[h].t() @ q[t, h]
    return out, state


def lightning_mixer(h, w, p, m, eps):
    T = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].t()).view(T, heads, dim)
    k = silu(h @ w[p + "k"].t()).view(T, heads, dim)
    v = silu(h @ w[p + "v"].t()).view(T, heads, vdim)
    o, _ = lightning_recurrence(q, k, v, m["decay"])
    o = rms(o.reshape(T, heads * vdim), eps) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t()


def attention_keys_values(h, w, p, m, eps, positions):
    """Keys as the cache holds them (convolved, normed, rotated) and values (convolved, then
    each head divided by its root mean square)."""
    T, G, dim, vdim = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = causal_conv(h @ w[p + "k"].t(), w[p + "k.conv"])
    k = rms(k, eps) * w[p + "k.norm"]
    k = rotate_interleaved(k, G, dim, m["rot"]["dims"], m["rot"]["base"], positions)
    v = causal_conv(h @ w[p + "v"].t(), w[p + "v.conv"])
    v = rms(v.view(T, G, vdim), eps).reshape(T, G * vdim)
    return k, v


def attention_mixer(h, w, p, m, eps, keys_values=None):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T))
    q = causal_conv(h @ w[p + "q"].t(), w[p + "q.conv"])
    q = rms(q, eps) * w[p + "q.norm"]
    q = rotate_interleaved(q, H, dim, m["rot"]["dims"], m["rot"]["base"], positions).view(T, H, dim)
    if keys_values is None:
        keys_values = attention_keys_values(h, w, p, m, eps, positions)
    k, v = keys_values[0].view(T, G, dim), keys_values[1].view(T, G, vdim)
    mask = m.get("mask") or {}
    size, keep = mask.get("size", 0), mask.get("keep_first", 0)
    see = torch.tensor([[visible(i, j, size, keep) for j in range(T)] for i in range(T)])
    weights = torch.zeros(H, T, T, dtype=F64)
    for hq in range(H):
        scores = (q[:, hq] @ k[:, hq // (H // G)].t()) * m["scale"]
        weights[hq] = torch.softmax(scores.masked_fill(~see, -math.inf), dim=1)
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], weights)
    out = torch.zeros(T, H, vdim, dtype=F64)
    for hq in range(H):
        out[:, hq] = mixed[hq] @ v[:, hq // (H // G)]
    return out.reshape(T, H * vdim) @ w[p + "o"].t(), keys_values


def feed_forward(h, w, p):
    gate = h @ w[p + "gate"].t() + w[p + "gate.b"]
    up = h @ w[p + "up"].t() + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].t() + w[p + "down.b"]


# --------------------------------------------------------------------------------- model
def forward(config, w, ids, layers_out=None):
    """float64 logits [len(ids), vocab]; `layers_out` (a list) receives the residual stream
    after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(ids, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "lightning":
            mixed = lightning_mixer(x, w, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            source = m.get("kv_from")
            mixed, kv = attention_mixer(x, w, p + "mix.", m, eps,
                                        None if source is None else kept[source])
            kept[i] = kv
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(mixed, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].t()


def logits_of(model_dir, ids):
    config, w = load(model_dir)
    return forward(config, w, ids)


def greedy_generate(model_dir, prompt, count):
    config, w = load(model_dir)
    seq, out = list(prompt), []
    for _ in range(count):
        token = int(forward(config, w, seq)[-1].argmax())
        out.append(token)
        seq.append(token)
    return out
