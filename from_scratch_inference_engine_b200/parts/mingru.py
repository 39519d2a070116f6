"""minGRU: an element-wise recurrence over per-request state; gate and candidate of a token come
from that token's projections alone."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, StateNeed, register_part


@register_part("mixer", "mingru")
class MinGru(Mixer):
    """With a = W_z y + b_z and u = W_x y + b_x (`width` channels each): z = sigmoid(a),
    cand = sigmoid(u) for negative u and u + 0.5 otherwise, and per channel
    S_t = S_{t-1} + z (cand - S_{t-1}), written as (1 - z) S_{t-1} + z cand; the mixer returns
    W_o (S_t * silu(W_g y)).

    The state S [width] is float32, zero when a request starts, and lives in the request's state
    slot; gates, candidate and state are computed in 32-bit.  The three projections are one
    matrix product over the stacked weight [z | x | g] (the gate g has no bias: zeros are
    stacked for it).  `names` gives the tensor names below the prefix.
    """

    capturable = True
    CHUNK_TOKENS = 64          # tokens of one chunk when long prompts run chunk-parallel

    NAMES = {"z": "z", "x": "x", "g": "g", "o": "o", "bias": ".b"}

    def __init__(self, prefix: str, hidden_size: int, width: int,
                 names: Optional[Dict[str, str]] = None):
        self.prefix, self.hidden_size, self.width = prefix, int(hidden_size), int(width)
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_in = self.b_in = self.w_o = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, w, n = self.prefix, self.hidden_size, self.width, self.names
        return [TensorSpec(p + n["z"], (w, h)), TensorSpec(p + n["z"] + n["bias"], (w,)),
                TensorSpec(p + n["x"], (w, h)), TensorSpec(p + n["x"] + n["bias"], (w,)),
                TensorSpec(p + n["g"], (w, h)), TensorSpec(p + n["o"], (h, w))]

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.width,), torch.float32)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p, n = self.prefix, self.names
        self.w_in = torch.cat([tensors[p + n[k]] for k in ("z", "x", "g")]).contiguous()
        bz, bx = tensors[p + n["z"] + n["bias"]], tensors[p + n["x"] + n["bias"]]
        self.b_in = torch.cat([bz, bx, torch.zeros_like(bz)]).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        runtime.prepare_weight(self.w_in)
        runtime.prepare_weight(self.w_o)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        proj = rt.linear(y, self.w_in, self.b_in, "mingru.in")
        gated = rt.buffer("mingru.gated", tokens, self.width, proj.dtype)
        chunks = {}
        if int(ctx.h_qlen.max()) > 2 * self.CHUNK_TOKENS:
            # long prompts: the chunks of every request side by side, then each again from the
            # state the chunks before it leave
            tiles = ctx.attention_tiles(1, self.CHUNK_TOKENS)
            chunks = dict(seg_item=tiles.item, seg_row0=tiles.row0, num_segs=tiles.count,
                          seg_tokens=self.CHUNK_TOKENS,
                          seg_ab=ctx.scratch("mingru.seg_ab", 2 * tiles.count * self.width),
                          seg_start=ctx.scratch("mingru.seg_start", tiles.count * self.width))
        ops.mingru_scan(proj, self.width, ctx.item_qstart, ctx.item_qlen, ctx.item_slots,
                        ctx.num_items, cache.state, gated, **chunks)
        return rt.linear(gated, self.w_o, None, "mingru.out")
