"""Linear attention with a per-head decay over per-request state ("lightning attention")."""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, StateNeed, register_part


@register_part("mixer", "lightning_attention")
class LightningAttention(Mixer):
    """q, k = silu(W_q y), silu(W_k y) [heads, dim]; v = silu(W_v y) [heads, vdim]; per head
    S_t = decay_h S_{t-1} + k_t v_t^T and o_t = S_t^T q_t, no other scale; the heads of o
    together are RMS-normed with a gain, multiplied by sigmoid(W_g y) and projected by W_o.

    The state S [heads, dim, vdim] is float32, zero when a request starts, and lives in the
    request's state slot: a step carries it on token by token from where the last one left it.
    The four projections are one matrix product over the stacked weight [q | k | v | g].
    `names` gives the tensor names below the prefix.
    """

    capturable = True
    CHUNK_TOKENS = 64          # tokens of one chunk when long prompts run chunk-parallel

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, vdim: int,
                 decay: Sequence[float], eps: float, names: Optional[Dict[str, str]] = None):
        if len(decay) != heads:
            raise ValueError("lightning_attention: one decay factor per head")
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.dim, self.vdim, self.eps = int(heads), int(dim), int(vdim), float(eps)
        self.decay_values = tuple(float(d) for d in decay)
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.vdim
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_in = self.w_o = self.gain = self.decay = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, n = self.prefix, self.hidden_size, self.names
        return [TensorSpec(p + n["q"], (self.qk_width, h)),
                TensorSpec(p + n["k"], (self.qk_width, h)),
                TensorSpec(p + n["v"], (self.v_width, h)),
                TensorSpec(p + n["g"], (self.v_width, h)),
                TensorSpec(p + n["o"], (h, self.v_width)),
                TensorSpec(p + n["norm"], (self.v_width,), role="vector", init="gain")]

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p, n = self.prefix, self.names
        self.w_in = torch.cat([tensors[p + n[k]] for k in ("q", "k", "v", "g")]).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        self.gain = tensors[p + n["norm"]].to(torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)
        runtime.prepare_weight(self.w_in)
        runtime.prepare_weight(self.w_o)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        proj = rt.linear(y, self.w_in, None, "lightning.in")
        o = rt.buffer("lightning.o", tokens, self.v_width, torch.float32)
        chunks = {}
        if int(ctx.h_qlen.max()) > 2 * self.CHUNK_TOKENS:
            # long prompts: chunks of every request side by side instead of one block per request
            # and head walking all its tokens
            tiles = ctx.attention_tiles(1, self.CHUNK_TOKENS)
            chunks = dict(seg_item=tiles.item, seg_row0=tiles.row0, num_segs=tiles.count,
                          seg_tokens=self.CHUNK_TOKENS,
                          chunk_states=ctx.scratch("lightning.chunk_states",
                                                   tiles.count * self.heads * self.dim * self.vdim))
        # the activations of q, k and v once, in 32-bit: the scan reads each of them several times
        width = 2 * self.qk_width + self.v_width
        act = ops.silu_rows(proj, width, rt.buffer("lightning.act", tokens, width, torch.float32))
        ops.lightning_scan(act, 0, self.qk_width, 2 * self.qk_width, ctx.item_qstart,
                           ctx.item_qlen, ctx.item_slots, ctx.num_items, cache.state, self.decay, o,
                           self.heads, self.dim, self.vdim, **chunks)
        gated = rt.buffer("lightning.gated", tokens, self.v_width, proj.dtype)
        ops.gated_rmsnorm(o, proj, 2 * self.qk_width + self.v_width, self.gain, self.eps, gated)
        return rt.linear(gated, self.w_o, None, "lightning.out")
