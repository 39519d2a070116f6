"""Windowed attention with mixed heads behind a short convolution of the projections."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, StateNeed, build_part, register_part


@register_part("mixer", "talking_window_attention")
class TalkingWindowAttention(Mixer):
    """Grouped-query attention with these steps, in this order:

    * q, k, v projections without bias (one product over the stacked weight);
    * a causal convolution over time on every channel of q, k and v (`taps` taps, weights
      [channels, taps], zeros before the sequence starts); the last taps - 1 projected rows of a
      request are part of its state;
    * RMS norm of the whole q row and of the whole k row with gains; rotation of q and k by
      `position` (the pairing is the part's); every head of v divided by its root mean square;
    * scores (q . k) * scale over the visible keys: j <= i and (window == 0 or i - j < window or
      j < keep_first); softmax per head; the weights of the heads mixed by `talk` [heads, heads];
      head h applies its mixed weights to the values of key/value head h // (heads / kv_heads);
    * output projection without bias.

    With `own_keys=False` the layer has no key and value tensors: it reads the cache entry of
    another layer (the run order names it) with its own queries, mask and mixing matrix.
    `names` gives the tensor names below the prefix.
    """

    capturable = True

    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "talk": "talk", "conv": ".conv",
             "norm": ".norm"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int,
                 vdim: int, taps: int, scale: float, eps: float, position: PartSpec,
                 window: int = 0, keep_first: int = 0, own_keys: bool = True,
                 names: Optional[Dict[str, str]] = None):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if taps < 1:
            raise ValueError("taps must be at least 1")
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.scale, self.eps = int(taps), float(scale), float(eps)
        self.window, self.keep_first, self.own_keys = int(window), int(keep_first), bool(own_keys)
        self.q_width = self.heads * self.dim
        self.k_width = self.kv_heads * self.dim if self.own_keys else 0
        self.v_width = self.kv_heads * self.vdim if self.own_keys else 0
        self.width = self.q_width + self.k_width + self.v_width
        self.position = build_part("position", position, prefix)
        if self.position.rotary_dim > self.dim:
            raise ValueError("the rotated size exceeds dim")
        if self.position.rotary_dim and getattr(self.position, "pairing", "") != "interleaved":
            raise ValueError("talking_window_attention rotates interleaved pairs")
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_in = self.w_o = self.conv = self.q_gain = self.k_gain = self.talk = None

    def _projections(self):
        return ("q", "k", "v") if self.own_keys else ("q",)

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, n = self.prefix, self.hidden_size, self.names
        widths = {"q": self.q_width, "k": self.k_width, "v": self.v_width}
        specs = []
        for which in self._projections():
            specs.append(TensorSpec(p + n[which], (widths[which], h)))
            specs.append(TensorSpec(p + n[which] + n["conv"], (widths[which], self.taps),
                                    role="vector", init="taps"))
            if which != "v":
                specs.append(TensorSpec(p + n[which] + n["norm"], (widths[which],),
                                        role="vector", init="gain"))
        specs.append(TensorSpec(p + n["talk"], (self.heads, self.heads), role="vector", init="eye"))
        specs.append(TensorSpec(p + n["o"], (h, self.heads * self.vdim)))
        return specs + self.position.tensor_specs()

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(self.kv_heads, self.dim, self.window, self.keep_first, self.vdim)

    def state_need(self) -> Optional[StateNeed]:
        if self.taps == 1:
            return None
        return StateNeed((self.taps - 1, self.width), torch.float32)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p, n = self.prefix, self.names
        which = self._projections()
        self.w_in = torch.cat([tensors[p + n[k]] for k in which]).contiguous()
        self.conv = torch.cat([tensors[p + n[k] + n["conv"]] for k in which]).to(torch.float32).contiguous()
        self.q_gain = tensors[p + n["q"] + n["norm"]].to(torch.float32).contiguous()
        self.k_gain = (tensors[p + n["k"] + n["norm"]].to(torch.float32).contiguous()
                       if self.own_keys else None)
        self.talk = tensors[p + n["talk"]].to(torch.float32).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        runtime.prepare_weight(self.w_in)
        runtime.prepare_weight(self.w_o)
        self.position.bind(tensors, runtime)
        self.tile_tokens = ops.talking_attention_tile_tokens(self.heads)
        if self.tile_tokens <= 0:
            raise ValueError(f"talking_window_attention: {self.heads} heads are more than the "
                             f"attention kernel holds in one block")
        self.key_tile = ops.talking_attention_key_tile(self.heads, self.kv_heads, self.dim,
                                                       self.vdim, runtime.dtype)
        # bfloat16 prompt portions run on the tensor cores where the sizes allow (`tensor_cores`
        # may be switched off to measure or test the 32-bit form)
        self.tensor_cores = ops.talking_attention_mma_takes(self.heads, self.kv_heads, self.dim,
                                                            self.vdim, runtime.dtype)
        if self.key_tile <= 0:
            raise ValueError("talking_window_attention: these head counts and sizes do not fit "
                             "the attention kernel's shared memory")

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        if cache.writes != self.own_keys:
            raise ValueError("talking_window_attention: a layer with keys of its own writes its "
                             "cache entry, one without reads another's")
        group = ctx.groups[cache.group]
        proj = rt.linear(y, self.w_in, None, "talking.in")
        q = rt.buffer("talking.q", tokens, self.q_width, torch.float32)
        ops.conv_norm_rotate(proj, ctx.num_items, ctx.item_qstart, ctx.item_pos0, ctx.item_slots,
                             cache.state, self.conv, self.taps, self.q_gain, self.k_gain,
                             self.position.table, self.position.rotary_dim,
                             group.slot_of if self.own_keys else None,
                             cache.k_pages if self.own_keys else None,
                             cache.v_pages if self.own_keys else None,
                             cache.page_stride, group.page_size, q, self.heads, self.kv_heads,
                             self.dim, self.vdim, self.own_keys, self.eps, ctx.error)
        if self.taps > 1:
            ops.conv_tails(proj, ctx.item_qstart, ctx.item_qlen, ctx.item_slots, ctx.num_items,
                           cache.state, self.taps)
        out = rt.buffer("talking.out", tokens, self.heads * self.vdim, proj.dtype)
        if self.tensor_cores and ctx.num_tokens != ctx.num_items:
            # a step with prompt portions, bfloat16, sizes the tensor-core form takes
            tiles = ctx.attention_tiles(1, ops.TALKING_MMA_TILE_TOKENS)
            partial = ctx.scratch("talking.partial", tokens * self.heads * self.kv_heads * self.vdim)
            ops.talking_attention_mma(q, cache.k_pages, cache.v_pages, cache.page_stride,
                                      group.page_size, group.block_tables, tiles.item, tiles.row0,
                                      tiles.count, ctx.item_qstart, ctx.item_qlen, ctx.item_pos0,
                                      ctx.item_slots, self.talk, partial, out, self.heads,
                                      self.kv_heads, self.dim, self.vdim, self.window,
                                      self.keep_first, self.scale, ctx.error)
            return rt.linear(out, self.w_o, None, "talking.o")
        # a step of single tokens takes tiles of one token, a step with prompt portions the
        # largest tile a block holds for this many heads
        tile_tokens = 1 if ctx.num_tokens == ctx.num_items else self.tile_tokens
        tiles = ctx.attention_tiles(1, tile_tokens)
        # fewer tiles than the GPU has room for blocks: every tile's keys are split over several
        keys = ctx.max_context if self.window <= 0 else \
            min(ctx.max_context, self.window + self.keep_first + tile_tokens - 1)
        nsplit = max(1, min(-(-keys // self.key_tile), 2 * rt.sm_count // max(tiles.count, 1), 32))
        part_stats = part_out = None
        if nsplit > 1:
            part_stats = ctx.scratch("talking.part_stats", tiles.count * nsplit * 128)
            part_out = ctx.scratch("talking.part_out", nsplit * tokens * self.heads * self.vdim)
        ops.talking_attention(q, cache.k_pages, cache.v_pages, cache.page_stride, group.page_size,
                              group.block_tables, tiles.item, tiles.row0, tiles.count,
                              ctx.item_qstart, ctx.item_qlen, ctx.item_pos0, ctx.item_slots,
                              self.talk, out, self.heads, self.kv_heads, self.dim, self.vdim,
                              self.window, self.keep_first, tile_tokens, self.scale, ctx.error,
                              nsplit, part_stats, part_out)
        return rt.linear(out, self.w_o, None, "talking.o")
