"""Block arrangements: how a layer's parts are wired around the residual.

"prenorm": h += mixer(norm1(h)); h += ffn(norm2(h))
(src/model/dense.rs:1441-1484).  "parallel": n = norm1(h); h += mixer(n) + ffn(n),
one norm that both sublayers read.  "sandwich": a norm on both sides of every
sublayer, h += m * post1(mixer(norm1(h))); h += m * post2(ffn(norm2(h))), m one
number of the layer.  The residual stream is 32-bit; each add is
fused into the norm that follows it, so a block hands its last delta on as
`pending` and the next block's (or the model's final) norm adds it
(src/model/decode_step.rs:199-210, 293-300).
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LayerSpec, names_dict
from .registry import FEED_FORWARDS, MIXERS, NORMS, TensorInfo, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, dtype, device)
        # a layer may be its mixer alone
        self.has_feed_forward = spec.feed_forward is not None
        self.feed_forward_norm = self.feed_forward = None
        if self.has_feed_forward:
            self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(
                spec.feed_forward_norm, dtype, device)
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, dtype, device)

    @property
    def fusable_first_norm(self):
        """The norm this layer starts with, if the product before it may begin it
        (the mixer then gets rows that await their norm factor, an
        `ops.NormedInput`, which only a mixer that says so accepts); else None."""
        return self.mixer_norm if getattr(self.mixer, "accepts_normed_input", False) else None

    @property
    def capturable(self) -> bool:
        """Whether every part of the layer allows its launches to be captured."""
        parts = [self.mixer_norm, self.mixer]
        if self.has_feed_forward:
            parts += [self.feed_forward_norm, self.feed_forward]
        return all(bool(getattr(p, "capturable", False)) for p in parts)

    @classmethod
    def tensor_names(cls, spec: LayerSpec) -> Dict[str, Tuple[str, str, TensorInfo]]:
        """full tensor name -> (part, role, info) for every tensor of the layer."""
        out: Dict[str, Tuple[str, str, TensorInfo]] = {}
        block_names = names_dict(spec.names)

        def add(part: str, infos: Dict[str, TensorInfo], names: Dict[str, str]) -> None:
            for role, info in infos.items():
                # "role#7": one of several tensors of a kind (an expert's); the
                # name pattern of the kind is filled with the index
                base, _, index = role.partition("#")
                suffix = names.get(base, base)
                if index:
                    suffix = suffix.format(expert=index)
                out[spec.prefix + suffix] = (part, role, info)

        add("mixer_norm", {"weight": NORMS.get(spec.mixer_norm.kind).tensor_specs(spec.mixer_norm)["weight"]},
            {"weight": block_names.get("mixer_norm", "mixer_norm.weight")})
        add("mixer", MIXERS.get(spec.mixer.kind).tensor_specs(spec.mixer), names_dict(spec.mixer.names))
        if spec.feed_forward is not None:
            add("feed_forward_norm",
                {"weight": NORMS.get(spec.feed_forward_norm.kind).tensor_specs(spec.feed_forward_norm)["weight"]},
                {"weight": block_names.get("feed_forward_norm", "feed_forward_norm.weight")})
            add("feed_forward", FEED_FORWARDS.get(spec.feed_forward.kind).tensor_specs(spec.feed_forward),
                names_dict(spec.feed_forward.names))
        return out

    def bind(self, by_part: Dict[str, Dict[str, torch.Tensor]]) -> None:
        self.mixer_norm.bind(by_part.get("mixer_norm", {}))
        self.mixer.bind(by_part.get("mixer", {}))
        if self.has_feed_forward:
            self.feed_forward_norm.bind(by_part.get("feed_forward_norm", {}))
            self.feed_forward.bind(by_part.get("feed_forward", {}))

    def forward(self, hidden: torch.Tensor, pending, ctx, next_norm=None):
        """`pending` is what the block before left: a delta still to be added to
        `hidden`, None (nothing to add), or an `ops.NormedInput`: `hidden` already
        holds the sum and the rows only await this block's first norm factor.
        `next_norm` is the norm that will consume this block's result; parts that
        can fuse the residual add and that norm into their last product do so."""
        from .. import ops

        if isinstance(pending, ops.NormedInput):
            x = pending
        else:
            x = self.mixer_norm(hidden, delta=pending)
            ops.prof_mark("norm")
        if not self.has_feed_forward:
            # the mixer's result is the layer's: the next norm takes it up
            if getattr(self.mixer, "supports_fused_residual", False):
                return hidden, self.mixer.forward(x, ctx, residual=(hidden, next_norm))
            return hidden, self.mixer.forward(x, ctx)
        if getattr(self.mixer, "supports_fused_residual", False):
            ffn_norm = self.feed_forward_norm if getattr(self.feed_forward, "accepts_normed_input", False) else None
            a = self.mixer.forward(x, ctx, residual=(hidden, ffn_norm))
        else:
            a = self.mixer.forward(x, ctx)
        if isinstance(a, ops.NormedInput):
            x = a
        else:
            x = self.feed_forward_norm(hidden, delta=a)
            ops.prof_mark("norm")
        if getattr(self.feed_forward, "supports_fused_residual", False):
            f = self.feed_forward.forward(x, residual=(hidden, next_norm))
        else:
            f = self.feed_forward.forward(x)
        return hidden, f


@register_block("parallel")
class ParallelBlock(PreNormBlock):
    """n = norm(h); h += mixer(n) + ffn(n): one norm, both sublayers read its
    output, their sum is the layer's delta.  The spec's `feed_forward_norm` is
    None; a layer without a feed-forward is h += mixer(norm(h)).  Where the mixer
    and the feed-forward both offer the matrix of their first product of the
    shared input (`input_weight` / `adopt_input_weight` / `forward(..., proj=)`: a
    pair mixer's stacked projections, a router), the block stacks the two and
    makes one product for both."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, dtype, device)
        self.has_feed_forward = spec.feed_forward is not None
        self.feed_forward_norm = None
        self.feed_forward = (FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, dtype, device)
                             if self.has_feed_forward else None)
        self.stacked = None  # the mixer's and the feed-forward's first matrices, one above the other
        self.ffn_col = 0

    fusable_first_norm = None  # its mixers take plain normed rows

    @property
    def capturable(self) -> bool:
        parts = [self.mixer_norm, self.mixer] + ([self.feed_forward] if self.has_feed_forward else [])
        return all(bool(getattr(p, "capturable", False)) for p in parts)

    @classmethod
    def tensor_names(cls, spec: LayerSpec) -> Dict[str, Tuple[str, str, TensorInfo]]:
        import dataclasses

        # the names of a pre-norm layer whose feed-forward has no norm of its own
        out = PreNormBlock.tensor_names(dataclasses.replace(spec, feed_forward=None))
        if spec.feed_forward is not None:
            names = names_dict(spec.feed_forward.names)
            for role, info in FEED_FORWARDS.get(spec.feed_forward.kind).tensor_specs(spec.feed_forward).items():
                base, _, index = role.partition("#")
                suffix = names.get(base, base)
                out[spec.prefix + (suffix.format(expert=index) if index else suffix)] = ("feed_forward", role, info)
        return out

    def bind(self, by_part: Dict[str, Dict[str, torch.Tensor]]) -> None:
        self.mixer_norm.bind(by_part.get("mixer_norm", {}))
        self.mixer.bind(by_part.get("mixer", {}))
        if self.has_feed_forward:
            self.feed_forward.bind(by_part.get("feed_forward", {}))
            both = [self.mixer, self.feed_forward]
            if all(hasattr(p, "input_weight") and hasattr(p, "adopt_input_weight") for p in both):
                mats = [p.input_weight() for p in both]
                if (all(m is not None for m in mats) and mats[0].dtype == mats[1].dtype
                        and mats[0].shape[1] == mats[1].shape[1] and getattr(self.feed_forward, "supports_onto", False)):
                    # zero rows up to a multiple of 8: the product's rows stay 16-byte aligned, which
                    # the library's products and the kernels that read four columns a thread want
                    rows = mats[0].shape[0] + mats[1].shape[0]
                    pad = torch.zeros((-rows % 8, mats[0].shape[1]), dtype=mats[0].dtype, device=mats[0].device)
                    self.stacked = torch.cat(mats + [pad], dim=0).contiguous()
                    self.ffn_col = mats[0].shape[0]
                    self.mixer.adopt_input_weight(self.stacked[:self.ffn_col])
                    self.feed_forward.adopt_input_weight(self.stacked[self.ffn_col:rows])

    def forward(self, hidden: torch.Tensor, pending, ctx, next_norm=None):
        from .. import ops

        if isinstance(pending, ops.NormedInput):
            pending = None  # the stream already holds the sum; this block's parts want plain normed rows
        x = self.mixer_norm(hidden, delta=pending)
        ops.prof_mark("norm")
        if self.stacked is not None:
            proj = ops.linear(x, self.stacked, out_dtype=torch.float32)
            ops.prof_mark("qkv_gemm")
            delta = self.mixer.forward(x, ctx, proj=(proj, 0))
            return hidden, self.feed_forward.forward(x, onto=delta, proj=(proj, self.ffn_col))
        delta = self.mixer.forward(x, ctx)
        if self.has_feed_forward:
            if getattr(self.feed_forward, "supports_onto", False):
                delta = self.feed_forward.forward(x, onto=delta)
            else:
                delta = ops.add_(delta, self.feed_forward.forward(x))
        return hidden, delta


@register_block("sandwich")
class SandwichBlock(PreNormBlock):
    """h += m * post1(mixer(norm1(h))); h += m * post2(ffn(norm2(h))): every
    sublayer's result is normed (weights `post_mixer`, `post_feed_forward` among
    the spec's `extra_norms`) and multiplied by the spec's `residual_mult` before
    it joins the 32-bit residual.  The norm after a sublayer and the norm before
    the next one are one pass over the row (`ops.sandwich_norm`): the block hands
    the next block its first norm's rows ready (`ReadyRows`) when it is told that
    norm, and adds into the residual itself, so it never leaves a delta pending."""

    class ReadyRows:
        """Rows the next block's first norm has already produced."""

        def __init__(self, rows):
            self.rows = rows

    skips_final_norm_fusion = True  # the model's last norm meets the wanted rows only

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device):
        super().__init__(spec, dtype, device)
        extra = dict(spec.extra_norms)
        self.dtype = dtype
        self.mult = float(dict(spec.params).get("residual_mult", 1.0))
        self.post_mixer = NORMS.get(extra["post_mixer"].kind)(extra["post_mixer"], dtype, device)
        self.post_feed_forward = (NORMS.get(extra["post_feed_forward"].kind)(extra["post_feed_forward"], dtype, device)
                                  if self.has_feed_forward else None)
        for n in (self.mixer_norm, self.feed_forward_norm, self.post_mixer, self.post_feed_forward):
            if n is not None and (n.spec.kind != "rmsnorm" or n.spec.weight_offset != 0.0):
                raise ValueError("sandwich block: takes RMS norms with a plain weight")

    @property
    def fusable_first_norm(self):
        return self.mixer_norm

    @property
    def capturable(self) -> bool:
        return PreNormBlock.capturable.fget(self) and bool(getattr(self.post_mixer, "capturable", False))

    @classmethod
    def tensor_names(cls, spec: LayerSpec) -> Dict[str, Tuple[str, str, TensorInfo]]:
        out = PreNormBlock.tensor_names(spec)
        block_names = names_dict(spec.names)
        for role, norm in spec.extra_norms:
            if role == "post_feed_forward" and spec.feed_forward is None:
                continue
            info = NORMS.get(norm.kind).tensor_specs(norm)["weight"]
            out[spec.prefix + block_names.get(role, role + ".weight")] = (role, "weight", info)
        return out

    def bind(self, by_part: Dict[str, Dict[str, torch.Tensor]]) -> None:
        super().bind(by_part)
        self.post_mixer.bind(by_part.get("post_mixer", {}))
        if self.has_feed_forward:
            self.post_feed_forward.bind(by_part.get("post_feed_forward", {}))

    def forward(self, hidden: torch.Tensor, pending, ctx, next_norm=None):
        from .. import ops

        if isinstance(pending, SandwichBlock.ReadyRows):
            x = pending.rows
        else:
            if isinstance(pending, ops.NormedInput):
                pending = None  # the stream already holds the sum
            x = self.mixer_norm(hidden, delta=pending)
            ops.prof_mark("norm")
        # the norm that follows this block, if it is one this kernel can make
        nxt = next_norm if isinstance(next_norm, type(self.mixer_norm)) and next_norm.spec.weight_offset == 0.0 else None
        y = self.mixer.forward(x, ctx)
        after = self.feed_forward_norm if self.has_feed_forward else nxt
        x = ops.sandwich_norm(y, hidden, self.post_mixer.weight, self.mult, self.post_mixer.spec.eps,
                              after.weight if after is not None else None,
                              after.spec.eps if after is not None else 0.0, self.dtype)
        ops.prof_mark("norm")
        if not self.has_feed_forward:
            return hidden, (SandwichBlock.ReadyRows(x) if x is not None else None)
        y = self.feed_forward.forward(x)
        x = ops.sandwich_norm(y, hidden, self.post_feed_forward.weight, self.mult, self.post_feed_forward.spec.eps,
                              nxt.weight if nxt is not None else None, nxt.spec.eps if nxt is not None else 0.0,
                              self.dtype)
        ops.prof_mark("norm")
        return hidden, (SandwichBlock.ReadyRows(x) if x is not None else None)
