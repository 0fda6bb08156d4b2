"""Block arrangement "hyper_prenorm": pre-norm sublayers around a residual that
is several parallel streams (hyper-connections), with a per-channel scale on
every sublayer's result.

With S streams x_1 .. x_S (all equal to the embedding output at the start) and
sublayer q of the layer (1: the mixer, 2: the feed-forward):
    u   = sum_s read_q[s] x_s
    y   = scale_q * sublayer_q(norm_q(u))               scale_q: a vector [hidden]
    x_t <- sum_s mix_q[s, t] x_s + write_q[t] y         every stream at once
The model's final norm meets the sum of the streams.  `LayerSpec.params`:
`streams` (S), `connections` (False: the layer has no read / write / mix
tensors, which is S = 1 with all of them 1, the ordinary x <- x + scale * y) and
`layer_scale` (False: no scale tensors).

The streams are one 32-bit tensor [rows, S * hidden].  A sublayer's write is
not a launch of its own: the block hands it on (`ops.StreamWrite`) and the next
read applies it first, in the same pass over the row that sums the streams and
norms the sum (`ops.hyper_step`); the layer's last write is the block's
`pending`, taken up by the next layer's first read or, after the last layer, by
`finish`, which also sums the streams.
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import ops
from ..config.spec import LayerSpec, names_dict
from ..errors import InvalidInput
from .registry import FEED_FORWARDS, MIXERS, NORMS, TensorInfo, register_block


@register_block("hyper_prenorm")
class HyperPreNormBlock:
    fusable_first_norm = None  # the first norm follows a read of all streams: nothing before it can begin it

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        params = dict(spec.params)
        self.streams = int(params.get("streams", 1))
        self.connections = bool(params.get("connections", self.streams > 1))
        self.layer_scale = bool(params.get("layer_scale", False))
        if self.streams > 1 and not self.connections:
            raise InvalidInput("hyper_prenorm: several streams need their read, write and mix tensors")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, dtype, device)
        self.has_feed_forward = spec.feed_forward is not None
        self.feed_forward = (FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, dtype, device)
                             if self.has_feed_forward else None)
        # per sublayer: norm weight, scale, read, write, mix
        self.norm_w = [None, None]
        self.scale = [None, None]
        self.read = [None, None]
        self.write = [None, None]
        self.mix = [None, None]

    @property
    def capturable(self) -> bool:
        parts = [self.mixer] + ([self.feed_forward] if self.has_feed_forward else [])
        return all(bool(getattr(p, "capturable", False)) for p in parts)

    SUBLAYERS = ("mixer", "feed_forward")

    @classmethod
    def tensor_names(cls, spec: LayerSpec) -> Dict[str, Tuple[str, str, TensorInfo]]:
        out: Dict[str, Tuple[str, str, TensorInfo]] = {}
        names = names_dict(spec.names)
        params = dict(spec.params)
        S = int(params.get("streams", 1))
        H = spec.mixer.hidden_size

        def add(part: str, infos: Dict[str, TensorInfo], part_names: Dict[str, str]) -> None:
            for role, info in infos.items():
                out[spec.prefix + part_names.get(role, role)] = (part, role, info)

        for q, sub in enumerate(cls.SUBLAYERS):
            if sub == "feed_forward" and spec.feed_forward is None:
                continue
            norm = spec.mixer_norm if q == 0 else spec.feed_forward_norm
            block = {f"{sub}_norm": NORMS.get(norm.kind).tensor_specs(norm)["weight"]}
            if params.get("layer_scale", False):
                block[f"{sub}_scale"] = TensorInfo((H,), "norm")
            if params.get("connections", S > 1):
                block[f"{sub}_read"] = TensorInfo((S,), "coef")
                block[f"{sub}_write"] = TensorInfo((S,), "coef")
                block[f"{sub}_mix"] = TensorInfo((S, S), "coef")
            add("block", block, names)
        add("mixer", MIXERS.get(spec.mixer.kind).tensor_specs(spec.mixer), names_dict(spec.mixer.names))
        if spec.feed_forward is not None:
            add("feed_forward", FEED_FORWARDS.get(spec.feed_forward.kind).tensor_specs(spec.feed_forward),
                names_dict(spec.feed_forward.names))
        return out

    def bind(self, by_part: Dict[str, Dict[str, torch.Tensor]]) -> None:
        block = by_part.get("block", {})

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        S = self.streams
        for q, sub in enumerate(self.SUBLAYERS):
            if sub == "feed_forward" and not self.has_feed_forward:
                continue
            self.norm_w[q] = f32(block[f"{sub}_norm"])
            self.scale[q] = f32(block[f"{sub}_scale"]) if self.layer_scale else None
            if self.connections:
                self.read[q] = f32(block[f"{sub}_read"]).reshape(S)
                self.write[q] = f32(block[f"{sub}_write"]).reshape(S)
                self.mix[q] = f32(block[f"{sub}_mix"]).reshape(S, S)
            else:  # one stream, x <- x + scale * y
                self.read[q] = torch.ones((1,), dtype=torch.float32, device=self.device)
                self.write[q] = torch.ones((1,), dtype=torch.float32, device=self.device)
                self.mix[q] = torch.ones((1, 1), dtype=torch.float32, device=self.device)
        self.mixer.bind(by_part.get("mixer", {}))
        if self.has_feed_forward:
            self.feed_forward.bind(by_part.get("feed_forward", {}))

    def _pending_write(self, hidden: torch.Tensor, pending):
        """What the block before left, as a write into the streams."""
        if pending is None or isinstance(pending, ops.StreamWrite):
            return pending
        if isinstance(pending, ops.NormedInput):
            return None  # the sum is already in `hidden`
        if self.streams != 1:
            raise InvalidInput("hyper_prenorm: a plain delta cannot be added to several streams")
        one = self.write[0]
        return ops.StreamWrite(pending, None, self.mix[0], one)

    def forward(self, hidden: torch.Tensor, pending, ctx, next_norm=None):
        write = self._pending_write(hidden, pending)
        for q, sub in enumerate(self.SUBLAYERS):
            if sub == "feed_forward" and not self.has_feed_forward:
                continue
            norm = self.spec.mixer_norm if q == 0 else self.spec.feed_forward_norm
            x = ops.hyper_step(hidden, write, self.read[q], self.norm_w[q], norm.eps, norm.weight_offset,
                               self.dtype, self.streams)
            ops.prof_mark("norm")
            y = self.mixer.forward(x, ctx) if q == 0 else self.feed_forward.forward(x)
            write = ops.StreamWrite(y, self.scale[q], self.mix[q], self.write[q])
        return hidden, write

    def finish(self, hidden: torch.Tensor, pending, rows=None):
        """After the last layer: the last write, then the sum of the streams, as
        the ordinary residual [rows, hidden] with nothing left to add.  With
        `rows` (int32 on the device) only those rows are made, in that order."""
        out = ops.hyper_collapse(hidden, self._pending_write(hidden, pending), self.streams, rows)
        ops.prof_mark("norm")
        return out, None
