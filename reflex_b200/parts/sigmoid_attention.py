"""Grouped-query attention whose weights are sigmoids, over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T (no bias); keys are `head_dim` wide, values
`v_head_dim`; an optional rotation of the first dimensions of q and k; k and v
go into the cache at the row's position; then for the query at position p of
head h (kv head h / group) and the keys j with 0 <= p - j < window (all j <= p
without a window)
    out_h = sum_j sigmoid((q . k_j) * scale + b_h) v_j,
with b_h one stored number a head.  The weights are not normalised over the
keys.  out = concat_h(out_h) Wo^T.  Scores, sigmoids and the sums are 32-bit.

The three matrices are stacked into one product; a caller with more matrices of
the same input (a pair of mixers) may stack them further (`input_weight`,
`adopt_input_weight`, `forward(..., proj=)`).
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import KVSpec
from ..config.spec import MixerSpec
from ..errors import InvalidInput
from .registry import POSITIONS, TensorInfo, register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention:
    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise InvalidInput("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.position = (POSITIONS.get(spec.position.kind)(spec.position, dtype, device)
                         if spec.position is not None else None)
        self.qkv = self.o = self.bias = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, d, dv = spec.hidden_size, spec.head_dim, spec.value_dim
        return {
            "q_proj": TensorInfo((spec.num_heads * d, W), "matrix"),
            "k_proj": TensorInfo((spec.num_kv_heads * d, W), "matrix"),
            "v_proj": TensorInfo((spec.num_kv_heads * dv, W), "matrix"),
            "score_bias": TensorInfo((spec.num_heads,), "bias"),
            "o_proj": TensorInfo((W, spec.num_heads * dv), "matrix"),
        }

    def cache_spec(self) -> KVSpec:
        s = self.spec
        return KVSpec(s.num_kv_heads, s.head_dim, s.window, v_head_dim=s.value_dim)

    @property
    def capturable(self) -> bool:
        return self.position is None or bool(getattr(self.position, "capturable", False))

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        self.qkv = torch.cat([dev(tensors["q_proj"]), dev(tensors["k_proj"]), dev(tensors["v_proj"])], dim=0).contiguous()
        self.o = dev(tensors["o_proj"]).contiguous()
        self.bias = tensors["score_bias"].to(device=self.device, dtype=torch.float32).contiguous()

    def input_weight(self):
        return self.qkv

    def adopt_input_weight(self, rows: torch.Tensor) -> None:
        self.qkv = rows

    def heads_out(self, x, ctx, proj=None):
        """The concatenated heads [rows, heads * v_head_dim] in the compute type,
        before the output product."""
        s, kv, batch = self.spec, ctx.kv, ctx.batch
        if not ctx.writes_cache:
            raise InvalidInput("sigmoid_attention: every run writes its own keys and values")
        if proj is None:
            proj, col0 = ops.linear(x, self.qkv, out_dtype=torch.float32), 0
            ops.prof_mark("qkv_gemm")
        else:
            proj, col0 = proj
        rotation = None if self.position is None else self.position.rotation()
        q = ops.sig_qkv_post(proj, col0, rotation, batch.row_pos, batch.row_slot, kv.k_pages, kv.v_pages,
                             kv.page_table, kv.page_size, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim,
                             True, self.dtype)
        ops.prof_mark("norm_rope")
        attn = ops.attention_sigmoid(q, kv.k_pages, kv.v_pages, kv.page_table, kv.page_size, batch, s.num_heads,
                                     s.num_kv_heads, s.head_dim, s.value_dim, s.window, s.scale, self.bias)
        ops.prof_mark("attn")
        return attn

    def forward(self, x, ctx, proj=None):
        out = ops.linear(self.heads_out(x, ctx, proj), self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
