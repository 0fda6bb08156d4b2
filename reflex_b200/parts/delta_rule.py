"""A generalized delta-rule mixer: a matrix memory per head with a decay and a
removal rate per key channel.

With h the mixer's input, `heads` heads of `dim` channels (keys and values
alike):
  r = W_r h, k = W_k h, v = W_v h
  w = exp(-rate * sigmoid(W_w2 tanh(W_w1 h) + w0))     decay, through a low rank
  a = sigmoid(W_a h + a_b)                              removal rate
  u = k / sqrt(sum(k^2) + unit_eps)                     per head
  S <- diag(w) S - (a * u) (u^T S) + k v^T              both terms read the old S
  o = S^T r
  o = o / rms(o) per head (eps), times a weight over all heads, times sigmoid(W_g h)
  out = W_o o
`rate` and `unit_eps` are the spec's parameters; the low rank is the shape of
W_w1.  Per sequence the state is S of every head, 32-bit, zero at a sequence's
start.  The projections are products in the compute type with 32-bit results;
everything between them and the output product is 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import StateSpec
from ..config.spec import MixerSpec
from ..errors import CheckpointError
from .registry import TensorInfo, register_mixer


@register_mixer("delta_rule")
class DeltaRule:
    capturable = True
    STACK = ("r_proj", "k_proj", "v_proj", "g_proj", "a_proj")  # hd rows each, then W_w1's rows

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.heads, self.dim = int(spec.num_heads), int(spec.head_dim)
        self.hd = self.heads * self.dim
        self.rate = float(spec.param("rate"))
        self.unit_eps = float(spec.param("unit_eps"))
        self.eps = float(spec.param("eps"))
        self.rank = 0
        self.stacked = self.w2 = self.w0 = self.a_bias = self.norm = self.o = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, hd = spec.hidden_size, int(spec.num_heads) * int(spec.head_dim)
        rank = int(spec.param("decay_rank", 0) or 0) or max(8, hd // 16)
        out = {role: TensorInfo((hd, W), "matrix") for role in cls.STACK}
        out.update({
            "a_bias": TensorInfo((hd,), "bias"),
            # the low rank is whatever the checkpoint's tensors have
            "w1_proj": TensorInfo((-1, W), "matrix", free=rank), "w2_proj": TensorInfo((hd, -1), "matrix", free=rank),
            "w0": TensorInfo((hd,), "bias"), "norm": TensorInfo((hd,), "norm"),
            "o_proj": TensorInfo((W, hd), "matrix"),
        })
        return out

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.heads * self.dim * self.dim,), "float32")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        w1, w2 = dev(tensors["w1_proj"]), dev(tensors["w2_proj"])
        if w1.shape[0] != w2.shape[1]:
            raise CheckpointError(f"delta_rule: the decay's two matrices disagree on their rank "
                                  f"({w1.shape[0]} and {w2.shape[1]})")
        self.rank = int(w1.shape[0])
        mats = [dev(tensors[r]) for r in self.STACK] + [w1]
        rows = sum(m.shape[0] for m in mats)
        # zero rows up to a multiple of 8: the product's rows stay 16-byte aligned
        pad = torch.zeros((-rows % 8, w1.shape[1]), dtype=self.dtype, device=self.device)
        self.stacked = torch.cat(mats + [pad], dim=0).contiguous()
        self.w2 = w2.contiguous()
        self.w0, self.a_bias, self.norm = f32(tensors["w0"]), f32(tensors["a_bias"]), f32(tensors["norm"])
        self.o = dev(tensors["o_proj"]).contiguous()

    def forward(self, x, ctx):
        hd, batch = self.hd, ctx.batch
        proj = ops.linear(x, self.stacked, out_dtype=torch.float32)  # [r | k | v | g | a | w1 rows | zeros]
        ops.prof_mark("qkv_gemm")
        low = ops.tanh_cols(proj, 5 * hd, self.rank, self.dtype)
        wpre = ops.linear(low, self.w2, out_dtype=torch.float32)
        ops.prof_mark("scan_proj")
        o = ops.delta_rule(proj, 0, hd, 2 * hd, 4 * hd, wpre, self.w0, self.a_bias, self.rate, self.unit_eps,
                           ctx.state, 0, batch, self.heads, self.dim)
        ops.prof_mark("scan")
        o = ops.group_norm_gate(o, self.norm, self.eps, self.heads, self.dtype, gate=proj, gate_col=3 * hd)
        ops.prof_mark("scan_norm")
        out = ops.linear(o, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
