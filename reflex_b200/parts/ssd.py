"""A state-space mixer with one decay a head (the "state-space duality" form).

With h the mixer's input [rows, hidden], `heads` heads of `vdim` channels
(inner = heads * vdim), N states, G groups that share their B and C vectors,
and a short filter of `taps` taps:
  [z | x | B | C | dt] = W_in h            inner, inner, G N, G N and heads columns
  [x | B | C] = silu(conv([x | B | C]) + b_conv)   one filter a channel over the last
                                           `taps` tokens (the last tap on the current
                                           one), zeros before the start
  dt  = softplus(dt + dt_bias)             one step size a head, no clamp
  S_h <- exp(-exp(A_log_h) dt_h) S_h + dt_h B_g x_h^T      (N x vdim, g = h / (heads / G))
  y_h = S_h^T C_g + D_h x_h
  y   = y * silu(z), then divided by its root mean square in `norm_groups` equal
        parts, times a weight
  out = W_o y
Per sequence the state is the last taps - 1 rows of the convolution's input and
S, 32-bit, one vector of the cache's state group, zero at a sequence's start.
The projections are products in the compute type with 32-bit results; the
convolution, step sizes, decays, the recurrence, the gate and the norm are 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import StateSpec
from ..config.spec import MixerSpec
from ..errors import InvalidInput
from .registry import TensorInfo, register_mixer


@register_mixer("ssd")
class StateSpaceDuality:
    capturable = True  # sequences' slots and rows are read from device memory

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.heads = int(spec.param("heads"))
        self.vdim = int(spec.param("vdim"))
        self.states = int(spec.param("state"))
        self.groups = int(spec.param("groups", 1))
        self.taps = int(spec.param("taps", 1))
        self.norm_groups = int(spec.param("norm_groups", 1))
        self.eps = float(spec.param("eps"))
        if self.heads % self.groups or (self.heads * self.vdim) % self.norm_groups:
            raise InvalidInput("ssd: groups must divide heads and norm_groups the inner width")
        self.inner = self.heads * self.vdim
        self.conv_channels = self.inner + 2 * self.groups * self.states
        self.w_in = self.filters = self.conv_bias = self.dt_bias = self.A = self.D = self.norm = self.o = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, Hh, P = spec.hidden_size, int(spec.param("heads")), int(spec.param("vdim"))
        N, G, taps = int(spec.param("state")), int(spec.param("groups", 1)), int(spec.param("taps", 1))
        inner, cc = Hh * P, Hh * P + 2 * G * N
        return {
            "in_proj": TensorInfo((inner + cc + Hh, W), "matrix"),
            "conv": TensorInfo((cc, taps), "filter"), "conv_bias": TensorInfo((cc,), "bias"),
            "dt_bias": TensorInfo((Hh,), "bias"), "A_log": TensorInfo((Hh,), "bias"), "D": TensorInfo((Hh,), "bias"),
            "norm": TensorInfo((inner,), "norm"), "o_proj": TensorInfo((W, inner), "matrix"),
        }

    def cache_spec(self) -> StateSpec:
        # [the last taps - 1 inputs of the convolution | S of every head]
        return StateSpec(((self.taps - 1) * self.conv_channels + self.heads * self.states * self.vdim,), "float32")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype).contiguous()

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.w_in = dev(tensors["in_proj"])
        self.filters, self.conv_bias = f32(tensors["conv"]).t().contiguous(), f32(tensors["conv_bias"])  # [taps, channels]
        self.dt_bias = f32(tensors["dt_bias"])
        self.A = (-torch.exp(f32(tensors["A_log"]))).contiguous()  # made once: the weights do not change
        self.D = f32(tensors["D"])
        self.norm = f32(tensors["norm"])
        self.o = dev(tensors["o_proj"])

    def input_weight(self):
        return self.w_in

    def adopt_input_weight(self, rows: torch.Tensor) -> None:
        self.w_in = rows

    def normed_out(self, x, ctx, proj=None):
        """The gated, normed y [rows, inner] in the compute type, before the output product."""
        batch, state = ctx.batch, ctx.state
        if proj is None:
            proj, col0 = ops.linear(x, self.w_in, out_dtype=torch.float32), 0
            ops.prof_mark("qkv_gemm")
        else:
            proj, col0 = proj
        cc = self.conv_channels
        single = proj.shape[0] == batch.seq_slot.numel()  # a row a sequence: the filter's launch moves its state on
        xbc = ops.short_conv(proj, col0 + self.inner, cc, None, self.filters, self.conv_bias,
                             state if self.taps > 1 else None, batch, activation="silu",
                             update_state=single and self.taps > 1)
        if not single:
            ops.conv_state_update(proj, col0 + self.inner, cc, None, self.taps, state, batch)
        ops.prof_mark("conv_post")
        y = ops.ssd_scan(xbc, proj, col0, col0 + self.inner + cc, self.dt_bias, self.A, self.D, state,
                         (self.taps - 1) * cc, batch, self.heads, self.vdim, self.states, self.groups)
        ops.prof_mark("scan")
        y = ops.group_norm_gate(y, self.norm, self.eps, self.norm_groups, self.dtype)
        ops.prof_mark("scan_norm")
        return y

    def forward(self, x, ctx, proj=None):
        out = ops.linear(self.normed_out(x, ctx, proj), self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
