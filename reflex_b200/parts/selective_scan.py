"""A selective state-space mixer (the Mamba recurrence).

With h the mixer's input [rows, hidden], `inner` channels, N states a channel,
a low rank R for the step sizes and a short filter of `taps` taps:
  [x | z] = W_in h
  x   = silu(conv(x) + b_conv)        one filter a channel over the last `taps`
                                      tokens (the last tap on the current one),
                                      zeros before the start
  [dt | B | C] = W_x x                 R, N and N columns
  dt  = softplus(W_dt dt + b_dt)       one step size a channel
  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,     A = -exp(A_log)
  y_c = sum_n S[c, n] C_n + D_c x_c
  out = W_o (y * silu(z))
Per sequence the state is the last taps - 1 rows of the convolution's input and
S, 32-bit, one vector of the cache's state group, zero at a sequence's start.
The projections are products in the compute type with 32-bit results; the
convolution, the step sizes, the decays and the recurrence are 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import StateSpec
from ..config.spec import MixerSpec
from .registry import TensorInfo, register_mixer


@register_mixer("selective_scan")
class SelectiveScan:
    capturable = True  # sequences' slots and rows are read from device memory

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.inner = int(spec.param("inner"))
        self.states = int(spec.param("state"))
        self.rank = int(spec.param("dt_rank"))
        self.taps = int(spec.param("taps", 1))
        self.w_in = self.filters = self.conv_bias = self.w_x = self.w_x_dt = self.w_x_bc = self.w_dt = self.dt_bias = None
        self.A = self.D = self.o = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, C, N = spec.hidden_size, int(spec.param("inner")), int(spec.param("state"))
        R, taps = int(spec.param("dt_rank")), int(spec.param("taps", 1))
        return {
            "in_proj": TensorInfo((2 * C, W), "matrix"),
            "conv": TensorInfo((C, taps), "filter"), "conv_bias": TensorInfo((C,), "bias"),
            "x_proj": TensorInfo((R + 2 * N, C), "matrix"),
            "dt_proj": TensorInfo((C, R), "matrix"), "dt_bias": TensorInfo((C,), "bias"),
            "A_log": TensorInfo((C, N), "bias"), "D": TensorInfo((C,), "bias"),
            "o_proj": TensorInfo((W, C), "matrix"),
        }

    def cache_spec(self) -> StateSpec:
        # [the last taps - 1 inputs of the convolution | S]
        return StateSpec(((self.taps - 1) * self.inner + self.inner * self.states,), "float32")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype).contiguous()

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.w_in = dev(tensors["in_proj"])
        self.filters, self.conv_bias = f32(tensors["conv"]).t().contiguous(), f32(tensors["conv_bias"])  # [taps, C]
        # the low-rank step-size rows and the B | C rows of W_x apart: the first product's
        # result is the next product's input (compute type), the second's enters the scan (32-bit)
        w_x = dev(tensors["x_proj"])
        self.w_x_dt, self.w_x_bc = w_x[: self.rank].contiguous(), w_x[self.rank:].contiguous()
        # and whole, [dt | B | C]: a row a sequence takes one product, its step sizes' last
        # product rides in the scan
        self.w_x = w_x.contiguous()
        self.w_dt = dev(tensors["dt_proj"])
        self.dt_bias = f32(tensors["dt_bias"])
        self.A = (-torch.exp(f32(tensors["A_log"]))).contiguous()  # made once: the weights do not change
        self.D = f32(tensors["D"])
        self.o = dev(tensors["o_proj"])

    def forward(self, x, ctx):
        batch, state, C, N = ctx.batch, ctx.state, self.inner, self.states
        lo = self.dtype == torch.bfloat16
        xz = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [rows, x | z]
        ops.prof_mark("qkv_gemm")
        # a row a sequence (decoding): the convolution's launch also moves the last inputs on
        single = xz.shape[0] == batch.seq_slot.numel()
        u = ops.short_conv(xz, 0, C, None, self.filters, self.conv_bias, state if self.taps > 1 else None, batch,
                           also_bf16=lo, activation="silu", update_state=single and self.taps > 1)
        u, u_in = u if lo else (u, u)
        if not single:
            # the sequences' new last inputs (the rows that read the old ones are done: the launch above)
            ops.conv_state_update(xz, 0, C, None, self.taps, state, batch)
        ops.prof_mark("conv_post")
        if single:
            # decoding: one product [rows, dt | B | C] in 32-bit; W_dt meets its vector in the scan
            proj = ops.linear(u_in, self.w_x, out_dtype=torch.float32)
            ops.prof_mark("scan_proj")
            y = ops.mamba_scan(u, None, self.dt_bias, proj, self.rank, self.rank + N, xz, C, self.A, self.D, state,
                               (self.taps - 1) * C, batch, self.dtype, dt_weight=self.w_dt, dt_low_off=0)
        else:
            bc = ops.linear(u_in, self.w_x_bc, out_dtype=torch.float32)  # [rows, B | C]
            dt_low = ops.linear(u_in, self.w_x_dt, out_dtype=self.dtype)  # [rows, R]
            dtpre = ops.linear(dt_low, self.w_dt, out_dtype=torch.float32)  # [rows, inner], before the bias
            ops.prof_mark("scan_proj")
            y = ops.mamba_scan(u, dtpre, self.dt_bias, bc, 0, N, xz, C, self.A, self.D, state,
                               (self.taps - 1) * C, batch, self.dtype)
        ops.prof_mark("scan")
        out = ops.linear(y, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
