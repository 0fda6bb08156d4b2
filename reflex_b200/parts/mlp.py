"""Gated feed-forward (SwiGLU), dense.

gate = x Wg^T, up = x Wu^T, act = gate / (1 + exp(-gate)) * up, out = act Wd^T
(src/model/dense.rs:1476-1481, src/kernels_cuda/silu_and_mul.cu:7-23).  The
gate and up weights are woven into one [2I, H] matrix at load, row 2j = gate_j
and row 2j + 1 = up_j, so that one product serves both (the reference's decode
path fuses them by kernel, src/kernels_cuda/gemv_fused.cu:143-203) and the
activation can be that product's epilogue; reordering rows changes no output.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import FeedForwardSpec
from .registry import TensorInfo, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    capturable = True  # launches read nothing from the host: may be captured into a CUDA graph

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.gate_up = None
        self.down = None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        H, I = spec.hidden_size, spec.intermediate_size
        return {
            "gate_proj": TensorInfo((I, H), "matrix"),
            "up_proj": TensorInfo((I, H), "matrix"),
            "down_proj": TensorInfo((H, I), "matrix"),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        g, u = dev(tensors["gate_proj"]), dev(tensors["up_proj"])
        self.gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
        self.down = dev(tensors["down_proj"]).contiguous()

    supports_fused_residual = True
    accepts_normed_input = True  # its first product finishes a norm that the product before began

    def forward(self, x, residual=None):
        """With `residual` = (hidden, next norm) the down projection may add itself
        to `hidden`; it then returns the rows for the product after that norm
        (`ops.NormedInput`) or None (added, the norm not begun).  Otherwise it
        returns the delta."""
        act = ops.linear_swiglu(x, self.gate_up)
        ops.prof_mark("ffn_gate_up")
        if residual is not None:
            fused = ops.linear_residual(act, self.down, residual[0], residual[1])
            if fused is not None:
                ops.prof_mark("ffn_down")
                return None if fused is ops.ADDED else fused  # None: nothing left to add
        out = ops.linear(act, self.down, out_dtype=torch.float32)
        ops.prof_mark("ffn_down")
        return out


@register_feed_forward("glu_clamped")
class ClampedGLU:
    """The clamped gated feed-forward: g = min(W_g x, limit), u = clamp(W_u x,
    -limit, limit), out = W_d (g * sigmoid(alpha g) * (u + 1)); `alpha` and
    `limit` are the spec's parameters.  Gate and up are one woven matrix, as in
    `SwiGLU`.  `forward(x, onto=delta)` adds the result onto a 32-bit delta
    another part made from the same input (a mixer beside it) and returns it."""

    capturable = True

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.alpha = float(spec.param("alpha", 1.0))
        self.limit = float(spec.param("limit"))
        self.gate_up = None
        self.down = None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        return SwiGLU.tensor_specs(spec)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        g, u = dev(tensors["gate_proj"]), dev(tensors["up_proj"])
        self.gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
        self.down = dev(tensors["down_proj"]).contiguous()

    supports_onto = True

    def forward(self, x, residual=None, onto=None):
        act = ops.linear_glu_clamped(x, self.gate_up, self.alpha, self.limit)
        ops.prof_mark("ffn_gate_up")
        if onto is not None:
            # many bfloat16 rows: the product accumulates onto the 32-bit delta
            if ops.linear_residual(act, self.down, onto, None) is not ops.ADDED:
                ops.add_(onto, ops.linear(act, self.down, out_dtype=torch.float32))
            ops.prof_mark("ffn_down")
            return onto
        out = ops.linear(act, self.down, out_dtype=torch.float32)
        ops.prof_mark("ffn_down")
        return out


@register_feed_forward("relu2")
class SquaredReLU:
    """out = W_down relu(W_up x)^2: no gate, the activation is the square of the
    rectified product."""

    capturable = True

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.up = None
        self.down = None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        H, I = spec.hidden_size, spec.intermediate_size
        return {"up_proj": TensorInfo((I, H), "matrix"), "down_proj": TensorInfo((H, I), "matrix")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.up = tensors["up_proj"].to(device=self.device, dtype=self.dtype).contiguous()
        self.down = tensors["down_proj"].to(device=self.device, dtype=self.dtype).contiguous()

    def forward(self, x, residual=None):
        act = ops.linear_relu2(x, self.up)
        ops.prof_mark("ffn_gate_up")
        out = ops.linear(act, self.down, out_dtype=torch.float32)
        ops.prof_mark("ffn_down")
        return out


@register_feed_forward("xielu")
class XieluFeedForward:
    """out = W_down act(W_up x) with act(z) = ap z^2 + z / 2 for z > 0 and
    an (e^z - 1 - z) + z / 2 otherwise, ap = softplus(p) and an = beta +
    softplus(q), p and q the two stored numbers of the layer (`act`), beta the
    spec's parameter.  The two softplus are taken once, when the weights are bound.
    For a few rows the activation is the product kernel's epilogue (`ops.linear_xielu`)."""

    capturable = True

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.beta = float(spec.param("beta", 0.5))
        self.up = self.down = None
        self.alpha_pos = self.alpha_neg = 0.0

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        H, I = spec.hidden_size, spec.intermediate_size
        return {"up_proj": TensorInfo((I, H), "matrix"), "down_proj": TensorInfo((H, I), "matrix"),
                "act": TensorInfo((2,), "bias")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.up = tensors["up_proj"].to(device=self.device, dtype=self.dtype).contiguous()
        self.down = tensors["down_proj"].to(device=self.device, dtype=self.dtype).contiguous()
        p, q = (float(v) for v in tensors["act"].to(device="cpu", dtype=torch.float64).tolist())
        import math

        def softplus(z: float) -> float:
            return max(z, 0.0) + math.log1p(math.exp(-abs(z)))

        self.alpha_pos, self.alpha_neg = softplus(p), self.beta + softplus(q)

    def forward(self, x, residual=None):
        act = ops.linear_xielu(x, self.up, self.alpha_pos, self.alpha_neg)
        ops.prof_mark("ffn_gate_up")
        out = ops.linear(act, self.down, out_dtype=torch.float32)
        ops.prof_mark("ffn_down")
        return out
