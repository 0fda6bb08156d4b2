"""Mixture-of-experts feed-forward with top-k routing.

Router logits z = W_r x (+ b), 32-bit; the `top` experts with the largest
logits are chosen (ties: the lower index) and weighted by the softmax over the
chosen logits only; an expert is W_down act(W_up x) without biases, act the
square of relu ("relu2") or silu; the output is the weighted sum of the chosen
experts' outputs, summed in the order of their rank in 32-bit, so a row's
result does not depend on what else is in the batch.  The experts' matrices
are stacked at load: up [experts, ff, hidden], down [experts, hidden, ff].

Variants, all by the spec's parameters.  `scores` "sigmoid": the chosen
experts' weights are the sigmoids of their logits, not renormalised.
`activation` "glu_clamped": an expert is the clamped gated form
W_down (g * sigmoid(alpha g) * (u + 1)) with g = min(W_gate x, limit) and
u = clamp(W_up x, -limit, limit) (its gate and up matrices stacked [experts,
2 ff, hidden]).  `weight_input`: the weight multiplies the expert's input, the
output is sum_k expert_k(w_k x).  `shared_ff` > 0: a shared expert of that
width (the same clamped gated form with `shared_limit`) runs for every row and
is added times sigmoid(w_sg . x), one number a row; its gate's row rides along
as one more row of the router's matrix.  `scores` "softmax_all": the weights are
the softmax over all experts' logits, the chosen ones' divided by their sum
(+ 1e-20); `score_scale` multiplies the weights.  `activation` "swiglu": an
expert is W_down (silu(W_gate x) * (W_up x)).  `shared_kind` "swiglu" (with
`shared_ff`): the shared expert is that gated silu form and is added as it is,
with no gate of its own.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import FeedForwardSpec
from .registry import TensorInfo, register_feed_forward


@register_feed_forward("moe")
class MixtureOfExperts:
    capturable = True  # routing stays on the device: ids and weights are read by the expert kernels

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.experts = int(spec.param("experts"))
        self.top = int(spec.param("top"))
        self.activation = str(spec.param("activation", "relu2"))
        self.scores = str(spec.param("scores", "softmax_top"))
        self.weight_input = bool(spec.param("weight_input", False))
        self.alpha = float(spec.param("alpha", 1.0))
        self.limit = float(spec.param("limit", 0.0))
        self.shared_ff = int(spec.param("shared_ff", 0) or 0)
        self.shared_limit = float(spec.param("shared_limit", 0.0))
        self.shared_kind = str(spec.param("shared_kind", "glu_clamped_gated"))
        self.score_scale = float(spec.param("score_scale", 1.0))
        self.router = self.router_bias = self.up = self.down = None
        self.shared_gate_up = self.shared_down = None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        H, I, E = spec.hidden_size, spec.intermediate_size, int(spec.param("experts"))
        out = {"router": TensorInfo((E, H), "matrix")}
        if spec.param("router_bias", False):
            out["router_bias"] = TensorInfo((E,), "bias")
        gated = spec.param("activation") in ("glu_clamped", "swiglu")
        for e in range(E):  # role#index: the checkpoint names every expert's tensors
            if gated:
                out[f"expert_gate#{e}"] = TensorInfo((I, H), "matrix")
            out[f"expert_up#{e}"] = TensorInfo((I, H), "matrix")
            out[f"expert_down#{e}"] = TensorInfo((H, I), "matrix")
        S = int(spec.param("shared_ff", 0) or 0)
        if S:
            out.update({"shared_gate": TensorInfo((S, H), "matrix"), "shared_up": TensorInfo((S, H), "matrix"),
                        "shared_down": TensorInfo((H, S), "matrix"), "shared_sg": TensorInfo((1, H), "matrix")})
            if spec.param("shared_kind", "glu_clamped_gated") == "swiglu":
                del out["shared_sg"]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        self.router = dev(tensors["router"]).contiguous()
        b = tensors.get("router_bias")
        self.router_bias = None if b is None else b.to(device=self.device, dtype=torch.float32).contiguous()
        if self.activation in ("glu_clamped", "swiglu"):  # an expert's gate rows, then its up rows
            self.up = torch.stack([torch.cat([dev(tensors[f"expert_gate#{e}"]), dev(tensors[f"expert_up#{e}"])])
                                   for e in range(self.experts)]).contiguous()
        else:
            self.up = torch.stack([dev(tensors[f"expert_up#{e}"]) for e in range(self.experts)]).contiguous()
        self.down = torch.stack([dev(tensors[f"expert_down#{e}"]) for e in range(self.experts)]).contiguous()
        if self.shared_ff:
            if self.shared_kind != "swiglu":
                self.router = torch.cat([self.router, dev(tensors["shared_sg"]).reshape(1, -1)]).contiguous()
            g, u = dev(tensors["shared_gate"]), dev(tensors["shared_up"])
            self.shared_gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
            self.shared_down = dev(tensors["shared_down"]).contiguous()

    supports_onto = True

    def input_weight(self):
        """The router's matrix (with the shared gate's row), for a caller that stacks
        it with other matrices of the same input; `adopt_input_weight` hands back
        this part's rows of the stacked matrix."""
        return self.router

    def adopt_input_weight(self, rows: torch.Tensor) -> None:
        self.router = rows

    def forward(self, x, residual=None, onto=None, proj=None):
        """`onto`: a 32-bit delta another part made from the same input (a mixer
        beside this feed-forward); the result is added onto it and it is returned.
        `proj` = (float32 rows, first column): the router's product, already made
        by the caller as part of a stacked one."""
        if proj is None:
            logits, col0 = ops.linear(x, self.router, out_dtype=torch.float32), 0  # [rows, experts (+ the shared gate)]
        else:
            logits, col0 = proj
        ids, wts = ops.moe_route(logits, self.router_bias, self.top, experts=self.experts, scores=self.scores,
                                 col0=col0, scale=self.score_scale)
        ops.prof_mark("moe_router")
        out = ops.moe_experts(x, self.up, self.down, ids, wts, self.activation, self.weight_input, self.alpha,
                              self.limit)
        ops.prof_mark("moe_experts")
        if self.shared_ff and self.shared_kind == "swiglu":
            # the shared expert as it is: gate and up woven into one product, added to the experts' sum
            shared = ops.linear(ops.linear_swiglu(x, self.shared_gate_up), self.shared_down, out_dtype=torch.float32)
            ops.add_(out, shared)
            ops.prof_mark("moe_shared")
        elif self.shared_ff:
            act = ops.linear_glu_clamped(x, self.shared_gate_up, self.alpha, self.shared_limit)
            shared = ops.linear(act, self.shared_down, out_dtype=torch.float32)
            if onto is not None:  # one launch adds both the experts' sum and the gated shared expert
                ops.row_gate_add_(onto, shared, logits, col0 + self.experts, extra=out)
                ops.prof_mark("moe_shared")
                return onto
            ops.row_gate_add_(out, shared, logits, col0 + self.experts)
            ops.prof_mark("moe_shared")
        return out if onto is None else ops.add_(onto, out)
