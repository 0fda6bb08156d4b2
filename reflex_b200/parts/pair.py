"""Two mixers side by side on the same input.

out = (norm_l(left(h)) + norm_r(right(h))) / 2, each branch's output over its
root mean square (over the model width) times a weight of its own; or, with the
spec's `combine` = "scaled_sum", out = left_scale * left(h) + right_scale *
right(h) with no norm and no tensors of the pair's own.  The two
branches are registered mixers of any kind, named by the spec's `left` and
`right` parameters; what they keep in the cache is asked for together (a tuple
of their specs) and handed to each in turn.  A branch may return `(delta,
bias)`: a bias of its last product that this part's kernel adds before the
norm.  Branches that offer the matrix of their first product (`input_weight`,
`adopt_input_weight`, `forward(..., proj=)`) get it stacked with the other's:
one product of the shared input serves both, each reads its own columns, and
the stacked matrix is the only copy of those weights.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import MixerSpec, names_dict
from .registry import MIXERS, TensorInfo, register_mixer


def _as_tuple(spec):
    if spec is None:
        return ()
    return tuple(spec) if isinstance(spec, (tuple, list)) else (spec,)


@register_mixer("pair")
class PairMixer:
    SIDES = ("left", "right")

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.combine = str(spec.param("combine", "norm_mean"))
        if self.combine not in ("norm_mean", "scaled_sum"):
            raise ValueError(f"pair: combine must be norm_mean or scaled_sum, got {self.combine!r}")
        self.eps = float(spec.param("eps", 0.0) or 0.0)
        self.scales = (float(spec.param("left_scale", 1.0)), float(spec.param("right_scale", 1.0)))
        self.branches = [MIXERS.get(spec.param(side).kind)(spec.param(side), dtype, device) for side in self.SIDES]
        self.weights = [None, None]
        self.stacked = None   # both branches' first matrices, one above the other
        self.first_col = [0, 0]
        self.part_rows = [0, 0]

    @property
    def capturable(self) -> bool:
        return all(bool(getattr(b, "capturable", False)) for b in self.branches)

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        out = {}
        for side in cls.SIDES:
            sub = spec.param(side)
            for role, info in MIXERS.get(sub.kind).tensor_specs(sub).items():
                out[f"{side}/{role}"] = info
            if spec.param("combine", "norm_mean") == "norm_mean":
                out[f"{side}_out"] = TensorInfo((spec.hidden_size,), "norm")
        return out

    def cache_spec(self):
        """Everything the two branches keep, the left one's parts first."""
        return tuple(p for b in self.branches for p in _as_tuple(b.cache_spec() if hasattr(b, "cache_spec") else None))

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for i, (side, branch) in enumerate(zip(self.SIDES, self.branches)):
            branch.bind({role[len(side) + 1:]: t for role, t in tensors.items() if role.startswith(side + "/")})
            if self.combine == "norm_mean":
                self.weights[i] = tensors[f"{side}_out"].to(device=self.device, dtype=torch.float32).contiguous()
        if all(hasattr(b, "input_weight") and hasattr(b, "adopt_input_weight") for b in self.branches):
            parts = [b.input_weight() for b in self.branches]
            if all(p is not None and p.dtype == parts[0].dtype and p.shape[1] == parts[0].shape[1] for p in parts):
                # zero rows up to a multiple of 8, so that the product's rows stay 16-byte aligned
                rows = sum(p.shape[0] for p in parts)
                pad = torch.zeros((-rows % 8, parts[0].shape[1]), dtype=parts[0].dtype, device=parts[0].device)
                self.stacked = torch.cat(parts + [pad], dim=0).contiguous()
                row = 0
                for i, (b, p) in enumerate(zip(self.branches, parts)):
                    self.first_col[i] = row
                    self.part_rows[i] = p.shape[0]
                    b.adopt_input_weight(self.stacked[row:row + p.shape[0]])
                    row += p.shape[0]

    def input_weight(self):
        """The stacked matrix, for a caller that stacks it further (a block whose
        feed-forward reads the same input); None if the branches offered none."""
        return self.stacked

    def adopt_input_weight(self, rows: torch.Tensor) -> None:
        self.stacked = rows
        for b, lo, n in zip(self.branches, self.first_col, self.part_rows):
            b.adopt_input_weight(rows[lo:lo + n])

    def forward(self, x, ctx, proj=None):
        from ..engine.model import RunContext

        views = list(ctx.parts) if ctx.parts is not None else [v for v in (ctx.kv, ctx.state) if v is not None]
        outs = []
        col0 = 0
        if proj is not None:
            proj, col0 = proj  # the caller made the product, stacked with more of its own
        elif self.stacked is not None:
            proj = ops.linear(x, self.stacked, out_dtype=torch.float32)
            ops.prof_mark("qkv_gemm")
        for bi, branch in enumerate(self.branches):
            n = len(_as_tuple(branch.cache_spec() if hasattr(branch, "cache_spec") else None))
            mine, views = views[:n], views[n:]
            sub = RunContext(batch=ctx.batch, writes_cache=ctx.writes_cache, entry=ctx.entry, parts=mine)
            sub.kv = next((v for v in mine if not isinstance(v, torch.Tensor)), None)
            sub.state = next((v for v in mine if isinstance(v, torch.Tensor)), None)
            r = (branch.forward(x, sub) if proj is None
                 else branch.forward(x, sub, proj=(proj, col0 + self.first_col[bi])))
            outs.append(r if isinstance(r, tuple) else (r, None))
        (a, a_bias), (b, b_bias) = outs
        if self.combine == "scaled_sum":
            if a_bias is not None or b_bias is not None:
                raise ValueError("pair: the scaled sum takes branches without a deferred bias")
            out = ops.scaled_sum_(a, b, self.scales[0], self.scales[1])
            ops.prof_mark("pair_out")
            return out
        if b_bias is not None:  # the kernel takes one bias: give it the branch that has one
            if a_bias is not None:
                b = b + b_bias
            else:
                out = ops.branch_norm_mean(b, b_bias, self.weights[1], a, self.weights[0], self.eps)
                ops.prof_mark("pair_out")
                return out
        out = ops.branch_norm_mean(a, a_bias, self.weights[0], b, self.weights[1], self.eps)
        ops.prof_mark("pair_out")
        return out
