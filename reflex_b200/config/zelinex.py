"""Typed configuration of the Zelinex design, read from config.json.

config.json keys: `architecture` ("Zelinex"), `vocab`, `width`, `norm.eps`,
`residual_mult` (the factor on every normed sublayer result), optional `loop`
(`start`, `stop`, `times`: layers start .. stop - 1 run `times` times in a row
with the same weights), and `layers`, a list whose entries give `type` (the
mixer: "parallel" or "general_delta"), `mixer` (its sizes) and `mlp` (`kind`
"dense" with `ff`; `kind` "moe" with `expert.ff`, `router.experts`,
`router.top`, `router.scale` and optional `shared.ff`; null for a layer
without a feed-forward).

A "parallel" mixer: `left` (an attention: `heads`, `kv_heads`, `dim`, `vdim`,
`scale`, optional `rot` {`base`, `dims`} and `mask` {`size`}), `right` (a
state-space recurrence: `heads`, `vdim`, `state`, `groups`, `conv`,
`norm_groups`), `left_scale`, `right_scale`.  A "general_delta" mixer: `heads`,
`dim`.  Every size and every constant that differs between models comes from
here.  Missing or ill-typed keys are reported together, by name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..errors import CheckpointError

NUM = (int, float)


@dataclass
class ZelinexLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class ZelinexConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float = 1.0
    loop: Optional[Dict[str, int]] = None
    layers: List[ZelinexLayer] = field(default_factory=list)
    torch_dtype: str = "bfloat16"
    # the design fixes no longest context; the cache bounds it
    max_positions: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "ZelinexConfig":
        problems: List[str] = []

        def need(d, key, types, where):
            v = d.get(key) if isinstance(d, dict) else None
            if v is None or isinstance(v, bool) or not isinstance(v, types):
                problems.append(f"{where}{key}")
                return None
            return v

        def optional(d, key, types, where):
            if not isinstance(d, dict) or d.get(key) is None:
                return None
            return need(d, key, types, where)

        vocab = need(cfg, "vocab", int, "")
        width = need(cfg, "width", int, "")
        norm = cfg.get("norm") if isinstance(cfg.get("norm"), dict) else {}
        eps = need(norm, "eps", NUM, "norm.")
        mult = optional(cfg, "residual_mult", NUM, "")
        loop = cfg.get("loop")
        if loop is not None:
            for k in ("start", "stop", "times"):
                need(loop, k, int, "loop.")
        layers_in = cfg.get("layers")
        layers: List[ZelinexLayer] = []
        if not isinstance(layers_in, list) or not layers_in:
            problems.append("layers")
            layers_in = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]."
            kind = need(l, "type", str, where)
            mixer = l.get("mixer") if isinstance(l, dict) and isinstance(l.get("mixer"), dict) else None
            if mixer is None:
                problems.append(where + "mixer")
                continue
            if kind == "parallel":
                left = mixer.get("left") if isinstance(mixer.get("left"), dict) else None
                right = mixer.get("right") if isinstance(mixer.get("right"), dict) else None
                if left is None:
                    problems.append(where + "mixer.left")
                else:
                    for k in ("heads", "kv_heads", "dim", "vdim"):
                        need(left, k, int, where + "mixer.left.")
                    need(left, "scale", NUM, where + "mixer.left.")
                    rot = left.get("rot")
                    if rot is not None:
                        need(rot, "base", NUM, where + "mixer.left.rot.")
                        need(rot, "dims", int, where + "mixer.left.rot.")
                    if left.get("mask") is not None:
                        need(left["mask"], "size", int, where + "mixer.left.mask.")
                if right is None:
                    problems.append(where + "mixer.right")
                else:
                    for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                        need(right, k, int, where + "mixer.right.")
                for k in ("left_scale", "right_scale"):
                    need(mixer, k, NUM, where + "mixer.")
            elif kind == "general_delta":
                for k in ("heads", "dim"):
                    need(mixer, k, int, where + "mixer.")
            elif kind is not None:
                problems.append(f"{where}type={kind!r} (known: parallel, general_delta)")
                continue
            mlp = l.get("mlp")
            if mlp is not None:
                mk = need(mlp, "kind", str, where + "mlp.")
                if mk == "dense":
                    need(mlp, "ff", int, where + "mlp.")
                elif mk == "moe":
                    need(mlp.get("expert"), "ff", int, where + "mlp.expert.")
                    for k in ("experts", "top"):
                        need(mlp.get("router"), k, int, where + "mlp.router.")
                    optional(mlp.get("router"), "scale", NUM, where + "mlp.router.")
                    if mlp.get("shared") is not None:
                        need(mlp["shared"], "ff", int, where + "mlp.shared.")
                elif mk is not None:
                    problems.append(f"{where}mlp.kind={mk!r} (known: dense, moe)")
            layers.append(ZelinexLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        if problems:
            raise CheckpointError("config.json: missing or ill-typed keys: " + ", ".join(problems))
        out = cls(vocab=vocab, width=width, norm_eps=float(eps),
                  residual_mult=1.0 if mult is None else float(mult),
                  loop=None if loop is None else {k: int(loop[k]) for k in ("start", "stop", "times")},
                  layers=layers, torch_dtype=str(cfg.get("torch_dtype", "bfloat16")),
                  max_positions=int(cfg.get("max_positions", 1 << 20)), raw=dict(cfg))
        out.validate()
        return out

    def validate(self) -> None:
        def bad(msg: str) -> None:
            raise CheckpointError(f"config.json: {msg}")

        if self.vocab <= 0 or self.width <= 0:
            bad("vocab and width must be positive")
        if not (self.norm_eps > 0):
            bad("norm.eps must be positive")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp["start"] < lp["stop"] <= len(self.layers)) or lp["times"] < 1:
                bad("loop: 0 <= start < stop <= number of layers and times >= 1 are needed")
        for i, l in enumerate(self.layers):
            m = l.mixer
            if l.type == "parallel":
                a, r = m["left"], m["right"]
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if a[k] <= 0:
                        bad(f"layers[{i}].mixer.left.{k} must be positive")
                if a["heads"] % a["kv_heads"]:
                    bad(f"layers[{i}].mixer.left: heads must be a multiple of kv_heads")
                rot = a.get("rot")
                if rot is not None and (rot["dims"] % 2 or not (0 <= rot["dims"] <= a["dim"])):
                    bad(f"layers[{i}].mixer.left.rot.dims must be even and at most dim")
                if a.get("mask") is not None and a["mask"]["size"] <= 0:
                    bad(f"layers[{i}].mixer.left.mask.size must be positive")
                for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    if r[k] <= 0:
                        bad(f"layers[{i}].mixer.right.{k} must be positive")
                if r["heads"] % r["groups"] or (r["heads"] * r["vdim"]) % r["norm_groups"]:
                    bad(f"layers[{i}].mixer.right: groups must divide heads and norm_groups heads * vdim")
            else:
                for k in ("heads", "dim"):
                    if m[k] <= 0:
                        bad(f"layers[{i}].mixer.{k} must be positive")
            if l.mlp is not None:
                if l.mlp["kind"] == "dense":
                    if l.mlp["ff"] <= 0:
                        bad(f"layers[{i}].mlp.ff must be positive")
                else:
                    rt = l.mlp["router"]
                    if l.mlp["expert"]["ff"] <= 0 or not (0 < rt["top"] <= rt["experts"]):
                        bad(f"layers[{i}].mlp: expert.ff must be positive and 0 < router.top <= router.experts")

    def to_dict(self) -> Dict[str, Any]:
        out = dict(self.raw)
        out.update({
            "architecture": "Zelinex", "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
            "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers],
        })
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out
