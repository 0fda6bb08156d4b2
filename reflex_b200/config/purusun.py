"""Typed configuration of the Purusun design, read from config.json.

config.json keys: `architecture` ("Purusun"), `vocab`, `width`, `norm.eps`,
optional `streams` (the residual as that many parallel copies; absent: the
ordinary single residual), optional `loop` (`start`, `stop`, `times`: layers
start .. stop - 1 run `times` times in a row with the same weights), and
`layers`, a list whose entries give `type` (the mixer: "attention" or
"mamba1"), `mixer` (its sizes) and `mlp` (`kind` "dense" with `ff`; null for a
layer without a feed-forward).

An attention's `mixer`: `heads`, `kv_heads`, `dim`, `vdim` (equal to `dim`: the
values are the keys as projected), `scale`, optional `rot` {`base`, `dims`,
optional `scaling` {`factor`, `low`, `high`, `original`}} and optional `mask`
{`size`, optional `keep_first`}.  A selective scan's: `inner`, `state`,
`dt_rank`, `conv`.  Every size and every constant that differs between models
comes from here.  Missing or ill-typed keys are reported together, by name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..errors import CheckpointError

NUM = (int, float)


@dataclass
class PurusunLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class PurusunConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: Optional[int] = None
    loop: Optional[Dict[str, int]] = None
    layers: List[PurusunLayer] = field(default_factory=list)
    torch_dtype: str = "bfloat16"
    # the design fixes no longest context; the cache bounds it
    max_positions: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "PurusunConfig":
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
        streams = optional(cfg, "streams", int, "")
        loop = cfg.get("loop")
        if loop is not None:
            for k in ("start", "stop", "times"):
                need(loop, k, int, "loop.")
        layers_in = cfg.get("layers")
        layers: List[PurusunLayer] = []
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
            if kind == "attention":
                for k in ("heads", "kv_heads", "dim"):
                    need(mixer, k, int, where + "mixer.")
                optional(mixer, "vdim", int, where + "mixer.")
                need(mixer, "scale", NUM, where + "mixer.")
                rot = mixer.get("rot")
                if rot is not None:
                    need(rot, "base", NUM, where + "mixer.rot.")
                    need(rot, "dims", int, where + "mixer.rot.")
                    sc = rot.get("scaling") if isinstance(rot, dict) else None
                    if sc is not None:
                        for k in ("factor", "low", "high", "original"):
                            need(sc, k, NUM, where + "mixer.rot.scaling.")
                mask = mixer.get("mask")
                if mask is not None:
                    need(mask, "size", int, where + "mixer.mask.")
                    optional(mask, "keep_first", int, where + "mixer.mask.")
            elif kind == "mamba1":
                for k in ("inner", "state", "dt_rank", "conv"):
                    need(mixer, k, int, where + "mixer.")
            elif kind is not None:
                problems.append(f"{where}type={kind!r} (known: attention, mamba1)")
                continue
            mlp = l.get("mlp")
            if mlp is not None:
                mk = need(mlp, "kind", str, where + "mlp.")
                if mk == "dense":
                    need(mlp, "ff", int, where + "mlp.")
                elif mk is not None:
                    problems.append(f"{where}mlp.kind={mk!r} (known: dense)")
            layers.append(PurusunLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        if problems:
            raise CheckpointError("config.json: missing or ill-typed keys: " + ", ".join(problems))
        out = cls(vocab=vocab, width=width, norm_eps=float(eps), streams=streams,
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
        if self.streams is not None and not (1 <= self.streams <= 8):
            bad("streams must be between 1 and 8")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp["start"] < lp["stop"] <= len(self.layers)) or lp["times"] < 1:
                bad("loop: 0 <= start < stop <= number of layers and times >= 1 are needed")
        for i, l in enumerate(self.layers):
            m = l.mixer
            if l.type == "attention":
                for k in ("heads", "kv_heads", "dim"):
                    if m[k] <= 0:
                        bad(f"layers[{i}].mixer.{k} must be positive")
                if m["heads"] % m["kv_heads"]:
                    bad(f"layers[{i}].mixer: heads must be a multiple of kv_heads")
                if m.get("vdim") is not None and m["vdim"] != m["dim"]:
                    bad(f"layers[{i}].mixer: vdim must equal dim (the values are the keys as projected)")
                rot = m.get("rot")
                if rot is not None and (rot["dims"] % 2 or not (0 <= rot["dims"] <= m["dim"])):
                    bad(f"layers[{i}].mixer.rot.dims must be even and at most dim")
                mask = m.get("mask")
                if mask is not None and (mask["size"] <= 0 or int(mask.get("keep_first") or 0) < 0):
                    bad(f"layers[{i}].mixer.mask: size must be positive and keep_first not negative")
            else:
                for k in ("inner", "state", "dt_rank", "conv"):
                    if m[k] <= 0:
                        bad(f"layers[{i}].mixer.{k} must be positive")
            if l.mlp is not None and l.mlp["ff"] <= 0:
                bad(f"layers[{i}].mlp.ff must be positive")

    def to_dict(self) -> Dict[str, Any]:
        out = dict(self.raw)
        out.update({
            "architecture": "Purusun", "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers],
        })
        if self.streams is not None:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out
