"""A causal language model put together from a `ModelSpec`.

embedding -> the layers in run order -> final norm -> head, with the logits
computed only at the rows a step asks for (the reference computes them for the
last row: src/model/dense.rs:2019-2025, src/model/mod.rs:1191-1202).  The model
holds parts and weights; what a step changes lives in the cache and the batch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import ops
from ..cache.specs import KVSpec, StateSpec
from ..config.spec import ModelSpec, RunEntry
from ..config.spec import names_dict
from ..parts.registry import BLOCKS, EMBEDDING_TERMS, NORMS, TensorInfo


@dataclass
class RunContext:
    """What a mixer gets besides its input rows."""

    batch: Any                 # StepBatch
    writes_cache: bool
    kv: Any = None             # KVView of this run's cache entry, if it has one
    state: Any = None          # [slots, *shape] tensor of this run's state, if any
    entry: int = -1
    # a mixer whose `cache_spec()` is a tuple: its views, in the tuple's order
    # (`kv` and `state` are then the first of each kind)
    parts: Any = None


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[Tuple[str, ...], TensorInfo]]:
    """tensor name -> (where it goes, TensorInfo) for the whole model."""
    out: Dict[str, Tuple[Tuple[str, ...], TensorInfo]] = {}
    out[spec.embedding_name] = (("embedding",), TensorInfo((spec.vocab_size, spec.hidden_size), "table"))
    for ti, term in enumerate(spec.embedding_terms):
        names = names_dict(term.names)
        for role, info in EMBEDDING_TERMS.get(term.kind).tensor_specs(term).items():
            out[names.get(role, role)] = (("embedding_term", str(ti), role), info)
    for li, layer in enumerate(spec.layers):
        for name, (part, role, info) in BLOCKS.get(layer.block).tensor_names(layer).items():
            out[name] = (("layer", str(li), part, role), info)
    if spec.stream_mix_name is not None:
        out[spec.stream_mix_name] = (("stream_mix",), TensorInfo((spec.hidden_size, 2 * spec.hidden_size), "matrix"))
    if spec.pass_vectors_name is not None:
        out[spec.pass_vectors_name] = (("pass_vectors",), TensorInfo((spec.pass_vectors, spec.hidden_size), "bias"))
    out[spec.final_norm_name] = (("final_norm",), NORMS.get(spec.final_norm.kind).tensor_specs(spec.final_norm)["weight"])
    if not spec.tie_word_embeddings:
        out[spec.head_name] = (("head",), TensorInfo((spec.vocab_size, spec.hidden_size), "matrix"))
    return out


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be float32 or bfloat16")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.layers = [BLOCKS.get(l.block)(l, dtype, self.device) for l in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, dtype, self.device)
        self.embedding_terms = [EMBEDDING_TERMS.get(t.kind)(t, dtype, self.device) for t in spec.embedding_terms]
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.stream_mix: Optional[torch.Tensor] = None
        self.pass_vectors: Optional[torch.Tensor] = None
        # a probe for tests and diagnostics: called after every layer run with (index,
        # run, layer, hidden, pending); None in normal use
        self.after_run = None
        if any(r.mixes_input for r in spec.run_order) and spec.stream_mix_name is None:
            raise ValueError("a run mixes its input but the model names no stream-mix matrix")
        if any(r.pass_vector is not None for r in spec.run_order) and spec.pass_vectors_name is None:
            raise ValueError("a run adds a pass vector but the model names no tensor of them")

    @property
    def capturable(self) -> bool:
        """True when every layer and the final norm declare `capturable = True`:
        their launches take positions, slots and lengths from device memory
        (`StepBatch`'s device fields) and nothing forces the host to wait, so a
        decode step can be captured once and replayed.  A part that walks host
        lists, or synchronises (a `.nonzero()`, an `.item()`), leaves the
        attribute out or sets it False, and the engine then runs every step
        eagerly."""
        return (all(bool(getattr(l, "capturable", False)) for l in self.layers)
                and all(bool(getattr(t, "capturable", False)) for t in self.embedding_terms)
                and bool(getattr(self.final_norm, "capturable", False)))

    # --- weights ----------------------------------------------------------
    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """`tensors`: every name of `expected_tensors`, already checked."""
        exp = expected_tensors(self.spec)
        per_layer: Dict[int, Dict[str, Dict[str, torch.Tensor]]] = {}
        per_term: Dict[int, Dict[str, torch.Tensor]] = {}
        for name, (where, _info) in exp.items():
            t = tensors[name]
            if where[0] == "embedding":
                self.embedding = t.to(device=self.device, dtype=self.dtype).contiguous()
            elif where[0] == "head":
                self.head = t.to(device=self.device, dtype=self.dtype).contiguous()
            elif where[0] == "final_norm":
                self.final_norm.bind({"weight": t})
            elif where[0] == "stream_mix":
                self.stream_mix = t.to(device=self.device, dtype=self.dtype).contiguous()
            elif where[0] == "pass_vectors":
                self.pass_vectors = t.to(device=self.device, dtype=torch.float32).contiguous()
            elif where[0] == "embedding_term":
                per_term.setdefault(int(where[1]), {})[where[2]] = t
            else:
                _, li, part, role = where
                per_layer.setdefault(int(li), {}).setdefault(part, {})[role] = t
        for li, layer in enumerate(self.layers):
            layer.bind(per_layer.get(li, {}))
        for ti, term in enumerate(self.embedding_terms):
            term.bind(per_term.get(ti, {}))
        if self.spec.tie_word_embeddings:
            self.head = self.embedding  # the same storage, no copy

    # --- cache ------------------------------------------------------------
    def cache_entry_specs(self) -> Dict[int, Any]:
        out = {}
        for entry, li in self.spec.cache_entries().items():
            mixer = self.layers[li].mixer
            out[entry] = mixer.cache_spec() if hasattr(mixer, "cache_spec") else None
        # what the embedding's terms keep per sequence: entries below zero, beside the runs' own
        for ti, term in enumerate(self.embedding_terms):
            st = term.state_spec()
            if st is not None:
                out[self.term_entry(ti)] = st
        return out

    @staticmethod
    def term_entry(index: int) -> int:
        """Cache entry of embedding term `index` (the runs' entries count from zero up)."""
        return -1 - index

    # --- forward ----------------------------------------------------------
    def hidden_states(self, batch, cache, rows=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """The residual after the last layer, [rows, hidden] 32-bit, and what is still
        to be added to it.  `rows` (int32 on the device) asks for those rows only;
        whether they were cut out says `self.cuts_rows` (a block arrangement that
        keeps the residual in a form of its own makes the ordinary one at the end,
        and then only for the rows that are wanted)."""
        ops.prof_mark("start")
        # a token id outside the vocabulary (possible only for ids fed from the device)
        # gives a zero row and sets the device's error word, which `check_errors` reads
        h = ops.embed(self.embedding, batch.tokens, self.spec.embedding_scale,
                      ops.device_error_word(self.device))
        for ti, term in enumerate(self.embedding_terms):
            entry = self.term_entry(ti)
            term.add(h, batch, cache.state(entry) if cache.has(entry) == "state" else None)
        if self.spec.residual_streams > 1:
            # the residual as several parallel copies: the embedding output into each
            h = ops.hyper_expand(h, self.spec.residual_streams)
        ops.prof_mark("embed")
        pending = None
        order = self.spec.run_order
        # the embedding output, for the runs that start from a mix of it and the stream
        x0 = ops.keep_copy(h) if any(r.mixes_input or r.adds_input for r in order) else None
        for i, run in enumerate(order):
            # the norm that will consume this run's result: the next run's first norm, or the final one
            if i + 1 == len(order):
                # a block that would make the last norm for every row leaves it to `logits`
                next_norm = (None if getattr(self.layers[run.layer], "skips_final_norm_fusion", False)
                             else self.final_norm)
            elif order[i + 1].mixes_input or order[i + 1].pass_vector is not None:
                next_norm = None  # the stream goes through the mix first: no norm to begin here
            else:
                next_norm = getattr(self.layers[order[i + 1].layer], "fusable_first_norm", None)
            ops.workspace.next_phase()  # this run's working memory; the last run's results stay readable
            if run.mixes_input:
                # x <- W [x; x0]: the stream (with what the run before left to add) beside the
                # embedding output, through one product; the new stream is 32-bit
                if isinstance(pending, ops.NormedInput):
                    pending = None  # the stream already holds the sum
                both = ops.stream_concat(h, pending, x0, self.dtype)
                h.copy_(ops.linear(both, self.stream_mix, out_dtype=torch.float32))  # the stream's own memory
                pending = None
                ops.prof_mark("stream_mix")
            if run.pass_vector is not None:
                # the start of a pass: x <- x (+ x0) + the pass's vector, in the stream's own memory
                if pending is not None and not isinstance(pending, ops.NormedInput):
                    ops.add_(h, pending)
                pending = None
                ops.loop_input_(h, x0 if run.adds_input else None, self.pass_vectors[run.pass_vector])
                ops.prof_mark("stream_mix")
            ctx = RunContext(batch=batch, writes_cache=run.writes_cache, entry=run.cache)
            kind = cache.has(run.cache)
            if kind == "kv":
                ctx.kv = cache.kv(run.cache)
            elif kind == "state":
                ctx.state = cache.state(run.cache)
            elif kind == "parts":
                ctx.parts = cache.views(run.cache)
                ctx.kv = next((v for v in ctx.parts if not isinstance(v, torch.Tensor)), None)
                ctx.state = next((v for v in ctx.parts if isinstance(v, torch.Tensor)), None)
            layer = self.layers[run.layer]
            if hasattr(layer, "fusable_first_norm"):
                h, pending = layer.forward(h, pending, ctx, next_norm=next_norm)
            else:
                h, pending = layer.forward(h, pending, ctx)
            if self.after_run is not None:
                self.after_run(i, run, layer, h, pending)
        # a block arrangement that keeps the residual in a form of its own (several
        # streams) hands back the ordinary one: [rows, hidden] and a delta or None
        last = self.layers[order[-1].layer] if order else None
        if last is not None and hasattr(last, "finish"):
            h, pending = last.finish(h, pending, rows=rows)
        return h, pending

    @property
    def cuts_rows(self) -> bool:
        order = self.spec.run_order
        return bool(order) and hasattr(self.layers[order[-1].layer], "finish")

    def logits(self, hidden: torch.Tensor, pending, rows: torch.Tensor, rows_host=None) -> torch.Tensor:
        """Final norm and head on the wanted rows only; float32 [len(rows), V]."""
        if isinstance(pending, ops.NormedInput):
            # fused decode path: hidden already holds the last delta
            if rows_host is not None and list(rows_host) == list(range(hidden.shape[0])):
                normed = pending  # every row wanted, in order: the head product takes them as they are
            else:
                normed = self.final_norm(hidden, rows=rows)
        else:
            normed = self.final_norm(hidden, delta=pending, rows=rows)
        out = ops.linear(normed, self.head, out_dtype=torch.float32, own=True)  # the caller's to keep
        out = self.finish_logits(out)
        ops.prof_mark("head")
        return out

    def finish_logits(self, out: torch.Tensor) -> torch.Tensor:
        """The model's scale on the logits and, where it has one, the tanh cap."""
        if self.spec.logit_softcap:
            return ops.logit_finish_(out, self.spec.logit_scale, self.spec.logit_softcap)
        if self.spec.logit_scale != 1.0:
            out = out * self.spec.logit_scale
        return out

    def normed_rows(self, hidden: torch.Tensor, pending, rows: torch.Tensor) -> torch.Tensor:
        """The final norm on the wanted rows, in the model's dtype."""
        if isinstance(pending, ops.NormedInput):
            return self.final_norm(hidden, rows=rows)  # hidden already holds the last delta
        return self.final_norm(hidden, delta=pending, rows=rows)

    def scores(self, batch, cache, ids: torch.Tensor) -> torch.Tensor:
        """For each wanted row the head's logit of one given token id
        (`ids`, int32 on the device, one per wanted row), float32 [wanted]: only
        those rows of the head are read (src/model/dense.rs:2073-2133)."""
        h, pending = self.hidden_states(batch, cache, rows=batch.want_rows)
        rows = None if self.cuts_rows else batch.want_rows
        out = self.finish_logits(ops.gather_dot(self.normed_rows(h, pending, rows), self.head, ids))
        ops.prof_mark("head")
        return out

    def forward(self, batch, cache) -> torch.Tensor:
        h, pending = self.hidden_states(batch, cache, rows=batch.want_rows)
        if self.cuts_rows:  # h holds the wanted rows, in order
            return self.logits(h, pending, None)
        return self.logits(h, pending, batch.want_rows, batch.want_rows_host)
