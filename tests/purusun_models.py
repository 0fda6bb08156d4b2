"""Tiny Purusun models for tests: configurations that differ in every size and
option, and weights reshaped so that a fault shows.

Random N(0, 0.02) weights would hide most faults: the values (the raw keys)
and every sublayer's result would be tiny beside the residual, the step sizes
of the scan nearly constant and the gates all near a half.  `sharpen` scales
groups of tensors so that the attention's scores spread over several units (a
few keys dominate each softmax, so a window that is one token off, a kept
first token or a wrong angle shows), the values and the sublayers' results
weigh as much as the residual, the scan's step sizes and decays cover their
range and the gates swing.
"""

from __future__ import annotations

import os
import tempfile
from typing import Dict, Tuple

import numpy as np


def attention(heads, kv_heads, dim, scale, rot=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot is not None:
        base, dims, scaling = rot
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if mask is not None:
        m["mask"] = {"size": mask[0]}
        if mask[1] is not None:
            m["mask"]["keep_first"] = mask[1]
    return {"type": "attention", "mixer": m}


def scan(inner, state, dt_rank, conv):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(vocab, width, eps, streams, loop, layers):
    out = {"architecture": "Purusun", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(l, mlp=m) for l, m in layers]}
    if streams is not None:
        out["streams"] = streams
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# A: two streams; the first two of three layers run twice; a rotation of half a head with scaled
# frequencies (wavelengths on both sides of the blend and inside it), a window of 20 with 3 kept
# tokens; a scan; heads of 64 (the decode kernel takes their pages by TMA) with the whole head
# rotated, a window of 70 whose kept tokens (65) reach into a second page; a layer without a
# feed-forward
PUR_A = model(97, 64, 1e-5, 2, (0, 2, 2), [
    (attention(4, 2, 16, 0.9, (100.0, 8, (8.0, 1.0, 4.0, 64)), (20, 3)), dense(96)),
    (scan(48, 8, 4, 3), dense(40)),
    (attention(2, 1, 64, 0.4, (10000.0, 64, None), (70, 65)), None),
])
# B: the ordinary single residual (no streams key), no loop; an attention without a window and
# without a rotation; a scan without a filter state (one tap), one state a channel, rank one
PUR_B = model(130, 72, 1e-6, None, None, [
    (attention(6, 1, 8, 1.2, None, None), dense(80)),
    (scan(24, 1, 1, 1), dense(56)),
    (attention(2, 2, 32, 0.5, (50.0, 2, None), (5, 0)), dense(16)),
])
# C: one stream with its read, write and mix tensors; a width that is no multiple of 8, heads of
# 40 with 20 dimensions rotated, a window of exactly a page without kept tokens; the middle layer
# alone runs three times; five taps, five states, rank three
PUR_C = model(61, 100, 1e-5, 1, (1, 2, 3), [
    (attention(3, 3, 40, 0.5, (1000.0, 20, (2.0, 0.5, 2.0, 32)), (64, None)), dense(52)),
    (scan(50, 5, 3, 5), None),
    (attention(1, 1, 12, 1.0, (20.0, 12, None), (33, 1)), dense(24)),
])
# D: heads of 128 (prompts take the tensor-core kernel with accumulators in tensor memory), four
# streams, a loop of one pass, 64 states a channel (sixteen lanes a channel)
PUR_D = model(200, 128, 1e-5, 4, (0, 2, 1), [
    (attention(8, 2, 128, 0.2, (500000.0, 32, (4.0, 1.0, 4.0, 128)), (33, 1)), dense(256)),
    (scan(256, 64, 8, 4), dense(64)),
])
# E: kept tokens over more than two pages (130) with a window of 200, six heads on one key head;
# 130 states a channel (more than four a lane), two taps; the whole model runs twice
PUR_E = model(77, 96, 1e-5, 3, (0, 2, 2), [
    (attention(6, 1, 64, 0.35, (10000.0, 16, (16.0, 1.0, 8.0, 256)), (200, 130)), dense(40)),
    (scan(16, 130, 2, 2), dense(48)),
])

ALL = {"A": PUR_A, "B": PUR_B, "C": PUR_C, "D": PUR_D, "E": PUR_E}

# tensor-name suffix -> factor (the longest matching suffix counts)
SHARP = (("mix.q", 8.0), ("mix.k", 30.0), ("mix.g", 15.0), ("mix.o", 12.0), ("q.norm", 1.5),
         ("mix.in", 20.0), ("mix.x", 15.0), ("mix.dt", 15.0), ("mlp.up", 15.0), ("mlp.down", 4.0),
         ("embed", 25.0))

_FOLDERS: Dict[Tuple[str, int, str, object], str] = {}


def factor(name: str) -> float:
    best, f = -1, 1.0
    for suffix, value in SHARP:
        if name.endswith(suffix) and len(suffix) > best:
            best, f = len(suffix), value
    return f


def model_folder(name: str, seed: int = 3, dtype: str = "float32", sharp=True) -> str:
    """A model folder with the framework's random weights, sharpened; made once.
    `sharp` "mild": the square roots of the factors, for runs in bfloat16, whose
    rounding the full factors would amplify beyond what a tolerance can tell
    from a fault."""
    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors

    key = (name, seed, dtype, sharp)
    if key not in _FOLDERS:
        d = tempfile.mkdtemp(prefix=f"rfx_pur_{name}_")
        write_random_model(ALL[name], seed, d, dtype)
        if sharp:
            path = os.path.join(d, "model.safetensors")
            f = SafetensorsFile(path)
            tensors = [(k, f.tensor(k).clone()) for k in f.keys()]
            f.close()
            write_safetensors(path, [(k, (t.float() * (factor(k) ** 0.5 if sharp == "mild" else factor(k))).to(t.dtype)) for k, t in tensors])
        _FOLDERS[key] = d
    return _FOLDERS[key]


def tokens(n: int, vocab: int, seed: int):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]
