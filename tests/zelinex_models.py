"""Tiny Zelinex models for tests: configurations that differ in every size and
option, and weights reshaped so that a fault shows.

Random N(0, 0.02) weights would hide most faults: every score would be near
zero and every sigmoid weight near a half, the recurrences' inputs tiny, the
step sizes and decays nearly constant and the gates all near a half.  `sharpen`
scales groups of tensors so that the attention's scores spread over several
units on both sides of zero (some keys count fully, others not at all, so a
window that is one token off or a wrong angle shows), the recurrences' decays
and removal rates cover their range, the gates swing and the router's logits
part.
"""

from __future__ import annotations

import os
import tempfile
from typing import Dict, Tuple

import numpy as np


def pair(heads, kv_heads, dim, vdim, scale, rot, mask, s_heads, s_vdim, state, groups, conv, norm_groups,
         left_scale, right_scale):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        left["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask is not None:
        left["mask"] = {"size": mask}
    right = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv,
             "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}}


def delta(heads, dim):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale, shared):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def model(vocab, width, eps, mult, loop, layers):
    out = {"architecture": "Zelinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": [dict(l, mlp=m) for l, m in layers]}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# A: the first two of three layers run twice; values wider than keys, a quarter of each head
# rotated, a window of 20; two state-space heads on one group, three taps; a delta rule beside
# four experts of which two are chosen and a shared one; heads of 64 with the whole head
# rotated, a window of 70 (longer than a page), two groups, four norm parts; a layer without
# a feed-forward
ZEL_A = model(97, 64, 1e-5, 0.8, (0, 2, 2), [
    (pair(4, 2, 16, 24, 0.5, (100.0, 8), 20, 2, 16, 8, 1, 3, 1, 0.7, 1.2), dense(96)),
    (delta(2, 16), moe(24, 4, 2, 1.0, 32)),
    (pair(2, 1, 64, 32, 0.25, (10000.0, 64), 70, 4, 8, 16, 2, 4, 4, 1.0, 0.4), None),
])
# B: no loop; an attention without a window and without a rotation, six heads on one key
# head; one state a head, one tap (no filter state), as many groups as heads; one delta head;
# one expert; a multiplier of one
ZEL_B = model(130, 72, 1e-6, 1.0, None, [
    (pair(6, 1, 8, 8, 1.2, None, None, 3, 24, 1, 3, 1, 1, 0.5, 0.5), dense(80)),
    (delta(1, 32), moe(16, 1, 1, 2.0, 0)),
    (delta(3, 8), dense(56)),
])
# C: a width that is no multiple of 8; the middle layer alone runs three times; five delta
# heads of 20; every expert chosen; a window of exactly a page; values narrower than keys;
# 48 channels a state-space head (a block takes them in two slices), 40 states, five taps
ZEL_C = model(61, 100, 1e-5, 0.6, (1, 2, 3), [
    (delta(5, 20), moe(12, 3, 3, 0.5, 20)),
    (pair(3, 3, 40, 16, 0.3, (1000.0, 20), 64, 2, 48, 40, 2, 5, 2, 1.5, 0.3), dense(52)),
    (delta(2, 50), dense(24)),
])
# D: heads of 128 with values of 64, a window of 33; eight state-space heads of 64 channels and
# 64 states; delta heads of 128 (a block takes their columns in four slices); a loop of one pass
ZEL_D = model(200, 256, 1e-5, 0.75, (0, 2, 1), [
    (pair(8, 2, 128, 64, 0.1, (500000.0, 32), 33, 8, 64, 64, 2, 4, 2, 0.9, 0.45), dense(256)),
    (delta(2, 128), moe(64, 8, 3, 1.25, 64)),
])
# E: the whole model runs three times; a long window (200) over several pages, twelve heads
# on three key heads, keys of 32 and values of 128; two taps
ZEL_E = model(77, 96, 1e-5, 0.9, (0, 2, 3), [
    (pair(12, 3, 32, 128, 0.2, (10000.0, 16), 200, 6, 16, 24, 3, 2, 3, 0.8, 0.8), moe(40, 6, 2, 1.0, 0)),
    (delta(3, 32), dense(48)),
])

ALL = {"A": ZEL_A, "B": ZEL_B, "C": ZEL_C, "D": ZEL_D, "E": ZEL_E}

# tensor-name suffix -> factor (the longest matching suffix counts)
SHARP = (("left.q", 10.0), ("left.k", 30.0), ("left.pb", 3.0), ("right.in", 12.0), ("right.dt_bias", 2.0),
         ("mix.r", 10.0), ("mix.k", 25.0), ("mix.v", 10.0), ("mix.g", 15.0), ("mix.a", 15.0), ("mix.w1", 20.0),
         ("mix.w2", 40.0), ("mlp.up", 15.0), ("gate", 15.0), ("mlp.router", 30.0), ("embed", 25.0),
         ("loop.step", 0.5))

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
        d = tempfile.mkdtemp(prefix=f"rfx_zel_{name}_")
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
