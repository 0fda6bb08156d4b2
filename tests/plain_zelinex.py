"""A plain, slow implementation of the Zelinex design, for tests.

Whole sequences, no cache, one function per mechanism, NumPy in double
precision; it shares no code with `reflex_b200`.  Linear weights are [out, in]
and applied as y = x W^T.

The design: a token embedding; layers with a norm before and a norm after each
sublayer, x <- x + m * post(sublayer(pre(x))), m one number of the model; the
mixer is either a pair side by side (an attention whose weights are sigmoids
of the biased scores, not normalised over the keys, with grouped heads, a
partial half-split rotation and a sliding window, beside a state-space
recurrence with one decay a head, a short convolution over x, B and C, and a
gated grouped norm; the two are summed with a weight each) or a delta-rule
recurrence with a decay and a removal rate per key channel; the feed-forward
is W_down xielu(W_up h) or a mixture of gated silu experts beside a shared one;
a stretch of layers may run several times with the same weights, each pass
starting from x + x0 (not the first) + a vector of the pass; the model's norm
and the embedding table as the head.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np

F = np.float64


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        b, e = ent["data_offsets"]
        raw = blob[b:e]
        if ent["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif ent["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif ent["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"plain reader: dtype {ent['dtype']} of {name}")
        out[name] = arr.astype(F).reshape(ent["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ------------------------------------------------------------------ elements
def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return rms_unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def xielu(z: np.ndarray, p: float, q: float) -> np.ndarray:
    """z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap, an = softplus(F(p)), 0.5 + softplus(F(q))
    zn = np.minimum(z, 0.0)
    return np.where(z > 0.0, ap * z * z + 0.5 * z, an * (np.expm1(zn) - zn) + 0.5 * z)


# ------------------------------------------------------------------ rotation
def rotate(t: np.ndarray, positions: np.ndarray, dims: int, base: float) -> np.ndarray:
    """t [T, heads, dim]: among the first `dims` dimensions i pairs with
    i + dims / 2 and the pair turns by position * base^(-2i / dims)."""
    half = dims // 2
    if half == 0:
        return t
    freqs = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions[:, None].astype(F) * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = t.copy()
    u, v = t[..., :half], t[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


# ------------------------------------------------- attention with sigmoid weights
def visible(T: int, window: Optional[int]) -> np.ndarray:
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    ok = j <= i
    if window:
        ok &= (i - j) < window
    return ok


def sigmoid_attention(h: np.ndarray, w: Dict[str, np.ndarray], m: dict) -> np.ndarray:
    """out_i = W_o concat_h sum_j sigmoid(q_i . k_j * scale + b_h) v_j over the
    visible j; nothing is normalised over the keys."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, dv)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        pos = np.arange(T)
        q, k = rotate(q, pos, int(rot["dims"]), float(rot["base"])), rotate(k, pos, int(rot["dims"]), float(rot["base"]))
    mask = visible(T, int(m["mask"]["size"]) if m.get("mask") else None)
    out = np.zeros((T, H, dv), dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"]) + w["pb"][hh]
        p = np.where(mask, sigmoid(s), 0.0)
        out[:, hh] = p @ v[:, g]
    return out.reshape(T, H * dv) @ w["o"].T


# ----------------------------------------------- state-space recurrence, a decay a head
def causal_conv(x: np.ndarray, taps_w: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """x [T, C]; taps_w [C, taps], the last tap meets the current token; zeros
    before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), x])
    out = np.tile(bias, (T, 1)).astype(F)
    for j in range(taps):
        out += padded[j:j + T] * taps_w[:, j]
    return out


def ssd_scan(x, B, C, dt, A, D, heads, groups):
    """x [T, heads, P], B and C [T, groups, N], dt [T, heads] (already positive),
    A [heads] (negative): S <- exp(A dt) S + dt B x^T, y = S^T C + D x."""
    T, _, P = x.shape
    N = B.shape[2]
    y = np.zeros_like(x)
    S = np.zeros((heads, N, P), dtype=F)
    for t in range(T):
        for hh in range(heads):
            g = hh // (heads // groups)
            S[hh] = math.exp(A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + D[hh] * x[t, hh]
    return y


def ssd_mixer(h: np.ndarray, w: Dict[str, np.ndarray], m: dict, eps: float) -> np.ndarray:
    T = h.shape[0]
    Hh, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = Hh * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = ssd_scan(x, B, C, dt, -np.exp(w["A_log"]), w["D"], Hh, G).reshape(T, inner)
    y = y * silu(z)
    parts = int(m["norm_groups"])
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def pair_mixer(h, w, m, eps):
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.")}
    return (float(m["left_scale"]) * sigmoid_attention(h, left, m["left"])
            + float(m["right_scale"]) * ssd_mixer(h, right, m["right"], eps))


# ------------------------------------------------------------ delta rule
DECAY_RATE = math.exp(-0.5)   # the decay's exponent lies in (-e^(-1/2), 0)
UNIT_EPS = 1e-6               # under the root of the unit key


def delta_scan(r, k, v, w, a):
    """All [T, heads, d].  u = k / sqrt(|k|^2 + 1e-6);
    S <- diag(w) S - (a * u) (u^T S) + k v^T, both terms from the old S; o = S^T r."""
    T, Hh, d = r.shape
    o = np.zeros_like(v)
    S = np.zeros((Hh, d, d), dtype=F)
    for t in range(T):
        for hh in range(Hh):
            u = k[t, hh] / math.sqrt((k[t, hh] ** 2).sum() + UNIT_EPS)
            old = S[hh]
            S[hh] = w[t, hh][:, None] * old - np.outer(a[t, hh] * u, u @ old) + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ r[t, hh]
    return o


def delta_mixer(h: np.ndarray, w: Dict[str, np.ndarray], m: dict, eps: float) -> np.ndarray:
    T = h.shape[0]
    Hh, d = int(m["heads"]), int(m["dim"])
    shape = (T, Hh, d)
    r, k, v = ((h @ w[n].T).reshape(shape) for n in ("r", "k", "v"))
    decay = np.exp(-DECAY_RATE * sigmoid(np.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(shape)
    rate = sigmoid(h @ w["a"].T + w["a.b"]).reshape(shape)
    o = delta_scan(r, k, v, decay, rate)
    o = rms_unit(o, eps).reshape(T, Hh * d) * w["norm"] * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ------------------------------------------------------------ feed-forwards
def dense_ff(h, w):
    return xielu(h @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, top, scale):
    """ids [T, top] and weights [T, top]: softmax over all experts, the `top`
    largest, their scores over their sum (+ 1e-20), times `scale`."""
    z = h @ router.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    ids = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(s, ids, axis=-1)
    return ids, chosen / (chosen.sum(axis=-1, keepdims=True) + 1e-20) * scale


def moe_ff(h, w, mlp):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    ids, wts = route(h, w["router"], top, float(mlp["router"]["scale"]))
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        for e, c in zip(ids[t], wts[t]):
            out[t] += c * gated_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out += gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    assert E == sum(1 for k in w if k.endswith(".gate") and k.startswith("e"))
    return out


# ------------------------------------------------------------------ the model
def sub(tensors: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def run_order(cfg) -> List[tuple]:
    """(layer, pass number or None, first of its pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    out = [(i, None, False) for i in range(start)]
    for t in range(times):
        out += [(i, t, i == start) for i in range(start, stop)]
    return out + [(i, None, False) for i in range(stop, n)]


def layer_forward(x, cfg, tensors, li):
    L = cfg["layers"][li]
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    pre = f"l{li}."
    mix_w = sub(tensors, pre + "mix.")
    h = rms_norm(x, tensors[pre + "norm1"], eps)
    if L["type"] == "parallel":
        y = pair_mixer(h, mix_w, L["mixer"], eps)
    elif L["type"] == "general_delta":
        y = delta_mixer(h, mix_w, L["mixer"], eps)
    else:
        raise ValueError(L["type"])
    x = x + mult * rms_norm(y, tensors[pre + "norm1b"], eps)
    if L.get("mlp") is not None:
        h = rms_norm(x, tensors[pre + "norm2"], eps)
        ff_w = sub(tensors, pre + "mlp.")
        y = dense_ff(h, ff_w) if L["mlp"]["kind"] == "dense" else moe_ff(h, ff_w, L["mlp"])
        x = x + mult * rms_norm(y, tensors[pre + "norm2b"], eps)
    return x


def forward(cfg, tensors, tokens, want=None, layers_out: Optional[list] = None) -> np.ndarray:
    """Logits [len(want) or T, vocab] of one whole sequence."""
    x0 = tensors["embed"][np.asarray(tokens)]
    x = x0.copy()
    for li, t, first in run_order(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + tensors["loop.step"][t]
        x = layer_forward(x, cfg, tensors, li)
        if layers_out is not None:
            layers_out.append(x.copy())
    x = rms_norm(x, tensors["final.norm"], float(cfg["norm"]["eps"]))
    if want is not None:
        x = x[np.asarray(want, dtype=np.int64)]
    return x @ tensors["embed"].T
