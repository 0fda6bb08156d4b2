"""A plain, slow implementation of the Purusun design, for tests.

Whole sequences, no cache, one function per mechanism, NumPy in double
precision; it shares no code with `reflex_b200`.  Linear weights are [out, in]
and applied as y = x W^T.

The design: a token embedding; the residual is `streams` copies of the
embedding output (hyper-connections): a sublayer reads a weighted sum of the
copies and its result goes back to every copy with a weight of its own while
the copies are mixed among themselves by a small matrix; pre-norm layers with
RMS norms whose weight is stored around zero (1 + w), a per-channel scale on
every sublayer's result; the mixer is an attention (grouped heads whose values
are the keys as projected, per-head RMS norm of q and k, a rotation of the
first few dimensions with frequency-scaled angles, a sliding window that also
keeps the first few tokens, a sigmoid gate on the heads' outputs) or a
selective scan (a short causal convolution, input-dependent step sizes, a
diagonal state per channel); the feed-forward is W_down relu(W_up h)^2; a
stretch of layers may run several times with the same weights; the model's
norm and the embedding table as the head.
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


def norm_one_plus(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """The layers' and the model's norm: the weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


# ------------------------------------------------------------------ rotation
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]) -> np.ndarray:
    """f_i = base^(-2i/dims), i < dims/2, then the wavelength-dependent scaling:
    short waves kept, long waves slowed by `factor`, a linear blend between."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < orig / high:
            out[i] = fi
        elif wave > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(t: np.ndarray, positions: np.ndarray, freqs: np.ndarray) -> np.ndarray:
    """t [T, heads, dim]: dimension i pairs with i + len(freqs) among the first
    2 len(freqs) dimensions; the rest pass."""
    half = len(freqs)
    if half == 0:
        return t
    ang = positions[:, None].astype(F) * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = t.copy()
    u, v = t[..., :half], t[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


# ----------------------------------------------------------------- attention
def visible(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    return j <= i and (size is None or i - j < size or j < keep_first)


def attention(h: np.ndarray, w: Dict[str, np.ndarray], m: dict, eps: float, positions=None) -> np.ndarray:
    """h [T, width] -> [T, width].  `w`: q, k, q.norm, k.norm, g, o."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    pos = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = k.copy()  # the values are the keys as projected
    q = rms_unit(q, eps) * w["q.norm"]
    k = rms_unit(k, eps) * w["k.norm"]
    rot = m.get("rot")
    if rot:
        f = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q, k = rotate(q, pos, f), rotate(k, pos, f)
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first", 0) or 0)
    out = np.zeros((T, H, d), dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            js = [j for j in range(T) if visible(int(pos[i]), int(pos[j]), size, keep)]
            s = (k[js, g] @ q[i, head]) * float(m["scale"])
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, head] = p @ v[js, g]
    gate = sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * d) * gate) @ w["o"].T


# ------------------------------------------------------------ selective scan
def causal_conv(x: np.ndarray, taps: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """x [T, C], taps [C, K] (the last column on the current token), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C), dtype=F), x], axis=0)
    out = np.tile(bias, (T, 1)).astype(F)
    for j in range(K):
        out += padded[j:j + T] * taps[:, j]
    return out


def selective_scan(h: np.ndarray, w: Dict[str, np.ndarray], m: dict) -> np.ndarray:
    """h [T, width] -> [T, width].  `w`: in, conv, conv.b, x, dt, dt.b, A_log, D, o."""
    T = h.shape[0]
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = h @ w["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w["conv"], w["conv.b"]))
    p = x @ w["x"].T
    dt, B, C = p[:, :R], p[:, R:R + N], p[:, R + N:R + 2 * N]
    dt = softplus(dt @ w["dt"].T + w["dt.b"])          # [T, inner]
    y = scan_core(x, dt, -np.exp(w["A_log"]), B, C, w["D"])
    return (y * silu(z)) @ w["o"].T


def scan_core(x, dt, A, B, C, D, S0=None):
    """x, dt [T, inner]; A [inner, N]; B, C [T, N]; D [inner]: the recurrence
    S <- exp(dt A) S + dt x B, y = S C + D x, from the state S0 (zeros)."""
    T, inner = x.shape
    S = np.zeros(A.shape, dtype=F) if S0 is None else S0.copy()
    y = np.zeros((T, inner), dtype=F)
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


# -------------------------------------------------------------- feed-forward
def relu2_ff(h: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


# --------------------------------------------------------- hyper-connections
def hyper_read(xs: np.ndarray, w_in: np.ndarray) -> np.ndarray:
    """xs [streams, T, width] -> the sublayer's input, sum_s in[s] x_s."""
    return np.tensordot(w_in, xs, axes=(0, 0))


def hyper_write(xs: np.ndarray, y: np.ndarray, mix: np.ndarray, w_out: np.ndarray) -> np.ndarray:
    """x_t <- sum_s mix[s, t] x_s + out[t] y, all copies at once from the old ones."""
    return np.tensordot(mix.T, xs, axes=(1, 0)) + w_out[:, None, None] * y[None]


# --------------------------------------------------------------------- model
def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sub(w: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, want_layers: bool = False):
    """Logits [T, vocab] of one whole sequence; with `want_layers` also the sum of
    the residual copies after every layer run, [runs, T, width]."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)]
    streams = cfg.get("streams")
    xs = np.stack([x] * int(streams)) if streams else x[None]
    after = []
    for li in run_order(cfg):
        layer = cfg["layers"][li]
        p = f"l{li}."
        for q, kind in ((1, "mixer"), (2, "mlp")):
            if kind == "mlp" and layer.get("mlp") is None:
                continue
            if streams:
                u = hyper_read(xs, w[f"{p}hc{q}.in"])
            else:
                u = xs[0]
            n = norm_one_plus(u, w[f"{p}norm{q}"], eps)
            if kind == "mixer":
                if layer["type"] == "attention":
                    y = attention(n, sub(w, p + "mix."), layer["mixer"], eps)
                elif layer["type"] == "mamba1":
                    y = selective_scan(n, sub(w, p + "mix."), layer["mixer"])
                else:
                    raise ValueError(layer["type"])
            else:
                if layer["mlp"]["kind"] != "dense":
                    raise ValueError(layer["mlp"]["kind"])
                y = relu2_ff(n, w[p + "mlp.up"], w[p + "mlp.down"])
            if f"{p}ls{q}" in w:
                y = y * w[f"{p}ls{q}"]
            if streams:
                xs = hyper_write(xs, y, w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"])
            else:
                xs = xs + y[None]
        after.append(xs.sum(axis=0))
    x = xs.sum(axis=0)
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["embed"].T
    if want_layers:
        return logits, np.stack(after)
    return logits


def argmax_last(logits: np.ndarray) -> int:
    """Ties go to the highest index, as the library's argmax does."""
    v = np.asarray(logits)
    return int(len(v) - 1 - np.argmax(v[::-1]))
