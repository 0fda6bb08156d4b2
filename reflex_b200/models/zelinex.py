"""Zelinex as data: its typed config turned into a `ModelSpec`.

The design: a token embedding; layers with an RMS norm before and after each
sublayer, x <- x + m * post(sublayer(pre(x))) with m one number of the model;
the mixer is either two mixers side by side, summed with a weight each (an
attention whose weights are sigmoids of the biased scores, not normalised over
the keys, with grouped heads, values of another size than keys, a half-split
rotation of a head's first dimensions and a sliding window; beside it a
state-space recurrence with one decay a head, a short convolution over x, B
and C, a silu gate and a norm in equal parts) or a generalized delta rule (a
matrix memory per head with a decay and a removal rate per key channel, a
per-head norm and a sigmoid gate); the feed-forward is W_down xielu(W_up h)
with two stored numbers a layer, or a mixture of gated silu experts (softmax
over all experts, the chosen scores renormalised and scaled) beside a shared
expert; a stretch of layers may run several times with the same weights, each
pass with cache entries of its own and starting from x + x0 (not the first
pass) + a vector of the pass; the model's norm, and the embedding table as the
head.  Tensor names are the checkpoint's; the right columns of `*_NAMES` are
the only place they occur.
"""

from __future__ import annotations

import math

from ..config.registry import register_architecture
from ..config.spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, RunEntry
from ..config.zelinex import ZelinexConfig

LEFT_NAMES = (("q_proj", "q"), ("k_proj", "k"), ("v_proj", "v"), ("score_bias", "pb"), ("o_proj", "o"))
RIGHT_NAMES = (("in_proj", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"),
               ("A_log", "A_log"), ("D", "D"), ("norm", "norm"), ("o_proj", "o"))
PAIR_NAMES = (tuple((f"left/{r}", f"mix.left.{n}") for r, n in LEFT_NAMES)
              + tuple((f"right/{r}", f"mix.right.{n}") for r, n in RIGHT_NAMES))
DELTA_NAMES = (("r_proj", "mix.r"), ("k_proj", "mix.k"), ("v_proj", "mix.v"), ("g_proj", "mix.g"),
               ("a_proj", "mix.a"), ("a_bias", "mix.a.b"), ("w1_proj", "mix.w1"), ("w2_proj", "mix.w2"),
               ("w0", "mix.w0"), ("norm", "mix.norm"), ("o_proj", "mix.o"))
DENSE_NAMES = (("up_proj", "mlp.up"), ("down_proj", "mlp.down"), ("act", "mlp.act"))
MOE_NAMES = (("router", "mlp.router"), ("expert_gate", "mlp.e{expert}.gate"), ("expert_up", "mlp.e{expert}.up"),
             ("expert_down", "mlp.e{expert}.down"), ("shared_gate", "mlp.shared.gate"),
             ("shared_up", "mlp.shared.up"), ("shared_down", "mlp.shared.down"))
BLOCK_NAMES = (("mixer_norm", "norm1"), ("feed_forward_norm", "norm2"), ("post_mixer", "norm1b"),
               ("post_feed_forward", "norm2b"))

# fixed by the design
DECAY_RATE = math.exp(-0.5)   # the delta rule's decay is exp(-e^(-1/2) sigmoid(.))
UNIT_KEY_EPS = 1e-6           # under the root of the delta rule's unit key
XIELU_BETA = 0.5              # the negative branch's coefficient is 1/2 + softplus(q)


def build_zelinex_spec(cfg: ZelinexConfig) -> ModelSpec:
    eps, W = cfg.norm_eps, cfg.width
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.type == "parallel":
            a, r = m["left"], m["right"]
            d = int(a["dim"])
            rot, position = a.get("rot"), None
            if rot is not None and int(rot["dims"]) > 0:
                position = PositionSpec("rope_neox", head_dim=d, rotary_dim=int(rot["dims"]), theta=float(rot["base"]))
            mask = a.get("mask") or {}
            left = MixerSpec(
                "sigmoid_attention", hidden_size=W, num_heads=int(a["heads"]), num_kv_heads=int(a["kv_heads"]),
                head_dim=d, v_head_dim=int(a["vdim"]), scale=float(a["scale"]),
                window=int(mask["size"]) if mask.get("size") else None, position=position)
            right = MixerSpec(
                "ssd", hidden_size=W,
                params=(("heads", int(r["heads"])), ("vdim", int(r["vdim"])), ("state", int(r["state"])),
                        ("groups", int(r["groups"])), ("taps", int(r["conv"])),
                        ("norm_groups", int(r["norm_groups"])), ("eps", eps)))
            mixer = MixerSpec("pair", hidden_size=W, names=PAIR_NAMES,
                              params=(("left", left), ("right", right), ("combine", "scaled_sum"),
                                      ("left_scale", float(m["left_scale"])), ("right_scale", float(m["right_scale"]))))
        else:
            mixer = MixerSpec(
                "delta_rule", hidden_size=W, num_heads=int(m["heads"]), head_dim=int(m["dim"]), names=DELTA_NAMES,
                params=(("rate", DECAY_RATE), ("unit_eps", UNIT_KEY_EPS), ("eps", eps)))
        ffn = None
        if l.mlp is not None and l.mlp["kind"] == "dense":
            ffn = FeedForwardSpec("xielu", hidden_size=W, intermediate_size=int(l.mlp["ff"]), names=DENSE_NAMES,
                                  params=(("beta", XIELU_BETA),))
        elif l.mlp is not None:
            shared = l.mlp.get("shared")
            ffn = FeedForwardSpec(
                "moe", hidden_size=W, intermediate_size=int(l.mlp["expert"]["ff"]), names=MOE_NAMES,
                params=(("experts", int(l.mlp["router"]["experts"])), ("top", int(l.mlp["router"]["top"])),
                        ("activation", "swiglu"), ("scores", "softmax_all"),
                        ("score_scale", float(l.mlp["router"].get("scale", 1.0))), ("router_bias", False),
                        ("shared_ff", int(shared["ff"]) if shared else 0), ("shared_kind", "swiglu")))
        norm = NormSpec("rmsnorm", W, eps)
        layers.append(LayerSpec(
            block="sandwich", prefix=f"l{i}.", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
            feed_forward_norm=norm if ffn is not None else None, names=BLOCK_NAMES,
            extra_norms=(("post_mixer", norm),) + ((("post_feed_forward", norm),) if ffn is not None else ()),
            params=(("residual_mult", cfg.residual_mult),)))
    # the order of the runs: a looped stretch names its layers once per pass, every run with a
    # cache entry of its own; a pass starts from x (+ x0 from the second pass on) + its vector
    n = len(layers)
    if cfg.loop is None:
        runs = [(i, None) for i in range(n)]
        times = 0
    else:
        start, stop, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
        runs = [(i, None) for i in range(start)]
        for t in range(times):
            runs += [(i, t if i == start else None) for i in range(start, stop)]
        runs += [(i, None) for i in range(stop, n)]
    order = [RunEntry(layer, entry, True, pass_vector=t, adds_input=bool(t)) for entry, (layer, t) in enumerate(runs)]
    return ModelSpec(
        architecture="zelinex", vocab_size=cfg.vocab, hidden_size=W, layers=layers,
        final_norm=NormSpec("rmsnorm", W, eps), tie_word_embeddings=True, max_positions=cfg.max_positions,
        embedding_name="embed", final_norm_name="final.norm", head_name="head", run_order=order,
        pass_vectors_name="loop.step" if cfg.loop is not None else None, pass_vectors=times)


ZELINEX = register_architecture(("Zelinex", "zelinex"), ZelinexConfig.from_dict, build_zelinex_spec)
