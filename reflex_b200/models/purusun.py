"""Purusun as data: its typed config turned into a `ModelSpec`.

The design: a token embedding; the residual as `streams` parallel copies of the
embedding output (hyper-connections: a sublayer reads a weighted sum of the
copies, and its result, times a per-channel scale, goes back into every copy
while the copies are mixed by a small matrix; without `streams` the ordinary
residual sum with the per-channel scale); pre-norm layers whose RMS norms keep
their weights around zero (1 + w); the mixer is an attention (grouped heads
whose values are the keys as projected, per-head RMS norm of q and k with a
plain weight, a rotation of the first few dimensions of a head with
wavelength-dependent frequency scaling, a sliding window that also keeps the
sequence's first tokens, a sigmoid gate on the concatenated heads before the
output projection) or a selective scan (a short causal convolution with silu,
input-dependent step sizes through a low-rank projection, a diagonal state per
channel, a silu gate); the feed-forward is W_down relu(W_up h)^2; a stretch of
layers may run several times with the same weights, each pass with cache
entries of its own; the model's norm, and the embedding table as the head.
Tensor names are the checkpoint's; the right columns of `*_NAMES` are the only
place they occur.
"""

from __future__ import annotations

from ..config.purusun import PurusunConfig
from ..config.registry import register_architecture
from ..config.spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, RunEntry

ATTENTION_NAMES = (("q_proj", "mix.q"), ("k_proj", "mix.k"), ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm"),
                   ("g_proj", "mix.g"), ("o_proj", "mix.o"))
SCAN_NAMES = (("in_proj", "mix.in"), ("conv", "mix.conv"), ("conv_bias", "mix.conv.b"), ("x_proj", "mix.x"),
              ("dt_proj", "mix.dt"), ("dt_bias", "mix.dt.b"), ("A_log", "mix.A_log"), ("D", "mix.D"),
              ("o_proj", "mix.o"))
DENSE_NAMES = (("up_proj", "mlp.up"), ("down_proj", "mlp.down"))
BLOCK_NAMES = (("mixer_norm", "norm1"), ("feed_forward_norm", "norm2"), ("mixer_scale", "ls1"),
               ("feed_forward_scale", "ls2"), ("mixer_read", "hc1.in"), ("mixer_write", "hc1.out"),
               ("mixer_mix", "hc1.mix"), ("feed_forward_read", "hc2.in"), ("feed_forward_write", "hc2.out"),
               ("feed_forward_mix", "hc2.mix"))

# fixed by the design: the layers' and the model's norms apply 1 + w
NORM_WEIGHT_OFFSET = 1.0


def build_purusun_spec(cfg: PurusunConfig) -> ModelSpec:
    eps, W = cfg.norm_eps, cfg.width
    streams = cfg.streams or 1
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.type == "attention":
            d = int(m["dim"])
            rot, position = m.get("rot"), None
            if rot is not None and int(rot["dims"]) > 0:
                sc = rot.get("scaling")
                position = PositionSpec(
                    "rope_scaled" if sc else "rope_neox", head_dim=d, rotary_dim=int(rot["dims"]),
                    theta=float(rot["base"]),
                    params=tuple((k, float(sc[k])) for k in ("factor", "low", "high", "original")) if sc else ())
            mask = m.get("mask") or {}
            mixer = MixerSpec(
                "gqa_attention", hidden_size=W, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                head_dim=d, scale=float(m["scale"]), window=int(mask["size"]) if mask.get("size") else None,
                qk_norm=NormSpec("rmsnorm", d, eps), position=position, names=ATTENTION_NAMES,
                params=(("values_are_keys", True), ("output_gate", True),
                        ("keep_first", int(mask.get("keep_first") or 0))))
        else:
            mixer = MixerSpec(
                "selective_scan", hidden_size=W, names=SCAN_NAMES,
                params=(("inner", int(m["inner"])), ("state", int(m["state"])), ("dt_rank", int(m["dt_rank"])),
                        ("taps", int(m["conv"]))))
        ffn = None
        if l.mlp is not None:
            ffn = FeedForwardSpec("relu2", hidden_size=W, intermediate_size=int(l.mlp["ff"]), names=DENSE_NAMES)
        layers.append(LayerSpec(
            block="hyper_prenorm", prefix=f"l{i}.", mixer=mixer, feed_forward=ffn,
            mixer_norm=NormSpec("rmsnorm", W, eps, NORM_WEIGHT_OFFSET),
            feed_forward_norm=NormSpec("rmsnorm", W, eps, NORM_WEIGHT_OFFSET) if ffn is not None else None,
            names=BLOCK_NAMES,
            params=(("streams", streams), ("connections", cfg.streams is not None), ("layer_scale", True))))
    # the order of the runs: a looped stretch names its layers once per pass, every run
    # with a cache entry of its own
    n = len(layers)
    if cfg.loop is None:
        runs = list(range(n))
    else:
        start, stop, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
        runs = list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))
    order = [RunEntry(layer, entry, True) for entry, layer in enumerate(runs)]
    return ModelSpec(
        architecture="purusun", vocab_size=cfg.vocab, hidden_size=W, layers=layers,
        final_norm=NormSpec("rmsnorm", W, eps, NORM_WEIGHT_OFFSET), tie_word_embeddings=True,
        max_positions=cfg.max_positions, embedding_name="embed", final_norm_name="final.norm",
        head_name="head", run_order=order, residual_streams=streams)


PURUSUN = register_architecture(("Purusun", "purusun"), PurusunConfig.from_dict, build_purusun_spec)
