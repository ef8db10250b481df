"""The Kakipel decoder put together from parts, layer by layer, from its configuration.

Tensor names: `embed`, `head`, `final.norm`, `loop.in`, `loop.step`, and per layer i `l<i>.norm1`, `l<i>.norm1b`,
`l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*` (the mixer), `l<i>.mlp.*` (the feed-forward).  A layer is a norm before and
after each sublayer; the layers of `loop` run `times` times in a row with the same weights, each pass with a cache
entry of its own per layer and a `LoopEntry` before its first layer.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.kakipel import KAKIPEL_ARCHITECTURE, KakipelConfig, RotarySpec
from ..config.registry import register_architecture
from ..parts.block import SandwichBlock
from ..parts.feedforward import GatedMLP, RoutedMLP
from ..parts.latent_attention import LatentAttention
from ..parts.model import DecoderModel, LayerCall
from ..parts.norm import RMSNorm
from ..parts.position import RampScaling, RotaryHalf
from ..parts.stream import LoopEntry

# Until the engine tells how long a request may get (it always does), rotation tables are made for this many positions.
DEFAULT_POSITIONS = 4096


def build_kakipel(config: KakipelConfig, dtype: str = "bfloat16", device: str = "cuda:0",
                  max_positions: Optional[int] = None) -> DecoderModel:
    c = config
    positions = max_positions or DEFAULT_POSITIONS
    rotations: Dict[tuple, RotaryHalf] = {}          # layers with equal rotation constants share one table

    def rotation(spec: RotarySpec) -> RotaryHalf:
        s = spec.scaling
        key = (spec.dims, spec.base, None if s is None else (s.factor, s.original, s.fast, s.slow))
        if key not in rotations:
            scaling = None if s is None else RampScaling(s.factor, s.original, s.fast, s.slow)
            rotations[key] = RotaryHalf(spec.dims, spec.base, positions, scaling)
        return rotations[key]

    blocks = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = LatentAttention(c.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, scale=m.scale, eps=c.norm_eps,
                                position=rotation(m.rot), prefix=p + "mix.", dtype=dtype)
        ffn = pre2 = post2 = None
        if layer.mlp is not None:
            pre2, post2 = RMSNorm(c.width, c.norm_eps, p + "norm2"), RMSNorm(c.width, c.norm_eps, p + "norm2b")
            if layer.mlp.kind == "dense":
                ffn = GatedMLP(c.width, layer.mlp.ff, activation="silu", prefix=p + "mlp.", dtype=dtype, names=("gate", "up", "down"))
            else:
                ffn = RoutedMLP(c.width, layer.mlp.ff, layer.mlp.experts, layer.mlp.top, activation="relu2", prefix=p + "mlp.",
                                dtype=dtype)
        blocks.append(SandwichBlock(c.width, RMSNorm(c.width, c.norm_eps, p + "norm1"), mixer,
                                    RMSNorm(c.width, c.norm_eps, p + "norm1b"), pre2, ffn, post2, dtype))
    # A checkpoint may carry the norms of a feed-forward that a layer does not have, or the loop's tensors without a loop:
    # they are left alone (with a line on standard error), not an error.
    unused = [f"l{i}.{name}" for i, layer in enumerate(c.layers) if layer.mlp is None for name in ("norm2", "norm2b")]
    if c.loop is None:
        unused += ["loop.in", "loop.step"]
    stream_parts = [LoopEntry(c.width, c.loop.times, "loop.in", "loop.step", dtype)] if c.loop is not None else []
    # Every layer run has a cache entry of its own: a looped layer's passes see different keys.
    schedule = [LayerCall(layer, run, True, (0, t) if opens else None) for run, (layer, t, opens) in enumerate(c.layer_runs())]
    return DecoderModel(config=c, dtype=dtype, vocab_size=c.vocab_size, width=c.width, embed_name="embed", head_name="head",
                        blocks=blocks, schedule=schedule, final_norm=RMSNorm(c.width, c.norm_eps, "final.norm"),
                        position=None, stream_parts=stream_parts, ignorable_tensors=unused)


register_architecture(KAKIPEL_ARCHITECTURE, KakipelConfig, build_kakipel, replace=True)
