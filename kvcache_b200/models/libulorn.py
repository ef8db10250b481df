"""The Libulorn decoder put together from parts, layer by layer, from its configuration.

Tensor names: `embed`, `bigram`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*` (the
mixer; the two sides of a parallel mixer under `left.` and `right.`), `l<i>.mlp.*` (router, experts `e<j>.`, `shared.`).
A layer normalises what its sublayers return, not what they read: x += norm1(mixer(x)); x += norm2(ff(x)).  The
embedding adds a row of a hashed table of token pairs.  Layer kinds: `parallel` - attention over a window of keys
(grouped heads, queries and keys normalised per head, part of each head rotated, a gate per head) beside gated linear
attention, summed with two scales; `mlstm` - a matrix memory with exponential gates.  Feed-forwards are mixtures of
clamped gated experts with a shared expert.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.libulorn import LIBULORN_ARCHITECTURE, LibulornConfig, MatrixMemorySpec, ParallelSpec, RotarySpec
from ..config.registry import register_architecture
from ..parts.attention import GQAAttention
from ..parts.block import SandwichBlock
from ..parts.embedding import HashedBigramEmbedding
from ..parts.feedforward import GatedMLP, RoutedMLP
from ..parts.model import DecoderModel, LayerCall
from ..parts.norm import PassNorm, RMSNorm
from ..parts.position import RotaryHalf, WavelengthScaling
from ..parts.recurrent import GatedLinearAttention, MatrixMemory, ParallelMixer

# Until the engine tells how long a request may get (it always does), rotation tables are made for this many positions.
DEFAULT_POSITIONS = 4096


def build_libulorn(config: LibulornConfig, dtype: str = "bfloat16", device: str = "cuda:0",
                   max_positions: Optional[int] = None) -> DecoderModel:
    c = config
    positions = max_positions or DEFAULT_POSITIONS
    rotations: Dict[tuple, RotaryHalf] = {}          # layers with equal rotation constants share one table

    def rotation(spec: Optional[RotarySpec]) -> Optional[RotaryHalf]:
        if spec is None:
            return None
        s = spec.scaling
        key = (spec.dims, spec.base, None if s is None else (s.factor, s.low, s.high, s.original))
        if key not in rotations:
            scaling = None if s is None else WavelengthScaling(s.factor, s.low, s.high, s.original)
            rotations[key] = RotaryHalf(spec.dims, spec.base, positions, scaling)
        return rotations[key]

    def mixer(spec, p: str):
        if isinstance(spec, MatrixMemorySpec):
            return MatrixMemory(c.width, spec.heads, spec.dim, spec.vdim, spec.gate_cap, eps=c.norm_eps, prefix=p, dtype=dtype)
        assert isinstance(spec, ParallelSpec)
        a, g = spec.left, spec.right
        left = GQAAttention(c.width, a.heads, a.kv_heads, a.dim, qkv_bias=False, out_bias=False, position=rotation(a.rot),
                            window=a.window, prefix=p + "left.", dtype=dtype, scale=a.scale, value_dim=a.vdim,
                            qk_norm_eps=c.norm_eps, head_gate="g", names=("q", "k", "v", "o"))
        right = GatedLinearAttention(c.width, g.heads, g.dim, g.vdim, g.decay_rank, g.tau, eps=c.norm_eps, prefix=p + "right.",
                                     dtype=dtype)
        return ParallelMixer(c.width, left, right, spec.left_scale, spec.right_scale, dtype)

    blocks = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = pre2 = post2 = None
        if layer.mlp is not None:
            m = layer.mlp
            shared = None
            if m.shared is not None:
                shared = GatedMLP(c.width, m.shared.ff, activation="clamped_swiglu", limit=m.shared.limit, prefix=p + "mlp.shared.",
                                  dtype=dtype, names=("gate", "up", "down"))
            ffn = RoutedMLP(c.width, m.expert.ff, m.experts, m.top, activation="clamped_swiglu", limit=m.expert.limit, scores="all",
                            prefix=p + "mlp.", dtype=dtype, shared=shared)
            pre2, post2 = PassNorm(), RMSNorm(c.width, c.norm_eps, p + "norm2")
        blocks.append(SandwichBlock(c.width, PassNorm(), mixer(layer.mixer, p + "mix."), RMSNorm(c.width, c.norm_eps, p + "norm1"),
                                    pre2, ffn, post2, dtype))
    # A checkpoint may carry the second norm of a layer that has no feed-forward: it is left alone.
    unused = [f"l{i}.norm2" for i, layer in enumerate(c.layers) if layer.mlp is None]
    embedding_parts = []
    if c.bigram is not None:
        embedding_parts.append(HashedBigramEmbedding(c.width, c.bigram.buckets, c.bigram.mul_prev, c.bigram.mul_cur, c.vocab_size,
                                                     "bigram", dtype))
    return DecoderModel(config=c, dtype=dtype, vocab_size=c.vocab_size, width=c.width, embed_name="embed", head_name="head",
                        blocks=blocks, schedule=[LayerCall(i, i) for i in range(len(c.layers))],
                        final_norm=RMSNorm(c.width, c.norm_eps, "final.norm"), position=None,
                        embedding_parts=embedding_parts, ignorable_tensors=unused)


register_architecture(LIBULORN_ARCHITECTURE, LibulornConfig, build_libulorn, replace=True)
