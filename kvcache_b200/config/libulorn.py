"""Configuration of the Libulorn decoder, read from its own config.json keys.

config.json of this design is nested: `layers` is a list with one object per layer (`type` names the mixer, its sizes
lie under `mixer`, the feed-forward under `mlp` or null), `embedding.bigram` gives the hashed pair table, `norm.eps`,
`vocab`, `width`.  Mixer types: `parallel` (windowed attention with grouped keys beside gated linear attention, both
reading the same rows) and `mlstm` (a matrix memory with exponential gates).  Every size and every constant that can
differ between models is read here; nothing of them stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .base import KeyReader, ModelConfig

LIBULORN_ARCHITECTURE = "Libulorn"


@dataclass(frozen=True)
class WavelengthScaling:
    """Frequencies slowed by `factor` where a turn is longer than original / low, kept where it is shorter than
    original / high, blended in between (see parts/position.py)."""
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int
    scaling: Optional[WavelengthScaling] = None


@dataclass(frozen=True)
class WindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                         # numbers of a head's query and key
    vdim: int                        # numbers of a head's value
    scale: float
    window: Optional[int]            # keys a query sees, its own included; None: all
    rot: Optional[RotarySpec]


@dataclass(frozen=True)
class GatedLinearSpec:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None   # inner size of the decay's two matrices; None: the checkpoint's shapes decide


@dataclass(frozen=True)
class ParallelSpec:
    left: WindowAttentionSpec
    right: GatedLinearSpec
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class MatrixMemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ExpertSpec:
    ff: int
    limit: float


@dataclass(frozen=True)
class RoutedSpec:
    expert: ExpertSpec
    experts: int
    top: int
    shared: Optional[ExpertSpec]


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: Union[ParallelSpec, MatrixMemorySpec, None]
    mlp: Optional[RoutedSpec]


@dataclass(frozen=True)
class BigramSpec:
    buckets: int
    mul_prev: int
    mul_cur: int


def _read_rot(m: KeyReader) -> Optional[RotarySpec]:
    rot = m.sub("rot", required=False)
    if rot is None:
        return None
    base, dims = rot.number("base", positive=True), rot.integer("dims", minimum=2)
    scaling = None
    s = rot.sub("scaling", required=False)
    if s is not None:
        scaling = WavelengthScaling(s.number("factor", positive=True), s.number("low", positive=True),
                                    s.number("high", positive=True), s.number("original", positive=True))
        if None not in (scaling.low, scaling.high) and scaling.low == scaling.high:
            s.fail("'low' and 'high' must differ")
        rot.absorb(s)
    if dims is not None and dims % 2:
        rot.fail(f"'dims' must be even, got {dims}")
    m.absorb(rot)
    return RotarySpec(base, dims, scaling)


def _read_window_attention(parent: KeyReader, key: str) -> Optional[WindowAttentionSpec]:
    m = parent.sub(key)
    if m is None:
        return None
    mask = m.sub("mask", required=False)
    window = mask.integer("size", minimum=1) if mask is not None else None
    m.absorb(mask)
    spec = WindowAttentionSpec(heads=m.integer("heads", minimum=1), kv_heads=m.integer("kv_heads", minimum=1),
                               dim=m.integer("dim", minimum=1), vdim=m.integer("vdim", minimum=1),
                               scale=m.number("scale", positive=True), window=window, rot=_read_rot(m))
    if None not in (spec.heads, spec.kv_heads) and spec.heads % spec.kv_heads:
        m.fail(f"heads {spec.heads} is not a multiple of kv_heads {spec.kv_heads}")
    if spec.rot is not None and None not in (spec.rot.dims, spec.dim) and spec.rot.dims > spec.dim:
        m.fail(f"rot.dims {spec.rot.dims} exceeds dim {spec.dim}")
    parent.absorb(m)
    return spec


def _read_gated_linear(parent: KeyReader, key: str) -> Optional[GatedLinearSpec]:
    m = parent.sub(key)
    if m is None:
        return None
    spec = GatedLinearSpec(m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("vdim", minimum=1),
                           m.number("tau", positive=True), m.integer("decay_rank", default=None, minimum=1))
    parent.absorb(m)
    return spec


def _read_mixer(lr: KeyReader, kind: Optional[str]):
    m = lr.sub("mixer")
    if m is None or kind is None:
        return None
    spec = None
    if kind == "parallel":
        spec = ParallelSpec(_read_window_attention(m, "left"), _read_gated_linear(m, "right"),
                            m.number("left_scale"), m.number("right_scale"))
    elif kind == "mlstm":
        spec = MatrixMemorySpec(m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("vdim", minimum=1),
                                m.number("gate_cap", positive=True))
    lr.absorb(m)
    return spec


def _read_expert(parent: KeyReader, key: str, required: bool) -> Optional[ExpertSpec]:
    e = parent.sub(key, required=required)
    if e is None:
        return None
    spec = ExpertSpec(e.integer("ff", minimum=1), e.number("limit", positive=True))
    parent.absorb(e)
    return spec


def _read_mlp(lr: KeyReader) -> Optional[RoutedSpec]:
    m = lr.sub("mlp", required=False)
    if m is None:
        return None
    kind = m.string("kind")
    spec = None
    if kind == "moe":
        router = m.sub("router")
        experts = router.integer("experts", minimum=1) if router is not None else None
        top = router.integer("top", minimum=1) if router is not None else None
        if None not in (experts, top) and top > experts:
            m.fail(f"router.top {top} exceeds router.experts {experts}")
        m.absorb(router)
        spec = RoutedSpec(_read_expert(m, "expert", True), experts or 0, top or 0, _read_expert(m, "shared", False))
    elif kind is not None:
        m.fail(f"unknown feed-forward kind '{kind}' (moe)")
    lr.absorb(m)
    return spec


@dataclass(frozen=True)
class LibulornConfig(ModelConfig):
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    bigram: Optional[BigramSpec]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "LibulornConfig":
        r = KeyReader(data, where)
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = r.sub("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        r.absorb(norm)
        bigram = None
        emb = r.sub("embedding", required=False)
        if emb is not None:
            b = emb.sub("bigram", required=False)
            if b is not None:
                bigram = BigramSpec(b.integer("buckets", minimum=1), b.integer("mul_prev", minimum=0), b.integer("mul_cur", minimum=0))
                emb.absorb(b)
            r.absorb(emb)
        raw_layers = data.get("layers")
        layers = []
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            r.fail("'layers' must be a non-empty list")
        else:
            for i, item in enumerate(raw_layers):
                if not isinstance(item, Mapping):
                    r.fail(f"layers[{i}] must be an object")
                    continue
                lr = KeyReader(item, f"{where}: layers[{i}]")
                kind = lr.string("type")
                if kind is not None and kind not in ("parallel", "mlstm"):
                    lr.fail(f"unknown mixer type '{kind}' (parallel, mlstm)")
                    kind = None
                layers.append(LayerSpec(kind, _read_mixer(lr, kind), _read_mlp(lr)))
                r.absorb(lr)
        eos = r.int_list("eos_token_id", default=())
        init_range = r.number("initializer_range", default=0.05, positive=True)
        r.finish()
        return cls(architecture=LIBULORN_ARCHITECTURE, vocab_size=vocab, width=width, norm_eps=eps, layers=tuple(layers),
                   bigram=bigram, eos_token_ids=eos, initializer_range=init_range)

    def to_dict(self) -> Dict[str, Any]:
        def rot(s: Optional[RotarySpec]):
            if s is None:
                return None
            out: Dict[str, Any] = {"base": s.base, "dims": s.dims}
            if s.scaling is not None:
                out["scaling"] = {"factor": s.scaling.factor, "low": s.scaling.low, "high": s.scaling.high,
                                  "original": s.scaling.original}
            return out

        def mixer(s):
            if isinstance(s, MatrixMemorySpec):
                return {"heads": s.heads, "dim": s.dim, "vdim": s.vdim, "gate_cap": s.gate_cap}
            left: Dict[str, Any] = {"heads": s.left.heads, "kv_heads": s.left.kv_heads, "dim": s.left.dim, "vdim": s.left.vdim,
                                    "scale": s.left.scale}
            if s.left.window is not None:
                left["mask"] = {"size": s.left.window}
            if s.left.rot is not None:
                left["rot"] = rot(s.left.rot)
            return {"left": left, "left_scale": s.left_scale, "right_scale": s.right_scale,
                    "right": {"heads": s.right.heads, "dim": s.right.dim, "vdim": s.right.vdim, "tau": s.right.tau,
                              **({} if s.right.decay_rank is None else {"decay_rank": s.right.decay_rank})}}

        def mlp(s: Optional[RoutedSpec]):
            if s is None:
                return None
            out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": s.expert.ff, "limit": s.expert.limit},
                                   "router": {"experts": s.experts, "top": s.top}}
            if s.shared is not None:
                out["shared"] = {"ff": s.shared.ff, "limit": s.shared.limit}
            return out

        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer), "mlp": mlp(l.mlp)} for l in self.layers],
            "initializer_range": self.initializer_range,
        }
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                           "mul_cur": self.bigram.mul_cur}}
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif len(self.eos_token_ids) > 1:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
