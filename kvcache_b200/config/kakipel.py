"""Configuration of the Kakipel decoder, read from its own config.json keys.

config.json of this design is nested: `layers` is a list with one object per layer
(`type`, the mixer's sizes under `mixer`, the feed-forward under `mlp` or null), `loop`
names a run of layers that is passed several times, `norm.eps`, `vocab`, `width`.  Every
size and every constant that can differ between models is read here; nothing of them
stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig

KAKIPEL_ARCHITECTURE = "Kakipel"


@dataclass(frozen=True)
class RotaryScaling:
    """Frequencies blended between f and f / factor by a ramp over the dimension pairs (see parts/position.py)."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int
    scaling: Optional[RotaryScaling] = None


@dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int            # unrotated query/key dimensions of a head
    rot_dim: int        # rotated ones (one rotated key part is shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotarySpec


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                    # "dense" or "moe"
    ff: int                      # hidden size (of one expert for "moe")
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[FeedForwardSpec]


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


def _sub(r: KeyReader, key: str, required: bool = True) -> Optional[KeyReader]:
    value = r.data.get(key)
    if value is None:
        if required:
            r.fail(f"missing key '{key}'")
        return None
    if not isinstance(value, Mapping):
        r.fail(f"'{key}' must be an object")
        return None
    return KeyReader(value, f"{r.where}: {key}")


def _absorb(parent: KeyReader, child: Optional[KeyReader]) -> None:
    if child is not None:
        parent.problems.extend(f"{child.where.split(': ', 1)[-1]}: {p}" for p in child.problems)
        child.problems.clear()


def _read_rot(r: KeyReader) -> Optional[RotarySpec]:
    rot = _sub(r, "rot")
    if rot is None:
        return None
    base, dims = rot.number("base", positive=True), rot.integer("dims", minimum=2)
    scaling = None
    s = _sub(rot, "scaling", required=False)
    if s is not None:
        scaling = RotaryScaling(s.number("factor", positive=True), s.number("original", positive=True),
                                s.number("fast", positive=True), s.number("slow", positive=True))
        _absorb(rot, s)
    if dims is not None and dims % 2:
        rot.fail(f"'dims' must be even, got {dims}")
    _absorb(r, rot)
    return RotarySpec(base, dims, scaling)


def _read_mixer(r: KeyReader) -> Optional[LatentAttentionSpec]:
    m = _sub(r, "mixer")
    if m is None:
        return None
    spec = LatentAttentionSpec(
        heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1), rot_dim=m.integer("rot_dim", minimum=2),
        vdim=m.integer("vdim", minimum=1), kv_rank=m.integer("kv_rank", minimum=1), q_rank=m.integer("q_rank", minimum=1),
        scale=m.number("scale", positive=True), rot=_read_rot(m))
    if spec.rot is not None and spec.rot.dims is not None and spec.rot_dim is not None and spec.rot.dims > spec.rot_dim:
        m.fail(f"rot.dims {spec.rot.dims} exceeds rot_dim {spec.rot_dim}")
    _absorb(r, m)
    return spec


def _read_mlp(r: KeyReader) -> Optional[FeedForwardSpec]:
    m = _sub(r, "mlp", required=False)
    if m is None:
        return None
    kind = m.string("kind")
    spec = None
    if kind == "dense":
        spec = FeedForwardSpec("dense", m.integer("ff", minimum=1))
    elif kind == "moe":
        expert, router = _sub(m, "expert"), _sub(m, "router")
        ff = expert.integer("ff", minimum=1) if expert is not None else None
        experts = router.integer("experts", minimum=1) if router is not None else None
        top = router.integer("top", minimum=1) if router is not None else None
        if experts is not None and top is not None and top > experts:
            m.fail(f"router.top {top} exceeds router.experts {experts}")
        _absorb(m, expert)
        _absorb(m, router)
        spec = FeedForwardSpec("moe", ff, experts or 0, top or 0)
    elif kind is not None:
        m.fail(f"unknown feed-forward kind '{kind}' (dense, moe)")
    _absorb(r, m)
    return spec


@dataclass(frozen=True)
class KakipelConfig(ModelConfig):
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    loop: Optional[LoopSpec]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "KakipelConfig":
        r = KeyReader(data, where)
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = _sub(r, "norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        _absorb(r, norm)
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
                if kind is not None and kind != "latent_attention":
                    lr.fail(f"unknown mixer type '{kind}' (latent_attention)")
                layers.append(LayerSpec(kind, _read_mixer(lr), _read_mlp(lr)))
                _absorb(r, lr)
        loop = None
        lp = _sub(r, "loop", required=False)
        if lp is not None:
            loop = LoopSpec(lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=1))
            if None not in (loop.start, loop.stop) and not loop.start < loop.stop <= max(len(layers), 1):
                lp.fail(f"start {loop.start} .. stop {loop.stop} is no run of the {len(layers)} layers")
            _absorb(r, lp)
        eos = r.int_list("eos_token_id", default=())
        init_range = r.number("initializer_range", default=0.05, positive=True)
        r.finish()
        return cls(architecture=KAKIPEL_ARCHITECTURE, vocab_size=vocab, width=width, norm_eps=eps, layers=tuple(layers),
                   loop=loop, eos_token_ids=eos, initializer_range=init_range)

    def to_dict(self) -> Dict[str, Any]:
        def rot(s: RotarySpec):
            out: Dict[str, Any] = {"base": s.base, "dims": s.dims}
            if s.scaling is not None:
                out["scaling"] = {"factor": s.scaling.factor, "original": s.scaling.original, "fast": s.scaling.fast,
                                  "slow": s.scaling.slow}
            return out

        def mlp(s: Optional[FeedForwardSpec]):
            if s is None:
                return None
            if s.kind == "dense":
                return {"kind": "dense", "ff": s.ff}
            return {"kind": "moe", "expert": {"ff": s.ff}, "router": {"experts": s.experts, "top": s.top}}

        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type,
                        "mixer": {"heads": l.mixer.heads, "dim": l.mixer.dim, "rot_dim": l.mixer.rot_dim, "vdim": l.mixer.vdim,
                                  "kv_rank": l.mixer.kv_rank, "q_rank": l.mixer.q_rank, "scale": l.mixer.scale,
                                  "rot": rot(l.mixer.rot)},
                        "mlp": mlp(l.mlp)} for l in self.layers],
            "initializer_range": self.initializer_range,
        }
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif len(self.eos_token_ids) > 1:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def layer_runs(self) -> Tuple[Tuple[int, Optional[int], bool], ...]:
        """(layer, pass or None, whether it opens its pass) for every layer run, in order."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, None, False) for i in range(n))
        lp = self.loop
        runs = [(i, None, False) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t, i == lp.start) for i in range(lp.start, lp.stop)]
        return tuple(runs + [(i, None, False) for i in range(lp.stop, n)])
