"""Typed configuration of the Korirax decoder, read from its own ``config.json`` keys.

Top level: ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (absent: 1),
``token_side.dim`` (absent, null or 0: no per-layer token input), ``loop`` (``start``, ``stop``, ``times``:
layers start .. stop - 1 run ``times`` times in a row with the same weights, each pass with a memory of
its own and a learned vector added to the stream in front of it; absent or null: every layer once) and
``layers``, a list with one entry per layer: ``type`` (which mixer), ``mixer`` (its sizes and constants)
and ``mlp`` (null, ``{"kind": "dense", "ff": n}``, or ``{"kind": "moe", "expert": {"ff": n}, "router":
{"experts", "top", "scale", "groups": {"count", "keep"}}, "shared": {"ff": n} or null}``).

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``bias_max`` (the distance from
  which all keys share the last row of the layer's table of distance terms; the number of rows is the
  table's shape), ``q_temp`` (``coef``, ``every``; absent or null: none).
* ``latent_attention``: ``heads``, ``dim`` (unrotated) and ``rot_dim`` (rotated) query/key dimensions a
  head, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``, ``rot`` (``dims``, ``base`` and optionally ``scaling``
  with ``factor``, ``original``, ``fast``, ``slow``).
* ``rglru``: ``width`` (channels), ``blocks`` (of the gates' block-diagonal matrices), ``conv`` (taps).

Every size and constant comes from the file; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, ModelConfig
from .zidivik_config import _number, _pos_int

NAME = "Korirax"

ATTENTION, LATENT, RGLRU = "attention", "latent_attention", "rglru"


@dataclass(frozen=True)
class YarnSpec:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotSpec:
    dims: int
    base: float
    scaling: Optional[YarnSpec]


@dataclass(frozen=True)
class BiasedAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int
    bias_rows: int                          # 0 until the checkpoint's table has told
    q_temp: Optional[Tuple[float, int]]     # (coef, every)


@dataclass(frozen=True)
class RotaryLatentSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[RotSpec]


@dataclass(frozen=True)
class RglruSpec:
    width: int
    blocks: int
    taps: int


@dataclass(frozen=True)
class DenseSpec:
    ff: int


@dataclass(frozen=True)
class MoeSpec:
    ff: int
    experts: int
    top: int
    scale: float
    groups: int
    keep: int
    shared_ff: int          # 0: no expert that every token takes


@dataclass(frozen=True)
class KoriraxLayer:
    kind: str
    mixer: Any              # BiasedAttentionSpec | RotaryLatentSpec | RglruSpec
    mlp: Any                # None | DenseSpec | MoeSpec


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


def _obj(raw: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return v


def _rot(m: Dict[str, Any], rot_dim: int, where: str) -> Optional[RotSpec]:
    r = _obj(m, "rot", where, optional=True)
    if r is None:
        return None
    w = where + ".rot"
    dims, base = _pos_int(r, "dims", w), _number(r, "base", w)
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json: {w}.dims {dims} must be even and at most rot_dim {rot_dim}")
    if base <= 1:
        raise ConfigError(f"config.json: {w}.base must exceed 1")
    sc = _obj(r, "scaling", w, optional=True)
    scaling = None
    if sc is not None:
        scaling = YarnSpec(*(_number(sc, k, w + ".scaling") for k in ("factor", "original", "fast", "slow")))
        if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
            raise ConfigError(f"config.json: {w}.scaling: factor, original, fast and slow must be positive")
    return RotSpec(dims, base, scaling)


def _mlp(f: Any, where: str):
    if f is None:
        return None
    if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where} must be null or of kind 'dense' or 'moe'")
    if f["kind"] == "dense":
        return DenseSpec(_pos_int(f, "ff", where))
    e, r = _obj(f, "expert", where), _obj(f, "router", where)
    experts, top = _pos_int(r, "experts", where + ".router"), _pos_int(r, "top", where + ".router")
    g = _obj(r, "groups", where + ".router", optional=True)
    groups, keep = (1, 1) if g is None else (_pos_int(g, "count", where + ".router.groups"), _pos_int(g, "keep", where + ".router.groups"))
    if experts % groups or keep > groups or top > keep * (experts // groups):
        raise ConfigError(f"config.json: {where}.router: {experts} experts in {groups} groups, {keep} kept, {top} chosen do not fit")
    scale = _number(r, "scale", where + ".router") if r.get("scale") is not None else 1.0
    s = _obj(f, "shared", where, optional=True)
    return MoeSpec(_pos_int(e, "ff", where + ".expert"), experts, top, scale, groups, keep, _pos_int(s, "ff", where + ".shared") if s else 0)


@dataclass(frozen=True)
class KoriraxConfig(ModelConfig):
    layers: Tuple[KoriraxLayer, ...] = ()
    norm_eps: float = 1e-6
    loop: Optional[LoopSpec] = None
    embedding_scale: float = 1.0
    side_dim: int = 0

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KoriraxConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        eps = _number(_obj(raw, "norm", "config"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must list the layers")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m, kind, w = L["mixer"], L.get("type"), where + ".mixer"
            if kind == ATTENTION:
                heads, kv = _pos_int(m, "heads", w), _pos_int(m, "kv_heads", w)
                if heads % kv:
                    raise ConfigError(f"config.json: {w}: {heads} heads are not a multiple of {kv} kv_heads")
                qt = _obj(m, "q_temp", w, optional=True)
                q_temp = (_number(qt, "coef", w + ".q_temp"), _pos_int(qt, "every", w + ".q_temp")) if qt else None
                rows = m.get("bias_rows")
                mixer: Any = BiasedAttentionSpec(heads, kv, _pos_int(m, "dim", w), _pos_int(m, "vdim", w), _number(m, "scale", w),
                                                 _pos_int(m, "bias_max", w), int(rows) if rows else 0, q_temp)
            elif kind == LATENT:
                rot_dim = _pos_int(m, "rot_dim", w, allow_zero=True)
                mixer = RotaryLatentSpec(_pos_int(m, "heads", w), _pos_int(m, "dim", w), rot_dim, _pos_int(m, "vdim", w), _pos_int(m, "q_rank", w),
                                         _pos_int(m, "kv_rank", w), _number(m, "scale", w), _rot(m, rot_dim, w))
            elif kind == RGLRU:
                mixer = RglruSpec(_pos_int(m, "width", w), _pos_int(m, "blocks", w), _pos_int(m, "conv", w))
                if mixer.width % mixer.blocks:
                    raise ConfigError(f"config.json: {w}: {mixer.width} channels do not divide into {mixer.blocks} blocks")
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is none of '{ATTENTION}', '{LATENT}', '{RGLRU}'")
            layers.append(KoriraxLayer(kind, mixer, _mlp(L.get("mlp"), where + ".mlp")))
        loop = None
        lp = _obj(raw, "loop", "config", optional=True)
        if lp is not None:
            loop = LoopSpec(_pos_int(lp, "start", "loop", allow_zero=True), _pos_int(lp, "stop", "loop", allow_zero=True), _pos_int(lp, "times", "loop"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start} .. {loop.stop} does not lie inside the {len(layers)} layers")
        emb = _obj(raw, "embedding", "config", optional=True)
        side = _obj(raw, "token_side", "config", optional=True)
        max_pos = raw.get("max_positions")
        return cls(architecture=NAME, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(max_pos) if max_pos else 1 << 17, bos_token_id=None,
                   eos_token_ids=tuple(int(e) for e in raw.get("eos", ())), layers=tuple(layers), norm_eps=eps, loop=loop,
                   embedding_scale=_number(emb, "scale", "embedding") if emb and emb.get("scale") is not None else 1.0,
                   side_dim=int(side["dim"]) if side and side.get("dim") else 0)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "KoriraxConfig":
        """The sizes that only the checkpoint tells: the rows of each attention layer's table of distance terms."""
        layers = list(self.layers)
        for i, L in enumerate(layers):
            if isinstance(L.mixer, BiasedAttentionSpec):
                rel = shapes.get(f"l{i}.mix.rel")
                if rel is None or len(rel) != 2:
                    raise ConfigError(f"layer {i}: the checkpoint has no l{i}.mix.rel to size the table of distance terms by")
                layers[i] = replace(L, mixer=replace(L.mixer, bias_rows=int(rel[0])))
        return replace(self, layers=tuple(layers))

    def layer_runs(self):
        """(layer, pass number if the layer opens a pass of the loop else None) for every layer run, in order."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop <= self.loop.start:
            return [(i, None) for i in range(n)]
        lp = self.loop
        runs = [(i, None) for i in range(lp.start)]
        for rep in range(lp.times):
            runs += [(i, rep if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    @property
    def loop_passes(self) -> int:
        return self.loop.times if self.loop is not None and self.loop.stop > self.loop.start else 0

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": NAME, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
                               "max_positions": self.max_position_embeddings, "embedding": {"scale": self.embedding_scale}, "layers": []}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_ids:
            out["eos"] = list(self.eos_token_ids)
        for L in self.layers:
            m = L.mixer
            if isinstance(m, BiasedAttentionSpec):
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                                         "bias_max": m.bias_max}
                if m.bias_rows:
                    mixer["bias_rows"] = m.bias_rows
                if m.q_temp:
                    mixer["q_temp"] = {"coef": m.q_temp[0], "every": m.q_temp[1]}
            elif isinstance(m, RotaryLatentSpec):
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                         "scale": m.scale}
                if m.rot is not None:
                    mixer["rot"] = {"dims": m.rot.dims, "base": m.rot.base}
                    if m.rot.scaling is not None:
                        s = m.rot.scaling
                        mixer["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            else:
                mixer = {"width": m.width, "blocks": m.blocks, "conv": m.taps}
            f = L.mlp
            if f is None:
                mlp: Any = None
            elif isinstance(f, DenseSpec):
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top, "scale": f.scale,
                                                                          "groups": {"count": f.groups, "keep": f.keep}},
                       "shared": {"ff": f.shared_ff} if f.shared_ff else None}
            out["layers"].append({"type": L.kind, "mixer": mixer, "mlp": mlp})
        return out
