"""Typed configuration of the Toredra decoder, read from its own ``config.json`` keys.

Top level: ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` and
``logit_softcap`` (absent: 1 and none), ``loop`` (``start``, ``stop``, ``times``: layers start ..
stop - 1 run ``times`` times in a row with the same weights, each pass with a memory of its own;
absent or null: every layer once) and ``layers``, a list with one entry per layer: ``type`` (which
mixer), ``mixer`` (its sizes and constants) and ``mlp`` (``{"kind": "dense", "ff": n}``, or null).

* ``parallel``: ``mixer.left`` - attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale`` and
  ``rot`` (``dims`` rotated dimensions of a head, ``base``, and optionally ``scaling`` with ``factor``,
  ``low``, ``high``, ``original``) - and ``mixer.right`` - a gated linear recurrence: ``heads``, ``dim``,
  ``vdim``.
* ``general_delta``: ``heads``, ``dim``; the rank of the decay's two-step projection is the size of
  a checkpoint tensor (``decay_rank`` may name it in the file; `with_tensor_shapes` fills it in).

Every size and constant comes from the file; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, ModelConfig
from .zidivik_config import _number, _pos_int

NAME = "Toredra"

PARALLEL, GENERAL_DELTA = "parallel", "general_delta"


@dataclass(frozen=True)
class RotarySpec:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]]      # factor, low, high, original; None: frequencies as they are


@dataclass(frozen=True)
class SinkAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotarySpec]


@dataclass(frozen=True)
class ForgetGateSpec:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class ParallelSpec:
    left: SinkAttentionSpec
    right: ForgetGateSpec


@dataclass(frozen=True)
class GeneralDeltaSpec:
    heads: int
    dim: int
    decay_rank: int           # 0 until known


@dataclass(frozen=True)
class DenseSpec:
    ff: int


@dataclass(frozen=True)
class ToredraLayer:
    kind: str
    mixer: Any                # ParallelSpec | GeneralDeltaSpec
    mlp: Optional[DenseSpec]


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


def _rot(m: Dict[str, Any], dim: int, where: str) -> Optional[RotarySpec]:
    r = m.get("rot")
    if r is None:
        return None
    if not isinstance(r, dict):
        raise ConfigError(f"config.json: {where}.rot must be an object with 'dims' and 'base'")
    dims, base = _pos_int(r, "dims", where + ".rot"), _number(r, "base", where + ".rot")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {dim}")
    if base <= 0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive")
    sc = r.get("scaling")
    scaling = None
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
        scaling = tuple(_number(sc, k, where + ".rot.scaling") for k in ("factor", "low", "high", "original"))
        if scaling[0] <= 0 or scaling[3] <= 0 or scaling[1] == scaling[2] or scaling[1] <= 0 or scaling[2] <= 0:
            raise ConfigError(f"config.json: {where}.rot.scaling: factor, low, high, original must be positive and low differ from high")
    return RotarySpec(dims, base, scaling)


@dataclass(frozen=True)
class ToredraConfig(ModelConfig):
    layers: Tuple[ToredraLayer, ...] = ()
    norm_eps: float = 1e-6
    loop: Optional[LoopSpec] = None
    logit_scale: float = 1.0
    logit_softcap: float = 0.0

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ToredraConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _number(norm, "eps", "norm")
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
            m, kind = L["mixer"], L.get("type")
            if kind == PARALLEL:
                a, b = m.get("left"), m.get("right")
                if not isinstance(a, dict) or not isinstance(b, dict):
                    raise ConfigError(f"config.json: {where}.mixer needs 'left' and 'right'")
                wl, wr = where + ".mixer.left", where + ".mixer.right"
                heads, kv = _pos_int(a, "heads", wl), _pos_int(a, "kv_heads", wl)
                if heads % kv:
                    raise ConfigError(f"config.json: {wl}: {heads} heads are not a multiple of {kv} kv_heads")
                dim = _pos_int(a, "dim", wl)
                left = SinkAttentionSpec(heads, kv, dim, _pos_int(a, "vdim", wl), _number(a, "scale", wl), _rot(a, dim, wl))
                mixer: Any = ParallelSpec(left, ForgetGateSpec(_pos_int(b, "heads", wr), _pos_int(b, "dim", wr), _pos_int(b, "vdim", wr)))
            elif kind == GENERAL_DELTA:
                rank = m.get("decay_rank")
                mixer = GeneralDeltaSpec(_pos_int(m, "heads", where), _pos_int(m, "dim", where), int(rank) if rank else 0)
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is none of '{PARALLEL}', '{GENERAL_DELTA}'")
            f = L.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or of kind 'dense' with 'ff'")
                mlp = DenseSpec(_pos_int(f, "ff", where + ".mlp"))
            layers.append(ToredraLayer(kind, mixer, mlp))
        loop = None
        lp = raw.get("loop")
        if lp is not None:
            if not isinstance(lp, dict):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop', 'times' or null")
            loop = LoopSpec(_pos_int(lp, "start", "loop", allow_zero=True), _pos_int(lp, "stop", "loop", allow_zero=True),
                            _pos_int(lp, "times", "loop"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start} .. {loop.stop} does not lie inside the {len(layers)} layers")
        scale = _number(raw, "logit_scale", "config") if raw.get("logit_scale") is not None else 1.0
        cap = _number(raw, "logit_softcap", "config") if raw.get("logit_softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError("config.json: logit_softcap must be positive (or 0, null or absent for none)")
        max_pos = raw.get("max_positions")
        return cls(architecture=NAME, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(max_pos) if max_pos else 1 << 17, bos_token_id=None,
                   eos_token_ids=tuple(int(e) for e in raw.get("eos", ())), layers=tuple(layers), norm_eps=eps, loop=loop,
                   logit_scale=scale, logit_softcap=cap)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "ToredraConfig":
        """The sizes that only the checkpoint tells: the rank of each delta-rule mixer's decay
        projection, from the shape of its first matrix."""
        layers = list(self.layers)
        for i, L in enumerate(layers):
            if isinstance(L.mixer, GeneralDeltaSpec):
                w1 = shapes.get(f"l{i}.mix.w1")
                if w1 is None or len(w1) != 2:
                    raise ConfigError(f"layer {i}: the checkpoint has no l{i}.mix.w1 to size the decay's projection by")
                layers[i] = replace(L, mixer=replace(L.mixer, decay_rank=int(w1[0])))
        return replace(self, layers=tuple(layers))

    def layer_runs(self):
        """(layer, pass, first of a further pass) for every layer run, in order."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop <= self.loop.start:
            return [(i, 0, False) for i in range(n)]
        lp = self.loop
        runs = [(i, 0, False) for i in range(lp.start)]
        for rep in range(lp.times):
            runs += [(i, rep, rep > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        return runs + [(i, 0, False) for i in range(lp.stop, n)]

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": NAME, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
                               "max_positions": self.max_position_embeddings, "logit_scale": self.logit_scale, "layers": []}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_ids:
            out["eos"] = list(self.eos_token_ids)
        for L in self.layers:
            m = L.mixer
            if isinstance(m, ParallelSpec):
                a, b = m.left, m.right
                left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.rot is not None:
                    left["rot"] = {"dims": a.rot.dims, "base": a.rot.base}
                    if a.rot.scaling is not None:
                        left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), a.rot.scaling))
                mixer: Dict[str, Any] = {"left": left, "right": {"heads": b.heads, "dim": b.dim, "vdim": b.vdim}}
            else:
                mixer = {"heads": m.heads, "dim": m.dim}
                if m.decay_rank:
                    mixer["decay_rank"] = m.decay_rank
            out["layers"].append({"type": L.kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": L.mlp.ff} if L.mlp is not None else None})
        return out
