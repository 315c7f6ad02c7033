"""Typed configuration of the Sogutar decoder, read from its config.json.

Keys: `architecture` ("Sogutar"), `vocab`, `width`, `norm.eps`, optional `logit_softcap`, `layers` (a list; each entry has
`type`: "attention" or "retention", `mixer` with that mixer's sizes and constants, and `mlp`: null, `{kind: dense, ff}` or
`{kind: moe, expert: {ff, limit}, router: {experts, identity, top, scale}, shared: {ff, limit}}`), optional `max_positions` (the
design has no position limit; the engine needs one for its rotation tables) and optional `eos_token_ids`.

attention mixer: heads, kv_heads, dim, vdim, scale, optional mask {size}, optional rot {dims, base, optional scaling {factor,
low, high, original}}, optional kv_from (the index of an earlier attention layer whose keys and values this layer reads).
retention mixer: heads, dim, vdim, decay (a number a head), optional rot {dims, base}.
A size that the file leaves out and a tensor's shape gives (vocab and width, a head's sizes, the feed-forwards' inner sizes)
is read from the checkpoint's header when a model folder is opened (`sizes_from_tensors`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, FrozenSet, Optional, Tuple, Union

from .files import ConfigError
from .vapelix import DEFAULT_MAX_POSITIONS, _need


@dataclass(frozen=True)
class FrequencyScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[FrequencyScaling] = None


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0            # mask.size; 0: every earlier position is seen
    rot: Optional[Rotation] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class RetentionMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[Rotation] = None


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class SharedExpert:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoEFF:
    ff: int
    limit: float
    experts: int
    identity: int
    top: int
    scale: float
    shared: Optional[SharedExpert] = None


@dataclass(frozen=True)
class SogutarLayer:
    type: str  # "attention" | "retention"
    mixer: Union[AttentionMixer, RetentionMixer]
    mlp: Union[None, DenseFF, MoEFF]


def _rotation(m: Dict[str, Any], where: str) -> Optional[Rotation]:
    rot = m.get("rot")
    if not rot:
        return None
    sc = rot.get("scaling")
    scaling = None
    if sc:
        w = where + ".rot.scaling"
        scaling = FrequencyScaling(float(_need(sc, "factor", w)), float(_need(sc, "low", w)), float(_need(sc, "high", w)), float(_need(sc, "original", w)))
    return Rotation(int(_need(rot, "dims", where + ".rot")), float(_need(rot, "base", where + ".rot")), scaling)


def _rotation_dict(r: Optional[Rotation]):
    if r is None:
        return None
    out: Dict[str, Any] = {"dims": r.dims, "base": r.base}
    if r.scaling is not None:
        s = r.scaling
        out["scaling"] = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
    return out


@dataclass(frozen=True)
class SogutarConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[SogutarLayer, ...]
    logit_softcap: float = 0.0   # 0: logits as they are
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: FrozenSet[int] = field(default_factory=frozenset)

    # names shared with the other configurations (the command line and the scheduler read them)
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, j: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "SogutarConfig":
        width, vocab = int(_need(j, "width", "config.json")), int(_need(j, "vocab", "config.json"))
        eps = float(_need(_need(j, "norm", "config.json"), "eps", "norm"))
        raw_layers = _need(j, "layers", "config.json")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind, m = _need(e, "type", where), _need(e, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                mask = m.get("mask")
                src = m.get("kv_from")
                mixer: Union[AttentionMixer, RetentionMixer] = AttentionMixer(
                    heads=int(_need(m, "heads", mw)), kv_heads=int(_need(m, "kv_heads", mw)), dim=int(_need(m, "dim", mw)),
                    vdim=int(_need(m, "vdim", mw)), scale=float(_need(m, "scale", mw)),
                    window=int(_need(mask, "size", mw + ".mask")) if mask else 0, rot=_rotation(m, mw),
                    kv_from=None if src is None else int(src))
            elif kind == "retention":
                decay = _need(m, "decay", mw)
                if not isinstance(decay, list):
                    raise ConfigError(f"config.json: {mw}.decay must be a list with a number a head")
                mixer = RetentionMixer(heads=int(_need(m, "heads", mw)), dim=int(_need(m, "dim", mw)), vdim=int(_need(m, "vdim", mw)),
                                       decay=tuple(float(d) for d in decay), rot=_rotation(m, mw))
            else:
                raise ConfigError(f"config.json: {where}: unknown layer type '{kind}' (attention, retention)")
            f = e.get("mlp")
            mlp: Union[None, DenseFF, MoEFF] = None
            if f:
                fw = where + ".mlp"
                fk = _need(f, "kind", fw)
                if fk == "dense":
                    mlp = DenseFF(ff=int(_need(f, "ff", fw)))
                elif fk == "moe":
                    ex, router, sh = _need(f, "expert", fw), _need(f, "router", fw), f.get("shared")
                    mlp = MoEFF(ff=int(_need(ex, "ff", fw + ".expert")), limit=float(_need(ex, "limit", fw + ".expert")),
                                experts=int(_need(router, "experts", fw + ".router")), identity=int(router.get("identity") or 0),
                                top=int(_need(router, "top", fw + ".router")), scale=float(router.get("scale", 1.0)),
                                shared=SharedExpert(int(_need(sh, "ff", fw + ".shared")), float(_need(sh, "limit", fw + ".shared"))) if sh else None)
                else:
                    raise ConfigError(f"config.json: {fw}: unknown kind '{fk}' (dense, moe)")
            layers.append(SogutarLayer(kind, mixer, mlp))
        eos = j.get("eos_token_ids") or []
        cfg = cls(architecture=j.get("architecture", "Sogutar"), vocab=vocab, width=width, eps=eps, layers=tuple(layers),
                  logit_softcap=float(j.get("logit_softcap") or 0.0), max_positions=int(j.get("max_positions") or DEFAULT_MAX_POSITIONS),
                  eos_token_ids=frozenset(int(t) for t in eos))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or self.eps < 0 or self.max_positions <= 0 or self.logit_softcap < 0:
            raise ConfigError("config.json: width, vocab and max_positions must be positive, eps and logit_softcap not negative")
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"config.json: layers[{i}]"
            if m.rot is not None:
                r = m.rot
                if r.dims < 0 or r.dims % 2 or r.dims > m.dim or not r.base > 0:
                    raise ConfigError(f"{where}.mixer.rot: dims must be even and at most dim, base positive")
                if r.scaling is not None and not (r.scaling.factor > 0 and r.scaling.original > 0 and r.scaling.high > r.scaling.low > 0):
                    raise ConfigError(f"{where}.mixer.rot.scaling: factor and original must be positive and high > low > 0")
            if l.type == "attention":
                if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads or m.window < 0:
                    raise ConfigError(f"{where}.mixer: sizes must be positive and heads a multiple of kv_heads")
                if m.kv_from is not None:
                    if not 0 <= m.kv_from < i or self.layers[m.kv_from].type != "attention":
                        raise ConfigError(f"{where}.mixer.kv_from: {m.kv_from} is no earlier attention layer")
                    o = self.layers[m.kv_from].mixer
                    if o.kv_from is not None:
                        raise ConfigError(f"{where}.mixer.kv_from: layer {m.kv_from} has no keys and values of its own")
                    if (o.kv_heads, o.dim, o.vdim, o.rot) != (m.kv_heads, m.dim, m.vdim, m.rot):
                        raise ConfigError(f"{where}.mixer.kv_from: layer {m.kv_from}'s key/value heads, head sizes or rotation differ from this layer's")
            else:
                if min(m.heads, m.dim, m.vdim) <= 0 or len(m.decay) != m.heads:
                    raise ConfigError(f"{where}.mixer: sizes must be positive, and decay has a number a head")
                if not all(0.0 <= d <= 1.0 for d in m.decay):
                    raise ConfigError(f"{where}.mixer.decay: every decay lies in [0, 1]")
            f = l.mlp
            if isinstance(f, DenseFF) and f.ff <= 0:
                raise ConfigError(f"{where}.mlp: ff must be positive")
            if isinstance(f, MoEFF):
                if f.ff <= 0 or f.experts < 1 or f.identity < 0 or not 1 <= f.top <= f.experts + f.identity or not f.limit > 0:
                    raise ConfigError(f"{where}.mlp: {f.top} of {f.experts} + {f.identity} experts of {f.ff} with limit {f.limit}")
                if f.shared is not None and (f.shared.ff <= 0 or not f.shared.limit > 0):
                    raise ConfigError(f"{where}.mlp.shared: ff and limit must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.window:
                    mixer["mask"] = {"size": m.window}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            if m.rot is not None:
                mixer["rot"] = _rotation_dict(m.rot)
            f, mlp = l.mlp, None
            if isinstance(f, DenseFF):
                mlp = {"kind": "dense", "ff": f.ff}
            elif isinstance(f, MoEFF):
                mlp = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                       "router": {"experts": f.experts, "identity": f.identity, "top": f.top, "scale": f.scale}}
                if f.shared is not None:
                    mlp["shared"] = {"ff": f.shared.ff, "limit": f.shared.limit}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                               "layers": layers, "max_positions": self.max_positions}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            out["eos_token_ids"] = sorted(self.eos_token_ids)
        return out


def sizes_from_tensors(j: Dict[str, Any], shape_of: Callable[[str], Optional[Tuple[int, ...]]]) -> Dict[str, Any]:
    """Sizes that the file leaves out and a tensor's shape gives, written into a copy of the configuration. shape_of(name) -> the
    checkpoint's shape of that tensor, or None. What the file says is never overruled here (the loader reports a disagreement)."""
    import copy
    j = copy.deepcopy(j)

    def fill(d, key, name, value_of):
        if isinstance(d, dict) and d.get(key) is None:
            shape = shape_of(name)
            if shape is not None:
                v = value_of(shape)
                if v is not None:
                    d[key] = int(v)

    fill(j, "vocab", "embed", lambda s: s[0])
    fill(j, "width", "embed", lambda s: s[1] if len(s) > 1 else None)
    for i, e in enumerate(j.get("layers") or []):
        if not isinstance(e, dict):
            continue
        m, p = e.get("mixer"), f"l{i}."
        if isinstance(m, dict) and m.get("heads"):
            H = int(m["heads"])
            fill(m, "dim", p + "mix.q", lambda s: s[0] // H if s[0] % H == 0 else None)
            fill(m, "vdim", p + "mix.o", lambda s: s[1] // H if len(s) > 1 and s[1] % H == 0 else None)
            if e.get("type") == "attention" and m.get("dim"):
                fill(m, "kv_heads", p + "mix.k", lambda s: s[0] // int(m["dim"]) if s[0] % int(m["dim"]) == 0 else None)
        f = e.get("mlp")
        if isinstance(f, dict):
            if f.get("kind") == "dense":
                fill(f, "ff", p + "mlp.gate", lambda s: s[0])
            elif f.get("kind") == "moe":
                fill(f.get("expert"), "ff", p + "mlp.e0.gate", lambda s: s[0])
                fill(f.get("shared"), "ff", p + "mlp.shared.gate", lambda s: s[0])
    return j
