"""Typed configuration of the Selinex decoder, read from its config.json.

Keys: `architecture` ("Selinex"), `vocab`, `width`, `norm.eps`, `residual_mult`, `layers` (a list; each entry has `type`:
"parallel", "parallel_2" or "delta", `mixer` with that mixer's sizes and constants, and `mlp`: null, `{kind: dense, ff, limit}`
or `{kind: moe, expert: {ff}, router: {experts, top, groups: {count, keep}}}`), optional `loop` {start, stop, times}: the block of
layers [start, stop) is repeated `times` times before the layers behind it run, its weights shared and its caches and states not, optional
`max_positions` (the design has no position limit; the engine needs one for its rotation tables) and optional `eos_token_ids`.

parallel / parallel_2 mixer: `left` (windowed attention: heads, kv_heads, dim, vdim, scale, mask {size}, optional rot {dims,
base}) and `right` (parallel: heads, dim, vdim, tau; parallel_2: heads, dim), for parallel also left_scale and right_scale.
delta mixer: heads, kv_heads, dim, vdim, conv (taps). The rank of a recurrent mixer's low-rank decay map is no key of the file:
it is the first dimension of that map's first matrix (`l<i>.mix.right.a1` / `l<i>.mix.right.w1`), read from the checkpoint's
header when a model folder is opened (`rank`, which the random-weights mode writes into its config.json, takes precedence).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, FrozenSet, Optional, Tuple, Union

from .files import ConfigError
from .vapelix import DEFAULT_MAX_POSITIONS, Loop, _need

DEFAULT_DECAY_RANK = 16  # what the random-weights mode uses when a configuration names no rank


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0       # mask.size; 0: every earlier position is seen
    rot_dims: int = 0     # 0: positions do not enter the scores
    rot_base: float = 10000.0


@dataclass(frozen=True)
class DecayedLinear:      # right side of "parallel"
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int


@dataclass(frozen=True)
class TokenShift:         # right side of "parallel_2"
    heads: int
    dim: int
    rank: int


@dataclass(frozen=True)
class PairMixer:
    left: WindowAttention
    right: Union[DecayedLinear, TokenShift]
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class DenseFF:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoEFF:
    ff: int
    experts: int
    top: int
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class SelinexLayer:
    type: str  # "parallel" | "parallel_2" | "delta"
    mixer: Union[PairMixer, DeltaMixer]
    mlp: Union[None, DenseFF, MoEFF]


def _attention(m: Dict[str, Any], where: str) -> WindowAttention:
    rot, mask = m.get("rot"), m.get("mask")
    return WindowAttention(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)), dim=int(_need(m, "dim", where)),
                           vdim=int(_need(m, "vdim", where)), scale=float(_need(m, "scale", where)),
                           window=int(_need(mask, "size", where + ".mask")) if mask else 0,
                           rot_dims=int(_need(rot, "dims", where + ".rot")) if rot else 0,
                           rot_base=float(_need(rot, "base", where + ".rot")) if rot else 10000.0)


@dataclass(frozen=True)
class SelinexConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[SelinexLayer, ...]
    loop: Optional[Loop] = None
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
    def from_dict(cls, j: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "SelinexConfig":
        width, vocab = int(_need(j, "width", "config.json")), int(_need(j, "vocab", "config.json"))
        eps = float(_need(_need(j, "norm", "config.json"), "eps", "norm"))
        raw_layers = _need(j, "layers", "config.json")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind, m = _need(e, "type", where), _need(e, "mixer", where)
            if kind in ("parallel", "parallel_2"):
                left = _attention(_need(m, "left", where + ".mixer"), where + ".mixer.left")
                r = _need(m, "right", where + ".mixer")
                rw = where + ".mixer.right"
                rank = int(r.get("rank") or DEFAULT_DECAY_RANK)
                if kind == "parallel":
                    right = DecayedLinear(heads=int(_need(r, "heads", rw)), dim=int(_need(r, "dim", rw)), vdim=int(_need(r, "vdim", rw)),
                                          tau=float(_need(r, "tau", rw)), rank=rank)
                    mixer = PairMixer(left, right, float(_need(m, "left_scale", where + ".mixer")), float(_need(m, "right_scale", where + ".mixer")))
                else:
                    mixer = PairMixer(left, TokenShift(heads=int(_need(r, "heads", rw)), dim=int(_need(r, "dim", rw)), rank=rank))
            elif kind == "delta":
                mw = where + ".mixer"
                mixer = DeltaMixer(heads=int(_need(m, "heads", mw)), kv_heads=int(_need(m, "kv_heads", mw)), dim=int(_need(m, "dim", mw)),
                                   vdim=int(_need(m, "vdim", mw)), taps=int(_need(m, "conv", mw)))
            else:
                raise ConfigError(f"config.json: {where}: unknown layer type '{kind}' (parallel, parallel_2, delta)")
            f = e.get("mlp")
            mlp = None
            if f:
                fk = _need(f, "kind", where + ".mlp")
                if fk == "dense":
                    mlp = DenseFF(ff=int(_need(f, "ff", where + ".mlp")), limit=float(_need(f, "limit", where + ".mlp")))
                elif fk == "moe":
                    router = _need(f, "router", where + ".mlp")
                    groups = router.get("groups") or {}
                    mlp = MoEFF(ff=int(_need(_need(f, "expert", where + ".mlp"), "ff", "expert")), experts=int(_need(router, "experts", "router")),
                                top=int(_need(router, "top", "router")), groups=int(groups.get("count", 1)),
                                keep=int(groups.get("keep", groups.get("count", 1))))
                else:
                    raise ConfigError(f"config.json: {where}.mlp: unknown kind '{fk}' (dense, moe)")
            layers.append(SelinexLayer(kind, mixer, mlp))
        lp = j.get("loop")
        loop = Loop(int(_need(lp, "start", "loop")), int(_need(lp, "stop", "loop")), int(_need(lp, "times", "loop"))) if lp else None
        eos = j.get("eos_token_ids") or []
        cfg = cls(architecture=j.get("architecture", "Selinex"), vocab=vocab, width=width, eps=eps,
                  residual_mult=float(j.get("residual_mult", 1.0)), layers=tuple(layers), loop=loop,
                  max_positions=int(j.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=frozenset(int(t) for t in eos))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or self.eps < 0 or self.max_positions <= 0:
            raise ConfigError("config.json: width, vocab and max_positions must be positive, eps not negative")
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"config.json: layers[{i}]"
            if l.type == "delta":
                if min(m.heads, m.kv_heads, m.dim, m.vdim, m.taps) <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"{where}.mixer: sizes must be positive and heads a multiple of kv_heads")
            else:
                a, r = m.left, m.right
                if min(a.heads, a.kv_heads, a.dim, a.vdim) <= 0 or a.heads % a.kv_heads or a.window < 0:
                    raise ConfigError(f"{where}.mixer.left: sizes must be positive and heads a multiple of kv_heads")
                if a.rot_dims < 0 or a.rot_dims % 2 or a.rot_dims > a.dim:
                    raise ConfigError(f"{where}.mixer.left: rot.dims must be even and at most dim")
                if min(r.heads, r.dim, r.rank) <= 0 or (l.type == "parallel" and (r.vdim <= 0 or not r.tau > 0)):
                    raise ConfigError(f"{where}.mixer.right: sizes and tau must be positive")
            f = l.mlp
            if isinstance(f, DenseFF) and (f.ff <= 0 or not f.limit > 0):
                raise ConfigError(f"{where}.mlp: ff and limit must be positive")
            if isinstance(f, MoEFF):
                if f.ff <= 0 or not 1 <= f.top <= f.experts:
                    raise ConfigError(f"{where}.mlp: bad sizes")
                if f.groups < 1 or f.experts % f.groups or not 1 <= f.keep <= f.groups or f.keep * (f.experts // f.groups) < f.top:
                    raise ConfigError(f"{where}.mlp.router.groups: {f.experts} experts, {f.groups} groups of which {f.keep} stay, {f.top} chosen")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError("config.json: loop: need 0 <= start < stop <= number of layers and times >= 1")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "delta":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.taps}
            else:
                a, r = m.left, m.right
                left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.window:
                    left["mask"] = {"size": a.window}
                if a.rot_dims:
                    left["rot"] = {"dims": a.rot_dims, "base": a.rot_base}
                if l.type == "parallel":
                    mixer = {"left": left, "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "tau": r.tau, "rank": r.rank},
                             "left_scale": m.left_scale, "right_scale": m.right_scale}
                else:
                    mixer = {"left": left, "right": {"heads": r.heads, "dim": r.dim, "rank": r.rank}}
            f, mlp = l.mlp, None
            if isinstance(f, DenseFF):
                mlp = {"kind": "dense", "ff": f.ff, "limit": f.limit}
            elif isinstance(f, MoEFF):
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top,
                                                                          "groups": {"count": f.groups, "keep": f.keep}}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                               "residual_mult": self.residual_mult, "layers": layers, "max_positions": self.max_positions}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_ids:
            out["eos_token_ids"] = sorted(self.eos_token_ids)
        return out


def sizes_from_tensors(j: Dict[str, Any], shape_of: Callable[[str], Optional[Tuple[int, ...]]]) -> Dict[str, Any]:
    """The sizes that only tensor shapes give, written into a copy of the configuration: the rank of every recurrent mixer's
    low-rank decay map. shape_of(name) -> the checkpoint's shape of that tensor, or None."""
    import copy
    j = copy.deepcopy(j)
    for i, e in enumerate(j.get("layers") or []):
        first = {"parallel": "a1", "parallel_2": "w1"}.get(e.get("type"))
        right = (e.get("mixer") or {}).get("right")
        if first and isinstance(right, dict) and not right.get("rank"):
            shape = shape_of(f"l{i}.mix.right.{first}")
            if shape is not None and len(shape) == 2:
                right["rank"] = int(shape[0])
    return j
