"""Typed configuration of the Kimilix decoder, read from the keys of its ``config.json``.

A Kimilix model is a list of layers whose sublayers read the residual itself and whose norms stand behind them:
x <- x + residual_mult * ls * norm(sublayer(x)), the norm's weight stored less one, ``ls`` a learned vector a
sublayer.  The file gives ``width``, ``vocab``, ``embedding.scale`` (the factor on the embedding rows), ``norm.eps``,
``residual_mult`` and, per entry of ``layers``, ``type`` (the mixer), ``mixer`` (its sizes and constants) and ``mlp``:
``{"kind": "dense", "ff": F}`` (down(relu(up x)^2)), ``{"kind": "moe", "expert": {"ff": F, "limit": L}, "router":
{"experts": E, "top": K}, "shared": {"ff": S, "limit": L}}`` (``shared`` may be left out) or null.  The head is the
embedding table.

Mixer ``attention``: differential attention.  ``heads``, ``kv_heads`` (absent: as many as heads), ``dim`` (a map's
query/key size), ``vdim`` (absent: ``dim``), ``scale``, ``diff`` (the constant in the second map's factor), ``rot``
(``dims``, ``base`` and optionally ``scaling`` {factor, low, high, original}; rotate-half over the first ``dims``
channels of each map; absent: none), ``mask.size`` (blocks of that many positions; absent: every earlier key).

Mixer ``latent_attention``: ``heads``, ``dim`` (plain query/key channels a head), ``rot_dim`` (rotated channels, one
rotated key part for all heads, neighbouring channels together), ``vdim``, ``q_rank``, ``kv_rank``, ``scale``, ``rot``
(``base``, ``dims`` = ``rot_dim``, optionally ``scaling``), ``mask.size`` (a sliding window; absent: every earlier key).

The constants the design fixes stand below and travel in the parts' specs.

Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.ls1``, ``l<i>.mix.q``, ``l<i>.mix.q.norm``,
``l<i>.mix.lq1``, ``l<i>.mix.dq``, ``l<i>.mix.dq.norm``, ``l<i>.mix.uk``, ``l<i>.mlp.up``, ``l<i>.mlp.e<j>.gate``,
``l<i>.mlp.router``, ``l<i>.mlp.router.b``, ``l<i>.mlp.shared.sg``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .pugalix import _LIMIT, _freeze, _get, _int, _pos, _thaw  # noqa: F401
from .qwen3 import ConfigError
from .spec import (ClampedGLUSpec, DiffAttentionSpec, EmbeddingSpec, HeadSpec, LatentAttentionSpec, ModelSpec, MoESpec, NoPositionSpec,
                   PairRotarySpec, PostNormLayerSpec, RMSNormSpec, ReluSquaredSpec, RotarySpec, ScheduleEntry)

MIXERS = ("attention", "latent_attention")
GATE_SLOPE = 1.702        # an expert's gate is g * sigmoid(GATE_SLOPE * g)
NORM_OFFSET = 1.0         # norm weights are stored less one


def _number(d, key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"config.json: '{where}{key}' must be a finite number, got {v!r}")
    return float(v)


def _rot(m: dict, ma: str, width: int) -> None:
    """Checks ``m['rot']``: ``dims`` even and at most ``width``, a positive ``base``, a usable ``scaling``."""
    rot = _get(m, "rot", ma)
    dims = _int(rot, "dims", ma + "rot.", low=0)
    if dims % 2 or dims > width:
        raise ConfigError(f"config.json: '{ma}rot.dims' {dims} must be even and at most {width}")
    _pos(rot, "base", ma + "rot.")
    if rot.get("scaling") is not None:
        sc, sa = rot["scaling"], ma + "rot.scaling."
        factor, low, high, orig = (_pos(sc, k, sa) for k in ("factor", "low", "high", "original"))
        if not high > low:
            raise ConfigError(f"config.json: '{sa}high' {high} must exceed '{sa}low' {low}")


@dataclass(frozen=True)
class KimilixLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's keys, as read (nested dicts as tuples of pairs)
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def get(self, *path):
        node: Any = dict(self.mixer)
        for k in path:
            node = dict(node)[k]
        return node

    def has(self, *path) -> bool:
        node: Any = dict(self.mixer)
        for k in path:
            if not isinstance(node, (dict, tuple)) or k not in dict(node):
                return False
            node = dict(node)[k]
        return True


@dataclass(frozen=True)
class KimilixConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[KimilixLayer, ...]
    architecture: str = "Kimilix"
    tie_word_embeddings = True              # the head is the embedding table (no field: the file has no such key)

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KimilixConfig":
        width, vocab = _int(d, "width", ""), _int(d, "vocab", "")
        eps = _pos(_get(d, "norm", ""), "eps", "norm.")
        emb = 1.0 if d.get("embedding") is None else _number(d["embedding"], "scale", "embedding.")
        mult = 1.0 if d.get("residual_mult") is None else _number(d, "residual_mult", "")
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[KimilixLayer] = []
        for i, raw in enumerate(raw_layers):
            at = f"layers[{i}]."
            kind = _get(raw, "type", at)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: '{at}type' is {kind!r}; this design has {', '.join(MIXERS)}")
            m = _get(raw, "mixer", at)
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: '{at}mixer' must be an object")
            ma = at + "mixer."
            m = {k: v for k, v in m.items() if v is not None}
            heads, dim = _int(m, "heads", ma), _int(m, "dim", ma)
            if "vdim" in m:
                _int(m, "vdim", ma)
            _pos(m, "scale", ma)
            if "mask" in m:
                _int(_get(m, "mask", ma), "size", ma + "mask.")
            if kind == "attention":
                if "kv_heads" in m and heads % _int(m, "kv_heads", ma):
                    raise ConfigError(f"config.json: '{ma}heads' {heads} is not a multiple of '{ma}kv_heads' {m['kv_heads']}")
                _number(m, "diff", ma)
                if "rot" in m:
                    _rot(m, ma, dim)
            else:
                _int(m, "q_rank", ma)
                _int(m, "kv_rank", ma)
                rd = _int(m, "rot_dim", ma, low=0)
                if rd % 2:
                    raise ConfigError(f"config.json: '{ma}rot_dim' {rd} must be even")
                if rd > 0:
                    _rot(m, ma, rd)
                    if m["rot"]["dims"] != rd:
                        raise ConfigError(f"config.json: '{ma}rot.dims' {m['rot']['dims']} must equal '{ma}rot_dim' {rd}")
            mlp = raw.get("mlp") if isinstance(raw, dict) else None
            if mlp is not None:
                fa = at + "mlp."
                fk = _get(mlp, "kind", fa)
                if fk == "dense":
                    _int(mlp, "ff", fa)
                elif fk == "moe":
                    ex = _get(mlp, "expert", fa)
                    _int(ex, "ff", fa + "expert.")
                    _pos(ex, "limit", fa + "expert.")
                    router = _get(mlp, "router", fa)
                    experts, top = _int(router, "experts", fa + "router."), _int(router, "top", fa + "router.")
                    if top > experts:
                        raise ConfigError(f"config.json: '{fa}router.top' {top} exceeds its {experts} experts")
                    if mlp.get("shared") is not None:
                        _int(mlp["shared"], "ff", fa + "shared.")
                        _pos(mlp["shared"], "limit", fa + "shared.")
                else:
                    raise ConfigError(f"config.json: '{fa}kind' is {fk!r}; this design has dense and moe feed-forwards")
                mlp = {k: v for k, v in mlp.items() if v is not None}
            layers.append(KimilixLayer(kind, _freeze(m), None if mlp is None else _freeze(mlp)))
        return cls(width=width, vocab=vocab, norm_eps=eps, embedding_scale=emb, residual_mult=mult, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Kimilix")))

    # ---- writing -------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": _thaw(l.mixer), "mlp": None if l.mlp is None else _thaw(l.mlp)} for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }

    def with_layers(self, n: int) -> "KimilixConfig":
        if not 0 < n <= len(self.layers):
            raise ValueError(f"layers={n} of a configuration with {len(self.layers)}")
        return KimilixConfig(self.width, self.vocab, self.norm_eps, self.embedding_scale, self.residual_mult, self.layers[:n], self.architecture)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    # ---- derived -------------------------------------------------------------------------
    @staticmethod
    def _scaling(l: KimilixLayer):
        if not l.has("rot", "scaling"):
            return None
        sc = _thaw(l.get("rot", "scaling"))
        return (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = lambda: RMSNormSpec(size=W, eps=eps, tensor="", offset=NORM_OFFSET)
        layers = []
        for i, l in enumerate(self.layers):
            heads, d = l.get("heads"), l.get("dim")
            dv = l.get("vdim") if l.has("vdim") else d
            size = l.get("mask", "size") if l.has("mask") else 0
            if l.type == "attention":
                position = (RotarySpec(head_dim=d, rotary_dim=l.get("rot", "dims"), theta=float(l.get("rot", "base")), scaling=self._scaling(l))
                            if l.has("rot") and l.get("rot", "dims") > 0 else NoPositionSpec(head_dim=d))
                mixer = DiffAttentionSpec(hidden=W, heads=heads, kv_heads=l.get("kv_heads") if l.has("kv_heads") else heads, head_dim=d,
                                          value_dim=dv, scale=float(l.get("scale")), position=position, lambda_init=float(l.get("diff")),
                                          eps=eps, qk_norm=RMSNormSpec(size=d, eps=eps), chunk=size)
            else:
                rd = l.get("rot_dim")
                position = (PairRotarySpec(head_dim=rd, rotary_dim=rd, theta=float(l.get("rot", "base")), scaling=self._scaling(l))
                            if rd > 0 else NoPositionSpec(head_dim=rd))
                mixer = LatentAttentionSpec(hidden=W, heads=heads, head_dim=d, rot_dim=rd, value_dim=dv, q_rank=l.get("q_rank"),
                                            kv_rank=l.get("kv_rank"), scale=float(l.get("scale")), position=position, eps=eps, window=size)
            ff = ff_norm = None
            if l.mlp is not None:
                mlp = _thaw(l.mlp)
                if mlp["kind"] == "dense":
                    ff = ReluSquaredSpec(hidden=W, intermediate=mlp["ff"])
                else:
                    shared = mlp.get("shared")
                    ff = MoESpec(hidden=W, experts=mlp["router"]["experts"], top=mlp["router"]["top"], intermediate=mlp["expert"]["ff"],
                                 renorm_eps=0.0, score="softmax", renorm=True, weight_on="output", act="glu_clamp",
                                 act_limit=float(mlp["expert"]["limit"]), act_slope=GATE_SLOPE, router_bias=True,
                                 shared=None if shared is None else ClampedGLUSpec(hidden=W, intermediate=shared["ff"], limit=float(shared["limit"]),
                                                                                   slope=GATE_SLOPE),
                                 shared_gate=shared is not None)
                ff_norm = norm()
            layers.append(PostNormLayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=norm(), feed_forward_norm=ff_norm,
                                            residual_mult=self.residual_mult))
        spec = ModelSpec(
            architecture=self.architecture, hidden=W, vocab=self.vocab, max_positions=1 << 30,
            embedding=EmbeddingSpec("embed", self.vocab, W, scale=self.embedding_scale), layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
            final_norm=RMSNormSpec(size=W, eps=eps, tensor="", offset=NORM_OFFSET), final_norm_name="final.norm",
            head=HeadSpec("head", self.vocab, W, tied_to="embed"))
        spec.validate()
        return spec
