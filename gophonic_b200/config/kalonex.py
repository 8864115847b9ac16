"""Typed configuration of the Kalonex decoder, read from the keys of its ``config.json``.

A Kalonex model is a list of pre-norm layers, a stretch of which may run several times in a row with the same
weights.  The file gives ``width``, ``vocab``, ``norm.eps``, ``logit_scale`` (the factor on the logits; 1 if absent),
``loop`` (``{"start": a, "stop": b, "times": n}``: layers a .. b-1 run n times, every pass with caches of its own;
absent: every layer runs once) and, per entry of ``layers``, ``type`` (the mixer: ``attention``), ``mixer`` (its
sizes and constants) and ``mlp``: ``{"kind": "dense", "ff": F}``, ``{"kind": "moe", "expert": {"ff": F}, "router":
{"experts": E, "top": K}, "shared": {"ff": S}}`` (``shared`` may be left out) or null.

Where a pass through the repeated layers begins, the residual x and the embedding output x0 are mixed,
x <- W [x; x0] + step[pass], with ``loop.in`` ([width, 2 width]) and ``loop.step`` ([times, width]).

The attention mixer: grouped queries (``heads``, ``kv_heads``; absent: as many key heads as query heads), query/key
heads of ``dim`` and value heads of ``vdim`` (absent: ``dim``), biases on all four projections, one RMS norm over all
query heads together and one over all key heads (weights ``q.norm``, ``k.norm``), rotate-half rotation of the first
``rot.dims`` channels of a head with base ``rot.base`` (absent: none), scores times ``scale``, a sliding window of
``mask.size`` keys (absent: none) and a learned score per head (``sink``) that enters the softmax's denominator
without a key or a value.  The mixture's router scores are sigmoids; the chosen scores multiply their experts'
inputs as they are.

Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1``, ``l<i>.mix.q`` (bias ``l<i>.mix.q.b``),
``l<i>.mix.q.norm``, ``l<i>.mix.sink``, ``l<i>.mlp.gate``, ``l<i>.mlp.e<j>.up``, ``l<i>.mlp.router``,
``l<i>.mlp.shared.down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .pugalix import _LIMIT, _freeze, _get, _int, _pos, _thaw
from .qwen3 import ConfigError
from .spec import (EmbeddingSpec, GatedAttentionSpec, HeadSpec, LayerSpec, ModelSpec, MoESpec, NoPositionSpec, RMSNormSpec,
                   ReinjectSpec, RotarySpec, ScheduleEntry, SwiGLUSpec)

MIXERS = ("attention",)


@dataclass(frozen=True)
class KalonexLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's keys, as read (nested dicts as tuples of pairs)
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def get(self, *path):
        node: Any = dict(self.mixer)
        for k in path:
            node = dict(node)[k]
        return node

    def has(self, key: str) -> bool:
        return key in dict(self.mixer)


@dataclass(frozen=True)
class KalonexConfig:
    width: int
    vocab: int
    norm_eps: float
    logit_scale: float
    loop: Optional[Tuple[int, int, int]]    # (start, stop, times) or None: every layer runs once
    layers: Tuple[KalonexLayer, ...]
    architecture: str = "Kalonex"

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KalonexConfig":
        width, vocab = _int(d, "width", ""), _int(d, "vocab", "")
        eps = _pos(_get(d, "norm", ""), "eps", "norm.")
        scale = 1.0
        if d.get("logit_scale") is not None:
            scale = d["logit_scale"]
            if isinstance(scale, bool) or not isinstance(scale, (int, float)) or not math.isfinite(float(scale)):
                raise ConfigError(f"config.json: 'logit_scale' must be a finite number, got {scale!r}")
            scale = float(scale)
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[KalonexLayer] = []
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
            if "kv_heads" in m and heads % _int(m, "kv_heads", ma):
                raise ConfigError(f"config.json: '{ma}heads' {heads} is not a multiple of '{ma}kv_heads' {m['kv_heads']}")
            _pos(m, "scale", ma)
            if "mask" in m:
                _int(_get(m, "mask", ma), "size", ma + "mask.")
            if "rot" in m:
                rot = _get(m, "rot", ma)
                dims = _int(rot, "dims", ma + "rot.", low=0)
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: '{ma}rot.dims' {dims} must be even and at most '{ma}dim' {dim}")
                _pos(rot, "base", ma + "rot.")
            mlp = raw.get("mlp") if isinstance(raw, dict) else None
            if mlp is not None:
                fa = at + "mlp."
                fk = _get(mlp, "kind", fa)
                if fk == "dense":
                    _int(mlp, "ff", fa)
                elif fk == "moe":
                    _int(_get(mlp, "expert", fa), "ff", fa + "expert.")
                    router = _get(mlp, "router", fa)
                    experts, top = _int(router, "experts", fa + "router."), _int(router, "top", fa + "router.")
                    if top > experts:
                        raise ConfigError(f"config.json: '{fa}router.top' {top} exceeds its {experts} experts")
                    if mlp.get("shared") is not None:
                        _int(mlp["shared"], "ff", fa + "shared.")
                else:
                    raise ConfigError(f"config.json: '{fa}kind' is {fk!r}; this design has dense and moe feed-forwards")
                mlp = {k: v for k, v in mlp.items() if v is not None}
            layers.append(KalonexLayer(kind, _freeze(m), None if mlp is None else _freeze(mlp)))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            start = _int(lp, "start", "loop.", low=0)
            stop, times = _int(lp, "stop", "loop."), _int(lp, "times", "loop.")
            if not start < stop <= len(layers):
                raise ConfigError(f"config.json: 'loop' runs layers {start} .. {stop} - 1 of {len(layers)}")
            loop = (start, stop, times)
        return cls(width=width, vocab=vocab, norm_eps=eps, logit_scale=scale, loop=loop, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Kalonex")))

    # ---- writing -------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out = {
            "architecture": self.architecture,
            "layers": [{"type": l.type, "mixer": _thaw(l.mixer), "mlp": None if l.mlp is None else _thaw(l.mlp)} for l in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def with_layers(self, n: int) -> "KalonexConfig":
        """The first ``n`` layers; a repeated stretch that reaches beyond them ends with them."""
        if not 0 < n <= len(self.layers):
            raise ValueError(f"layers={n} of a configuration with {len(self.layers)}")
        loop = self.loop
        if loop is not None:
            loop = (loop[0], min(loop[1], n), loop[2]) if loop[0] < n else None
        return KalonexConfig(self.width, self.vocab, self.norm_eps, self.logit_scale, loop, self.layers[:n], self.architecture)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def layer_runs(self) -> List[Tuple[int, int]]:
        """(layer, pass) in the order the layers run; pass -1 outside the repeated stretch."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, -1) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, -1) for i in range(start)]
        for t in range(times):
            runs += [(i, t) for i in range(start, stop)]
        return runs + [(i, -1) for i in range(stop, n)]

    # ---- derived -------------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = lambda: RMSNormSpec(size=W, eps=eps, tensor="")
        gated = lambda ff: SwiGLUSpec(hidden=W, intermediate=ff, names=("gate", "up", "down"))
        layers = []
        for i, l in enumerate(self.layers):
            heads, d = l.get("heads"), l.get("dim")
            position = (RotarySpec(head_dim=d, rotary_dim=l.get("rot", "dims"), theta=float(l.get("rot", "base")))
                        if l.has("rot") and l.get("rot", "dims") > 0 else NoPositionSpec(head_dim=d))
            mixer = GatedAttentionSpec(
                hidden=W, heads=heads, kv_heads=l.get("kv_heads") if l.has("kv_heads") else heads, head_dim=d,
                value_dim=l.get("vdim") if l.has("vdim") else d, scale=float(l.get("scale")), position=position,
                window=l.get("mask", "size") if l.has("mask") else 0, keep_first=0, sink=True, sink_learned=True, bias=True,
                out_bias=True, gate=False, qk_norm=RMSNormSpec(size=heads * d, eps=eps), qk_norm_span=True)
            ff = ff_norm = None
            if l.mlp is not None:
                mlp = _thaw(l.mlp)
                if mlp["kind"] == "dense":
                    ff = gated(mlp["ff"])
                else:
                    ff = MoESpec(hidden=W, experts=mlp["router"]["experts"], top=mlp["router"]["top"], intermediate=mlp["expert"]["ff"],
                                 score="sigmoid", renorm=False, weight_on="input", act="swiglu",
                                 shared=gated(mlp["shared"]["ff"]) if mlp.get("shared") is not None else None)
                ff_norm = norm()
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=norm(), feed_forward_norm=ff_norm,
                                    block="prenorm", mixer_prefix="mix.", feed_forward_prefix="mlp.", mixer_norm_prefix="norm1",
                                    feed_forward_norm_prefix="norm2"))
        schedule = []
        for i, t in self.layer_runs():
            enter = None
            if t >= 0 and i == self.loop[0]:
                enter = ReinjectSpec(hidden=W, passes=self.loop[2], index=t, weight="loop.in", steps="loop.step")
            schedule.append(ScheduleEntry(layer=i, enter=enter))
        spec = ModelSpec(
            architecture=self.architecture, hidden=W, vocab=self.vocab, max_positions=1 << 30,
            embedding=EmbeddingSpec("embed", self.vocab, W), layers=tuple(layers), schedule=tuple(schedule),
            # the head is linear, so the factor on the logits rides on the final norm's weight
            final_norm=RMSNormSpec(size=W, eps=eps, tensor="", gain=self.logit_scale), final_norm_name="final.norm",
            head=HeadSpec("head", self.vocab, W, tied_to=None))
        spec.validate()
        return spec
