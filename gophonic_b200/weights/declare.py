"""The list of tensors a model resolves, gathered from its parts' declarations."""
from __future__ import annotations

from typing import List

from .. import registry
from ..parts.base import TensorDecl


def final_norm_prefix(spec) -> str:
    """The prefix under which the final norm resolves its tensor: the tensor's full name less the
    suffix the norm's spec names (``weight`` unless the spec says otherwise)."""
    name, suffix = spec.final_norm_name, getattr(spec.final_norm, "tensor", "weight")
    if not name.endswith(suffix):
        raise ValueError(f"final norm tensor name '{name}' must end in '{suffix}'")
    return name[:len(name) - len(suffix)]


def declare_model(spec) -> List[TensorDecl]:
    """Every tensor of ``spec`` by checkpoint name: embedding, each layer's parts (each layer once,
    however often the schedule runs it), final norm, and the head (optional when it can be tied)."""
    from .. import parts  # noqa: F401  (registers the built-in parts)
    decls: List[TensorDecl] = [TensorDecl(spec.embedding.name, (spec.embedding.vocab, spec.embedding.hidden),
                                          role="embedding")]
    for layer in spec.layers:
        decls += registry.part_class("block", layer.block).declare(layer)
    # what the schedule's junctions resolve; positions that name the same tensor share it
    named = {d.name for d in decls}
    for entry in spec.schedule:
        enter = getattr(entry, "enter", None)
        if enter is not None:
            for d in registry.part_class("junction", enter.kind).declare(enter, ""):
                if d.name not in named:
                    named.add(d.name)
                    decls.append(d)
    decls += registry.part_class("norm", spec.final_norm.kind).declare(spec.final_norm, final_norm_prefix(spec))
    decls.append(TensorDecl(spec.head.name, (spec.head.vocab, spec.head.hidden), role="matrix",
                            optional=spec.head.tied_to is not None))
    seen = set()
    for d in decls:
        if d.name in seen:
            raise ValueError(f"tensor '{d.name}' is declared twice")
        seen.add(d.name)
    return decls
