"""A plain, slow Kalonex decoder in numpy float64: whole sequences, no cache, one function for each
mechanism.  It is the oracle of the Kalonex tests and shares no code with ``gophonic_b200``.

Kalonex is a pre-norm decoder whose middle layers may run several times with the same weights.  Every layer
has windowed grouped-query attention (biased projections, one RMS norm over all query heads together and
one over all key heads, rotate-half rotation of a part of each head, a learned sink per head in the
softmax's denominator) and, optionally, a dense gated feed-forward or a mixture of experts whose router
scores are sigmoids that multiply the chosen experts' inputs, with a shared expert beside them.  Before each
pass through the repeated layers the residual is mixed with the embedding output and a vector of the pass
is added.  The logits are multiplied by one number.

Everything takes the weights as a dict name -> float64 array and the configuration as the parsed
config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import numpy as np

from .pugalix_plain import from_bf16_bits, read_model, to_bf16_bits, write_model  # noqa: F401  (file helpers of the tests)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


# ---- attention -----------------------------------------------------------------------------------
def rotate_half(x, positions, dims: int, base: float):
    """x: [T, heads, d].  Channel i of a head turns with channel i + dims / 2, i < dims / 2, by the angle
    position * base^(-2 i / dims); channels from ``dims`` on pass."""
    out = x.copy()
    half = dims // 2
    for t, p in enumerate(positions):
        for i in range(half):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


def sink_window_attention(q, k, v, scale, size, sinks, first_pos: int = 0):
    """q: [T, H, d], k: [N, G, d], v: [N, G, dv]; row t stands at position first_pos + t and sees the keys
    j <= its position with position - j < size (None: all of them).  Head h's denominator also holds
    exp(sinks[h])."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        i = first_pos + t
        lo = 0 if size is None else max(0, i - size + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[t, h]) * scale
            m = max(float(s.max()), float(sinks[h]))
            e = np.exp(s - m)
            out[t, h] = (e @ v[lo:i + 1, g]) / (e.sum() + math.exp(float(sinks[h]) - m))
    return out


def attention_mixer(h, w, p, m, eps, first_pos: int = 0):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", d)
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)      # over all heads at once
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, d)
    positions = np.arange(first_pos, first_pos + T)
    if "rot" in m:
        q = rotate_half(q, positions, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_half(k, positions, m["rot"]["dims"], m["rot"]["base"])
    size = m["mask"]["size"] if "mask" in m else None
    o = sink_window_attention(q, k, v.reshape(T, G, dv), m["scale"], size, w[p + "sink"], first_pos)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


# ---- feed-forwards -------------------------------------------------------------------------------
def gated_feed_forward(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, top: int):
    """The chosen experts of every row (the lower index of equal scores first) and their weights: the
    sigmoid scores themselves."""
    s = sigmoid(h @ w[p + "router"].T)
    index = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return index, np.take_along_axis(s, index, axis=-1)


def mixture(h, w, p, mlp):
    top = mlp["router"]["top"]
    index, weight = route(h, w, p, top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(index[t, j])
            out[t] += gated_feed_forward(weight[t, j] * h[t:t + 1], w, f"{p}e{e}.")[0]     # the weight on the input
    if mlp.get("shared") is not None:
        out += gated_feed_forward(h, w, p + "shared.")
    return out


# ---- the model -----------------------------------------------------------------------------------
def layer_runs(cfg: dict) -> List[Tuple[int, int]]:
    """(layer, pass or -1) in the order the layers run; a pass's first entry is where the residual is mixed."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, -1) for i in range(n)]
    runs = [(i, -1) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, -1) for i in range(loop["stop"], n)]


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, return_layers: bool = False):
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)]
    x = x0.copy()
    after = []
    loop = cfg.get("loop")
    for i, t in layer_runs(cfg):
        if t >= 0 and i == loop["start"]:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T + w["loop.step"][t]
        L, p = cfg["layers"][i], f"l{i}."
        x = x + attention_mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            hh = rms_norm(x, w[p + "norm2"], eps)
            x = x + (gated_feed_forward(hh, w, p + "mlp.") if mlp["kind"] == "dense" else mixture(hh, w, p + "mlp.", mlp))
        after.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, np.stack(after)) if return_layers else logits


# ---- test models ---------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, d = m["heads"], m["dim"]
        G, dv = m.get("kv_heads", H), m.get("vdim", d)
        out[p + "norm1"] = (W,)
        out.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                    p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,),
                    p + "mix.sink": (H,), p + "mix.o": (W, H * dv), p + "mix.o.b": (W,)})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)

        def gated(q, ff):
            out.update({q + "gate": (ff, W), q + "up": (ff, W), q + "down": (W, ff)})
        if mlp["kind"] == "dense":
            gated(p + "mlp.", mlp["ff"])
        else:
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                gated(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared") is not None:
                gated(p + "mlp.shared.", mlp["shared"]["ff"])
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Random weights whose values bfloat16 holds exactly: matrices of deviation 1/sqrt(inputs), norm weights
    near 1, biases, sinks and pass vectors that matter."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "sink":
            v = 1.0 + rng.standard_normal(shape)
        elif last == "b" or name == "loop.step":
            v = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        elif name == "loop.in":
            v = rng.standard_normal(shape) / math.sqrt(shape[-1] / 2)
        elif last == "router":
            v = 2.0 * rng.standard_normal(shape) / math.sqrt(shape[-1])
        else:
            v = rng.standard_normal(shape) / math.sqrt(shape[-1])
        w[name] = from_bf16_bits(to_bf16_bits(v)).reshape(shape)
    return w


def greedy_generate(cfg, w, prompt, n: int) -> Tuple[List[int], List[float]]:
    """``n`` greedy tokens after ``prompt`` and, for each, the margin of its logit over the runner-up."""
    ids, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = forward(cfg, w, ids)[-1]
        order = np.argsort(logits)
        out.append(int(order[-1]))
        margins.append(float(logits[order[-1]] - logits[order[-2]]))
        ids.append(out[-1])
    return out, margins
