"""A plain, slow Kimilix decoder in numpy float64: whole sequences, no cache, one function for each
mechanism.  It is the oracle of the Kimilix tests and shares no code with ``gophonic_b200``.

Kimilix is a decoder whose sublayers read the residual x itself and whose norms stand behind the sublayers:

    x <- x + mult * scale1 * norm1(mixer(x)),    x <- x + mult * scale2 * norm2(feed_forward(x))

with norm(y) = y / sqrt(mean(y^2) + eps) * (1 + w) and a vector ``scale`` per sublayer.  A layer's mixer is
differential attention over chunks (two softmax maps per head that share the values, the second taken off
the first with a learned factor) or latent attention through a sliding window (queries, keys and values
made from low-rank latents, one rotated key part shared by the heads).  Its feed-forward is a dense one
with a squared relu or a mixture of clamped gated experts with a gated shared expert.  The embedding is
multiplied by a constant; the head is the embedding table.

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


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def one_plus_norm(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


# ---- rotations -----------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling=None) -> np.ndarray:
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` {factor, low, high, original} a frequency whose
    wavelength 2 pi / f is longer than original/low is divided by factor, one shorter than original/high stays,
    and between the two the divided and the plain frequency are blended linearly in original/wavelength."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    if not scaling:
        return f
    factor, low, high, orig = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < orig / high:
            continue
        if wave > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, freqs, layout: str):
    """x: [T, heads, d]; the first 2 len(freqs) channels of every head turn.  layout "half": channel i with
    channel i + n; "pairs": channel 2i with channel 2i + 1 (n = len(freqs)); the pair (u, v) at position p
    becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i."""
    n = len(freqs)
    out = x.copy()
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    if layout == "half":
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n], out[..., n:2 * n] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2], out[..., 1:2 * n:2] = u * c - v * s, v * c + u * s
    return out


# ---- masks and softmax attention -----------------------------------------------------------------
def visible(kind: str, size: int, T: int) -> np.ndarray:
    """[T, T] booleans: may row i see key j.  "chunk": j <= i in the same block of ``size`` positions counted
    from 0; "window": 0 <= i - j < size; ``size`` None: every j <= i."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    if size is None:
        return j <= i
    if kind == "chunk":
        return (j <= i) & (i // size == j // size)
    return (j <= i) & (i - j < size)


def softmax_attention(q, k, v, scale, mask):
    """q: [T, d], k: [T, d], v: [T, dv], mask [T, T] -> [T, dv]."""
    s = (q @ k.T) * scale
    s = np.where(mask, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)) @ v


# ---- mixers --------------------------------------------------------------------------------------
def differential_lambda(w, p, diff):
    return math.exp(float(w[p + "lq1"] @ w[p + "lk1"])) - math.exp(float(w[p + "lq2"] @ w[p + "lk2"])) + diff


def differential_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", d)
    q = (h @ w[p + "q"].T).reshape(T, H * 2, d)        # head by head, [map 1, map 2]
    k = (h @ w[p + "k"].T).reshape(T, G * 2, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot and rot["dims"] > 0:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate(q, np.arange(T), f, "half"), rotate(k, np.arange(T), f, "half")
    mask = visible("chunk", m["mask"]["size"] if "mask" in m else None, T)
    lam = differential_lambda(w, p, m["diff"])
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        a1 = softmax_attention(q[:, 2 * hd], k[:, 2 * g], v[:, g], m["scale"], mask)
        a2 = softmax_attention(q[:, 2 * hd + 1], k[:, 2 * g + 1], v[:, g], m["scale"], mask)
        out[:, hd] = unit_rms(a1 - lam * a2, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dr, R = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    dv = m.get("vdim", d)
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + dr)
    ckv = h @ w[p + "dkv"].T
    c = unit_rms(ckv[:, :R], eps) * w[p + "dkv.norm"]
    k_rot, q_rot = ckv[:, R:], q[:, :, d:]
    if dr > 0:
        f = rotary_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
        pos = np.arange(T)
        k_rot = rotate(k_rot.reshape(T, 1, dr), pos, f, "pairs")[:, 0]
        q_rot = rotate(q_rot, pos, f, "pairs")
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    mask = visible("window", m["mask"]["size"] if "mask" in m else None, T)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        qq = np.concatenate([q[:, hd, :d], q_rot[:, hd]], axis=-1)
        kk = np.concatenate([k_plain[:, hd], k_rot], axis=-1)
        out[:, hd] = softmax_attention(qq, kk, v[:, hd], m["scale"], mask)
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- feed-forwards -------------------------------------------------------------------------------
def squared_relu_feed_forward(h, w, p):
    return (np.maximum(h @ w[p + "up"].T, 0.0) ** 2) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, top: int):
    """The ``top`` experts with the largest logits of every row (the lower index of equal ones first) and the
    softmax over those logits alone."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    index = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, index, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return index, e / e.sum(axis=-1, keepdims=True)


def mixture(h, w, p, mlp):
    top = mlp["router"]["top"]
    index, weight = route(h, w, p, top)
    out = np.zeros_like(h)
    limit = mlp["expert"]["limit"]
    for e in range(mlp["router"]["experts"]):
        rows, js = np.nonzero(index == e)
        if len(rows):
            out[rows] += weight[rows, js][:, None] * clamped_expert(h[rows], w, f"{p}e{e}.", limit)
    if mlp.get("shared") is not None:
        out += sigmoid(h @ w[p + "shared.sg"].T) * clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# ---- the model -----------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, return_layers: bool = False):
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][np.asarray(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    after = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = differential_attention if L["type"] == "attention" else latent_attention
        x = x + mult * w[p + "ls1"] * one_plus_norm(mix(x, w, p + "mix.", L["mixer"], eps), w[p + "norm1"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            y = squared_relu_feed_forward(x, w, p + "mlp.") if mlp["kind"] == "dense" else mixture(x, w, p + "mlp.", mlp)
            x = x + mult * w[p + "ls2"] * one_plus_norm(y, w[p + "norm2"], eps)
        after.append(x.copy())
    logits = one_plus_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, np.stack(after)) if return_layers else logits


# ---- test models ---------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        out[p + "ls1"] = (W,)
        H, d = m["heads"], m["dim"]
        dv = m.get("vdim", d)
        if L["type"] == "attention":
            G = m.get("kv_heads", H)
            out.update({p + "mix.q": (H * 2 * d, W), p + "mix.k": (G * 2 * d, W), p + "mix.v": (G * dv, W), p + "mix.q.norm": (d,),
                        p + "mix.k.norm": (d,), p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,),
                        p + "mix.o": (W, H * dv)})
        else:
            R, Q, dr = m["kv_rank"], m["q_rank"], m["rot_dim"]
            out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (d + dr), Q), p + "mix.dkv": (R + dr, W),
                        p + "mix.dkv.norm": (R,), p + "mix.uk": (H * d, R), p + "mix.uv": (H * dv, R), p + "mix.o": (W, H * dv)})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        out[p + "ls2"] = (W,)

        def gated(q, ff):
            out.update({q + "gate": (ff, W), q + "up": (ff, W), q + "down": (W, ff)})
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            E = mlp["router"]["experts"]
            out[p + "mlp.router"] = (E, W)
            out[p + "mlp.router.b"] = (E,)
            for e in range(E):
                gated(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared") is not None:
                gated(p + "mlp.shared.", mlp["shared"]["ff"])
                out[p + "mlp.shared.sg"] = (1, W)
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Random weights whose values bfloat16 holds exactly: matrices of deviation 1/sqrt(inputs), norm
    weights (stored less one) and sublayer scales that matter, router biases that move the choice."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            v = 0.2 * rng.standard_normal(shape)
        elif last == "norm":
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last in ("ls1", "ls2"):
            v = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            v = 0.3 * rng.standard_normal(shape)
        elif last == "b":
            v = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        elif last == "router":
            v = 2.0 * rng.standard_normal(shape) / math.sqrt(shape[-1])
        elif last in ("q", "k", "uq", "uk"):
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
