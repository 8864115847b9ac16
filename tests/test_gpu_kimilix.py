"""The Kimilix design on the GPU against the plain implementation (tests/plain/kimilix_plain.py): each mechanism
alone, whole prompts against token-by-token decoding, prompts in portions down to two tokens, batches of unequal
requests, slots and pages that are used again, the edges of blocks and windows in prompts and in decoding, the first
tokens, keys far back, long decoding, odd sizes, the kernels by themselves, and greedy generation through the
entry point.  Every model here is made by the test (its own sizes, random weights that bfloat16 holds exactly)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.plain import kimilix_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCALING = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}     # short enough that all three ranges of wavelengths occur


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None, limit=1.5):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared, "limit": limit * 0.8}
    return m


def diff(heads=4, kv_heads=2, dim=16, vdim=24, size=40, rot=8, base=100.0, scale=0.3, d=0.25, scaling=None, mlp=None):
    m = {"heads": heads, "dim": dim, "scale": scale, "diff": d}
    if kv_heads is not None:
        m["kv_heads"] = kv_heads
    if vdim is not None:
        m["vdim"] = vdim
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, size=30, base=1000.0, scale=0.25, scaling=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if vdim is not None:
        m["vdim"] = vdim
    if size is not None:
        m["mask"] = {"size": size}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(layers, width=64, vocab=96, mult=0.4, emb=0.7, eps=1e-5):
    cfg = {"architecture": "Kimilix", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if mult is not None:
        cfg["residual_mult"] = mult
    if emb is not None:
        cfg["embedding"] = {"scale": emb}
    return cfg


CONFIGS = {
    # each mechanism alone
    "diff": config([diff(scaling=SCALING)]),
    "latent": config([latent()]),
    "dense": config([latent(mlp=dense(96))]),
    "moe": config([diff(mlp=moe(6, 2, 24, shared=40))]),
    # all together: blocks and windows shorter and longer than a page, rotation of a part of a map and of all of it
    "mix": config([latent(mlp=dense(80)), diff(mlp=moe(5, 2, 40, shared=24)), latent(heads=2, dim=24, rot_dim=16, vdim=8, q_rank=24, kv_rank=48,
                                                                                    size=100, scaling=SCALING, mlp=moe(4, 3, 16, shared=32)),
                   diff(heads=6, kv_heads=1, dim=8, vdim=16, size=70, rot=8, scale=0.4, d=0.6, mlp=None),
                   diff(heads=2, kv_heads=2, dim=32, vdim=32, size=130, rot=16, scaling=SCALING, mlp=dense(40))]),
    # sizes the tensor-core kernels take in bfloat16: maps of 128 and 64, latents that are multiples of 16
    "tensor": config([diff(heads=2, kv_heads=1, dim=128, vdim=128, size=70, rot=64, scale=0.09, mlp=dense(64)),
                      latent(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=96, kv_rank=128, size=64, scale=0.1, mlp=moe(8, 2, 32, shared=64)),
                      diff(heads=4, kv_heads=2, dim=64, vdim=64, size=64, rot=64, scale=0.12, mlp=moe(4, 1, 32)),
                      latent(heads=2, dim=32, rot_dim=64, vdim=32, q_rank=64, kv_rank=64, size=129, scale=0.1)], width=128, vocab=80),
    # what a file may leave out (no grouping, values as wide as keys, no mask, no rotation, no shared expert, no factors)
    # and sizes that are odd, equal or 1: one head, one expert, all experts used, a block and a window of one position
    "odd": config([diff(heads=3, kv_heads=None, dim=12, vdim=None, size=None, rot=None, scale=0.31, d=0.0, mlp=moe(1, 1, 56)),
                   latent(heads=1, dim=20, rot_dim=0, vdim=None, q_rank=7, kv_rank=9, size=None, scale=1.0),
                   diff(heads=1, kv_heads=1, dim=20, vdim=17, size=1, rot=20, scale=1.0, d=0.9),
                   latent(heads=5, dim=6, rot_dim=2, vdim=10, q_rank=48, kv_rank=5, size=1, mlp=moe(3, 3, 8, shared=8)),
                   diff(heads=2, kv_heads=2, dim=10, vdim=6, size=200, rot=4, mlp=dense(24))], width=48, vocab=61, mult=None, emb=None, eps=1e-6),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = P.random_weights(cfg, seed=270 + i)
        d = P.write_model(str(tmp_path_factory.mktemp(f"kimilix_{name}")), cfg, w)
        out[name] = (cfg, w, d)
    return out


_engines = {}


def engine_for(models, name, dtype, graphs=True, max_tokens=4096):
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    key = (name, dtype, graphs, max_tokens)
    if key not in _engines:
        _engines[key] = Engine(Model.from_dir(models[name][2], dtype=dtype), max_tokens=max_tokens, use_graphs=graphs)
    return _engines[key]


def tokens_for(cfg, seed, n):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def feed(engine, tokens, cuts=None):
    """All logits of one sequence fed in portions of the sizes ``cuts`` (the rest in one piece)."""
    slot = engine.new_sequence()
    out, at = [], 0
    sizes = list(cuts or []) + [len(tokens)]
    for n in sizes:
        n = min(n, len(tokens) - at)
        if n <= 0:
            break
        out.append(engine.step([(slot, tokens[at:at + n])], [list(range(n))]).cpu().numpy())
        at += n
    engine.end_sequence(slot)
    engine.check_kernels()
    return np.concatenate(out)


def close(got, want, tol, most=1.0):
    """Every row within ``tol`` (relative to the largest wanted value); with ``most`` < 1 that share of the rows
    must be, and the rest within five times as much: in bfloat16 a router may take another expert than the
    plain model where two logits nearly tie, and the rows that follow carry the difference."""
    scale = max(1.0, np.abs(want).max())
    err = np.abs(got - want).reshape(got.shape[0], -1).max(-1) / scale
    if most >= 1.0:
        assert err.max() < tol, f"relative error {err.max():.3e} (tolerance {tol})"
    else:
        assert (err < tol).mean() >= most and err.max() < 5 * tol, f"{(err >= tol).sum()} of {len(err)} rows over {tol}, worst {err.max():.3e}"


TOL = {"float32": 3e-5, "bfloat16": 6e-2}
MOST = {"float32": 1.0, "bfloat16": 0.95}


# ---- each mechanism alone, and all together ---------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts_match_the_plain_model(models, name, dtype):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 1, 230)
    close(feed(engine_for(models, name, dtype), toks), P.forward(cfg, w, toks), TOL[dtype], MOST[dtype])


def test_the_residual_after_every_layer(models):
    from gophonic_b200.parts.postnorm import PostNormBlock
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", "float32", graphs=False)
    toks = tokens_for(cfg, 2, 70)
    seen, orig = [], PostNormBlock.forward

    def spy(self, batch, h, pending, cache):
        out = orig(self, batch, h, pending, cache)
        seen.append(h.cpu().numpy())
        return out
    PostNormBlock.forward = spy
    try:
        feed(eng, toks)
    finally:
        PostNormBlock.forward = orig
    _, layers = P.forward(cfg, w, toks, return_layers=True)
    assert len(seen) == len(layers) == 5
    for got, want in zip(seen, layers):
        close(got, want, 2e-5)


# ---- prompts against decoding, portions, batches ----------------------------------------------
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["mix", "odd", "tensor"])
def test_token_by_token_equals_the_whole_prompt(models, name, graphs):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, "float32", graphs=graphs)
    toks = tokens_for(cfg, 3, 90)
    whole = feed(eng, toks)
    single = feed(eng, toks, cuts=[1] * len(toks))
    close(single, whole, 2e-5)
    close(single, P.forward(cfg, w, toks), TOL["float32"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "odd", "tensor"])
@pytest.mark.parametrize("cuts", [[2] * 40, [3, 64, 1, 2, 61], [63, 1, 1, 64], [130, 2]])
def test_portions_of_a_prompt(models, cuts, dtype, name):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, dtype)
    toks = tokens_for(cfg, 4, 140)
    got = feed(eng, toks, cuts=cuts)
    close(got, P.forward(cfg, w, toks), TOL[dtype], MOST[dtype])
    if dtype == "float32":
        close(got, feed(eng, toks), 2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "tensor"])
def test_a_batch_of_unequal_requests_equals_each_alone(models, dtype, name):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, dtype)
    prompts = [tokens_for(cfg, 10 + i, n) for i, n in enumerate([1, 70, 9, 33])]
    more = [tokens_for(cfg, 20 + i, 12) for i in range(4)]
    slots = [eng.new_sequence() for _ in prompts]
    got = [[] for _ in prompts]
    first = eng.step(list(zip(slots, prompts)), [list(range(len(p))) for p in prompts]).cpu().numpy()
    at = 0
    for i, p in enumerate(prompts):
        got[i].append(first[at:at + len(p)])
        at += len(p)
    live = list(range(len(prompts)))
    for t in range(12):
        if t == 5:                      # one request ends early; the others go on
            eng.end_sequence(slots[live.pop(1)])
        logits = eng.step([(slots[i], [more[i][t]]) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
    for i in live:
        eng.end_sequence(slots[i])
    eng.cache.check()
    for i, p in enumerate(prompts):
        n = 12 if i != 1 else 5
        close(np.concatenate(got[i]), P.forward(cfg, w, p + more[i][:n]), TOL[dtype], MOST[dtype])


def test_slots_and_pages_that_are_used_again(models):
    """A sequence that takes over the slot and the pages of one that ended sees nothing of it."""
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", "float32", max_tokens=256)     # four pages: the second sequence must reuse them
    a, b = tokens_for(cfg, 30, 200), tokens_for(cfg, 31, 130)
    close(feed(eng, a, cuts=[100]), P.forward(cfg, w, a), TOL["float32"])
    assert eng.cache.pages.held() == 0
    close(feed(eng, b, cuts=[64, 1, 1]), P.forward(cfg, w, b), TOL["float32"])
    s1 = eng.new_sequence()
    eng.step([(s1, a[:50])])
    eng.end_sequence(s1)
    s2 = eng.new_sequence()
    assert s2 == s1
    got = eng.step([(s2, b[:2])], [[0, 1]]).cpu().numpy()          # the first tokens of a sequence
    got = np.concatenate([got, eng.step([(s2, b[2:20])], [list(range(18))]).cpu().numpy()])
    eng.end_sequence(s2)
    close(got, P.forward(cfg, w, b[:20]), TOL["float32"])


@pytest.mark.parametrize("name", ["mix", "tensor", "odd"])
def test_long_decoding_past_blocks_windows_and_pages(models, name):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 5, 40 + 230)
    want = P.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        got = feed(engine_for(models, name, dtype), toks, cuts=[40] + [1] * 230)
        close(got, want, TOL[dtype], MOST[dtype])


# ---- a block's and a window's edge and a far key, through a whole model --------------------------
def _standout(tmp_path, kind, size):
    """One layer whose attention picks out one key.  Every embedding row carries the same large share along one
    direction a, from which the query projection makes queries along a fixed direction u (so every row asks for u);
    the token ``mark`` has an embedding that the key path turns into a key along u, ordinary tokens' keys point
    anywhere.  Whoever sees the marked token puts most of its weight on it; whoever does not, spreads it."""
    rng = np.random.default_rng(6)
    mark, width = 7, 32
    u = rng.standard_normal(16)
    u /= np.linalg.norm(u)
    a = rng.standard_normal(width)
    a /= np.linalg.norm(a)
    if kind == "diff":
        cfg = config([diff(heads=2, kv_heads=1, dim=16, vdim=16, size=size, rot=None, scale=0.5, d=0.2)], width=width, vocab=50)
    else:
        cfg = config([latent(heads=2, dim=16, rot_dim=0, vdim=16, q_rank=24, kv_rank=16, size=size, scale=0.25)], width=width, vocab=50)
    w = P.random_weights(cfg, seed=5)
    e = w["embed"][mark] - (w["embed"][mark] @ a) * a         # what only the marked token has much of
    e /= np.linalg.norm(e)
    w["embed"] += 4.0 * a
    if kind == "diff":
        w["l0.mix.k.norm"][:] = 1.0
        w["l0.mix.q.norm"][:] = 1.0
        w["l0.mix.k"] -= np.outer(w["l0.mix.k"] @ a, a)       # keys do not see the common share
        w["l0.mix.k"][:16] += np.outer(u, e) * 6.0            # map 1 of the key group: the marked token's key points along u
        w["l0.mix.q"] *= 0.05
        w["l0.mix.q"][0:16] += np.outer(u, a)                 # map 1 of head 0: every query points along u
    else:
        w["l0.mix.dkv.norm"][:] = 1.0
        w["l0.mix.dq.norm"][:] = 1.0
        w["l0.mix.dkv"] -= np.outer(w["l0.mix.dkv"] @ a, a)
        w["l0.mix.dkv"] *= 0.3
        w["l0.mix.dkv"] += np.outer(u, e) * 2.0               # the marked token's latent points along u
        w["l0.mix.uk"][:16] = np.eye(16) * 2.0                # head 0 reads the latent as its key
        w["l0.mix.dq"] *= 0.05
        w["l0.mix.dq"][0] = a                                 # the first latent channel of every query is large and positive
        w["l0.mix.uq"][:16] = 0.0
        w["l0.mix.uq"][:16, 0] = 1.5 * u                      # head 0's queries point along u
    w = {k: P.from_bf16_bits(P.to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    return cfg, w, P.write_model(str(tmp_path), cfg, w), mark


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [37, 64, 65, 130, None])
@pytest.mark.parametrize("kind", ["diff", "latent"])
def test_a_key_just_inside_and_just_outside_a_block_or_window(tmp_path, kind, size, dtype):
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    cfg, w, d, mark = _standout(tmp_path / "edge", kind, size)
    rng = np.random.default_rng(8)
    toks = [int(t) for t in rng.integers(8, cfg["vocab"], size=300)]
    # the marked token: the first of a block (seen up to the block's last position) or a position far back
    far = (size if kind == "diff" else 3) if size is not None else 3
    toks[far] = mark
    want = P.forward(cfg, w, toks)
    gone = P.forward(cfg, w, toks[:far] + [9] + toks[far + 1:])
    if size is not None:
        inside, outside = far + size - 1, far + size
        # the plain model itself must tell the two positions apart by much more than the tolerance
        assert np.abs(want[inside] - gone[inside]).max() > 0.05 and np.abs(want[outside] - gone[outside]).max() < 1e-9
    else:
        inside = 299
        assert np.abs(want[-1] - gone[-1]).max() > 0.02          # without a mask the far key is still seen at the end
    eng = Engine(Model.from_dir(d, dtype=dtype), max_tokens=1024)
    tol = TOL[dtype] if dtype == "float32" else 3e-2
    close(feed(eng, toks), want, tol)                                          # in a prompt
    edge = inside - 1
    close(feed(eng, toks, cuts=[edge] + [1] * 6), want, tol)                   # decoded across the edge
    close(feed(eng, toks, cuts=[edge - 1, 2, 2, 2, 70]), want, tol)            # in portions across the edge
    close(feed(eng, toks, cuts=[far + 1, 1, 1]), want, tol)                    # the first tokens behind the marked one


# ---- the attention kernels by themselves: edges, pages, key splits, shared values, values inside the keys ----
def _plain_masked(q, k, v, scale, window, chunk, share):
    """q [T, H, d], k [T, G, d], v [T, G / share, dv]: softmax attention, row i over j <= i inside the window and the block."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    mask = j <= i
    if window:
        mask &= i - j < window
    if chunk:
        mask &= i // chunk == j // chunk
    for h in range(H):
        g = h // (H // G)
        out[:, h] = P.softmax_attention(q[:, h], k[:, g], v[:, g // share], scale, mask)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [  # heads, kv heads, d, dv, window, chunk, key heads a value head, values inside the keys
    (4, 2, 16, 24, 0, 37, 2, False), (8, 4, 32, 32, 0, 64, 2, False), (4, 4, 128, 128, 0, 130, 2, False), (2, 2, 64, 64, 0, 65, 2, False),
    (6, 2, 8, 40, 0, 1, 1, False), (4, 2, 64, 64, 50, 128, 2, False), (4, 1, 96, 64, 70, 0, 1, True), (3, 1, 40, 33, 0, 0, 1, True),
    (8, 1, 160, 128, 64, 0, 1, True), (2, 1, 576, 512, 100, 0, 1, True)])
def test_attention_kernels_with_blocks_shared_values_and_values_inside_the_keys(shape, dtype):
    import torch
    from gophonic_b200 import ops
    heads, kv_heads, d, dv, window, chunk, share, in_keys = shape
    T, scale = 330, 0.5 if d < 100 else 0.1
    rng = np.random.default_rng(sum(shape[:6]))
    q = 0.3 * rng.standard_normal((T, heads, d))
    k = 0.3 * rng.standard_normal((T, kv_heads, d))
    v = rng.standard_normal((T, kv_heads // share, dv))
    size = chunk or window or 100
    for i in range(2, T, 7):          # one key stands out for some rows: at the edges of blocks and windows, at page borders, at the start
        j = [i - window + 1 if window else i - i % size, i - window if window else i - i % size - 1, 0, 63, 64, 1, i, i - 1][(i // 7) % 8]
        if 0 <= j <= i:
            u = rng.standard_normal(d)
            u /= np.linalg.norm(u)
            k[j, :, :] = (6.0 if d < 100 else 12.0) * u
            q[i, :, :] = (4.0 if d < 100 else 8.0) * u
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    ops.use_device(0)
    as_t = lambda a: torch.tensor(a, dtype=torch.float32).to(td).to(dev)
    qt, kt = as_t(q), as_t(k)
    vt = kt[:, :, :dv].contiguous() if in_keys else as_t(v)
    q, k, v = (t.float().cpu().numpy().astype(np.float64) for t in (qt, kt, vt))      # what the kernel sees
    want = _plain_masked(q, k, v, scale, window, chunk, share)
    pages = (T + 63) // 64
    perm = [3, 0, 5, 1, 4, 2][:pages]                                                  # physical pages in another order
    k_plane = torch.zeros((pages, kv_heads, 64, d), dtype=td, device=dev)
    v_plane = k_plane[..., :dv] if in_keys else torch.zeros((pages, kv_heads // share, 64, dv), dtype=td, device=dev)
    for lp, pp in enumerate(perm):
        n = min(64, T - lp * 64)
        k_plane[pp, :, :n] = kt[lp * 64:lp * 64 + n].transpose(0, 1)
        if not in_keys:
            v_plane[pp, :, :n] = vt[lp * 64:lp * 64 + n].transpose(0, 1)
    table = torch.tensor([[0] * pages, perm], dtype=torch.int32, device=dev)
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device=dev)
    tol = 2e-5 if dtype == "float32" else 2e-2

    def run(rows, first, kv_len, splits=1, algo="auto"):
        qq = qt[first:first + rows].reshape(rows, heads * d).contiguous()
        out = torch.zeros((rows, heads * dv), dtype=td, device=dev)
        scratch = torch.zeros(ops.attention_scratch_floats(1, heads, dv, splits), dtype=torch.float32, device=dev) if splits > 1 else None
        used = ops.attention(qq, out, k_plane, v_plane, table, i32(1), i32(0), i32(rows), i32(kv_len), 1, rows, heads, kv_heads, d, scale,
                             window, splits, scratch, algo=algo, value_dim=dv, chunk=chunk, v_share=share)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy().reshape(rows, heads, dv)
        err = np.abs(got - want[first:first + rows]).max()
        assert err < tol, f"{used}: rows {first}..{first + rows}: {err:.3e}"
        return used

    used = {run(T, 0, T), run(130, 200, T), run(2, 201, 203), run(40, 0, 40)}
    for pos in (0, 1, 63, 64, 65, size - 1, size, size + 1, 127, 128, 200, 2 * size, 329):
        if pos < T:
            used.add(run(1, pos, pos + 1))
            used.add(run(1, pos, pos + 1, splits=3))
    used.add(run(T, 0, T, algo="simt"))
    used.add(run(1, 300, 301, splits=4, algo="simt"))
    if dtype == "bfloat16" and in_keys and d % 16 == 0 and dv in (64, 128, 256, 512):
        assert "latent_mma" in used, used                                   # the tensor-core kernel for latents did run
    if dtype == "bfloat16" and not in_keys and d == dv and d % 16 == 0:
        assert used & {"decode_mma", "prefill_mma", "prefill_tc5"}, used     # the tensor-core kernels did run


# ---- the row-wise kernels by themselves ------------------------------------------------------------
@pytest.mark.parametrize("width", [48, 256, 2048, 2500])
@pytest.mark.parametrize("out_dtype", [None, "float32", "bfloat16"])
def test_norm_behind_a_sublayer_added_into_the_residual(width, out_dtype):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    rng = np.random.default_rng(width)
    rows, eps = 37, 1e-3
    h, y, w = rng.standard_normal((rows, width)), 3.0 * rng.standard_normal((rows, width)), 1.0 + 0.3 * rng.standard_normal(width)
    dev = torch.device("cuda:0")
    ht, yt, wt = (torch.tensor(a, dtype=torch.float32, device=dev) for a in (h, y, w))
    h, y, w = (t.double().cpu().numpy() for t in (ht, yt, wt))
    want = h + P.unit_rms(y, eps) * w
    x = None if out_dtype is None else torch.zeros((rows, width), dtype=getattr(torch, out_dtype), device=dev)
    ops.norm_scale_add(ht, yt, wt, eps, x)
    torch.cuda.synchronize()
    assert np.abs(ht.double().cpu().numpy() - want).max() < 2e-5
    if x is not None:
        assert np.abs(x.double().cpu().numpy() - want).max() < (2e-5 if out_dtype == "float32" else 4e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(4, 2, 24), (6, 1, 16), (3, 3, 40), (1, 1, 7), (8, 4, 128)])
def test_the_two_maps_combined(shape, dtype):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    heads, groups, dv = shape
    per = heads // groups
    rows, lam, eps, factor = 19, 0.37, 1e-4, 0.8
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(sum(shape))
    maps = torch.tensor(rng.standard_normal((rows, groups, 2, per, dv)), dtype=torch.float32).to(td).cuda()
    m = maps.double().cpu().numpy()
    o = m[:, :, 0] - lam * m[:, :, 1]                       # [rows, groups, per, dv]: the model's head order
    want = (P.unit_rms(o, eps) * factor).reshape(rows, heads * dv)
    out = torch.zeros((rows, heads * dv), dtype=td, device="cuda:0")
    ops.diff_combine(maps.reshape(rows, -1), out, heads, per, dv, lam, eps, factor)
    torch.cuda.synchronize()
    assert np.abs(out.double().cpu().numpy() - want).max() < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(24, 16, 8), (300, 70, 2), (7, 9, 0), (768, 512, 64)])
def test_latent_norms_rotation_and_cache_write(shape, dtype):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    Q, R, dr = shape
    rows, eps, base = 70, 1e-5, 50.0
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(Q + R)
    lat = torch.tensor(rng.standard_normal((rows, Q + R + dr + 3)), dtype=torch.float32).to(td).to(dev)       # wider than what is used
    qw, kw = (torch.tensor(1.0 + 0.2 * rng.standard_normal(n), dtype=torch.float32, device=dev) for n in (Q, R))
    positions = [5 + 2 * r for r in range(rows)]           # one sequence whose rows stand at scattered positions
    freqs = P.rotary_frequencies(dr, base) if dr else np.zeros(0)
    ang = np.arange(256)[:, None] * freqs[None, :]
    cos, sin = (torch.tensor(f(ang), dtype=torch.float32, device=dev) for f in (np.cos, np.sin)) if dr else (None, None)
    pages = 4
    k_plane = torch.zeros((pages, 1, 64, R + dr), dtype=td, device=dev)
    table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=dev)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    cq = torch.zeros((rows, Q), dtype=td, device=dev)
    ops.latent_prep(lat, cq, qw, kw, eps, cos, sin, Q, R, dr, i32(positions), i32([0] * rows), i32([0]), table, k_plane, True)
    torch.cuda.synchronize()
    x = lat.double().cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert np.abs(cq.double().cpu().numpy() - P.unit_rms(x[:, :Q], eps) * qw.double().cpu().numpy()).max() < tol
    c = P.unit_rms(x[:, Q:Q + R], eps) * kw.double().cpu().numpy()
    kr = P.rotate(x[:, Q + R:Q + R + dr].reshape(rows, 1, dr), positions, freqs, "pairs")[:, 0] if dr else np.zeros((rows, 0))
    phys = [2, 0, 3, 1]
    got = np.stack([k_plane[phys[p // 64], 0, p % 64].double().cpu().numpy() for p in positions])
    assert np.abs(got - np.concatenate([c, kr], axis=-1)).max() < tol
    held = {(phys[p // 64], p % 64) for p in positions}
    untouched = [k_plane[pg, 0, t].abs().max().item() for pg in range(pages) for t in range(64) if (pg, t) not in held]
    assert max(untouched) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 3, 16, 24), (9, 2, 128, 512), (33, 5, 7, 130), (8, 16, 512, 128)])
def test_a_product_for_every_head_in_one_launch(shape, dtype):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    rows, heads, K, N = shape
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(sum(shape))
    a = torch.tensor(rng.standard_normal((rows, heads, K + 5)), dtype=torch.float32).to(td).cuda()      # a view: rows wider than K
    w = torch.tensor(rng.standard_normal((heads, K, N)) / np.sqrt(K), dtype=torch.float32).to(td).cuda()
    out = torch.zeros((rows, heads, N + 3), dtype=td, device="cuda:0")
    ops.head_gemm(a[:, :, :K], w, out[:, :, :N])
    torch.cuda.synchronize()
    want = np.einsum("rhk,hkn->rhn", a[:, :, :K].double().cpu().numpy(), w.double().cpu().numpy())
    assert np.abs(out[:, :, :N].double().cpu().numpy() - want).max() < (3e-5 if dtype == "float32" else 3e-2)
    assert out[:, :, N:].abs().max().item() == 0.0


@pytest.mark.parametrize("shape", [(70, 3, 16, 24), (300, 2, 128, 512), (65, 5, 72, 130), (200, 16, 512, 128), (33, 1, 136, 7)])
def test_a_product_for_every_head_on_the_tensor_cores(shape):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    rows, heads, K, N = shape
    rng = np.random.default_rng(sum(shape))
    a = torch.tensor(rng.standard_normal((rows, heads, K + 8)), dtype=torch.float32).to(torch.bfloat16).cuda()      # a view: rows wider than K
    w = torch.tensor(rng.standard_normal((heads, N, K)) / np.sqrt(K), dtype=torch.float32).to(torch.bfloat16).cuda()
    out = torch.zeros((rows, heads, N + 2 + (N & 1)), dtype=torch.bfloat16, device="cuda:0")      # even strides
    assert ops.head_gemm_mma_accepts(a[:, :, :K], w, out[:, :, :N])
    ops.head_gemm_mma(a[:, :, :K], w, out[:, :, :N])
    torch.cuda.synchronize()
    want = np.einsum("rhk,hnk->rhn", a[:, :, :K].double().cpu().numpy(), w.double().cpu().numpy())
    assert np.abs(out[:, :, :N].double().cpu().numpy() - want).max() < 3e-2
    assert out[:, :, N:].abs().max().item() == 0.0
    assert not ops.head_gemm_mma_accepts(a[:, :, 1:K + 1], w, out[:, :, :N])      # rows that do not start on 16 bytes


def test_the_scaled_rotation_tables():
    """All three ranges of wavelengths (kept, blended, divided) in one table, against the plain frequencies."""
    import torch
    from gophonic_b200.config.spec import PairRotarySpec, RotarySpec
    from gophonic_b200.engine.model import make_runtime
    from gophonic_b200.parts.rope import PairRotaryEmbedding, RotaryEmbedding
    rt = make_runtime("float32", "cuda:0")
    sc = (8.0, 1.0, 4.0, 200.0)
    want = P.rotary_frequencies(32, 3000.0, dict(zip(("factor", "low", "high", "original"), sc)))
    plain = P.rotary_frequencies(32, 3000.0)
    assert (want == plain).any() and (np.isclose(want, plain / 8.0)).any() and ((want < plain * 0.999) & (want > plain / 8.0 * 1.001)).any()
    for cls, spec in ((RotaryEmbedding, RotarySpec(head_dim=48, rotary_dim=32, theta=3000.0, scaling=sc)),
                      (PairRotaryEmbedding, PairRotarySpec(head_dim=32, rotary_dim=32, theta=3000.0, scaling=sc))):
        part = cls(spec, "", {}, rt)
        part.prepare(300)
        cos, sin, rot = part.kernel_args()
        ang = np.arange(300)[:, None] * want[None, :]
        assert rot == 32 and np.abs(cos.cpu().numpy() - np.cos(ang)).max() < 1e-6 and np.abs(sin.cpu().numpy() - np.sin(ang)).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 3, 16, 17, 100, 230])
@pytest.mark.parametrize("sizes", [(6, 2, 24, 40), (12, 1, 48, None), (3, 3, 8, 16), (5, 4, 32, 8)])
def test_mixture_rows(rows, sizes, dtype):
    """The mixture part by itself in every range of rows (few rows reading only the chosen experts, the stacked
    products, the products grouped by expert) against the plain mixture."""
    import torch
    from gophonic_b200.config.spec import ClampedGLUSpec, MoESpec
    from gophonic_b200.engine.model import make_runtime
    from gophonic_b200.parts.moe import MoE
    experts, top, ff, shared = sizes
    hidden, limit = 64, 1.2
    mlp = moe(experts, top, ff, shared, limit=limit)
    cfg = config([diff(mlp=mlp)], width=hidden)
    w = {k[len("l0.mlp."):]: v for k, v in P.random_weights(cfg, seed=rows + experts).items() if k.startswith("l0.mlp.")}
    rt = make_runtime(dtype, "cuda:0")
    spec = MoESpec(hidden=hidden, experts=experts, top=top, intermediate=ff, renorm_eps=0.0, act="glu_clamp", act_limit=limit, act_slope=1.702,
                   router_bias=True, shared=None if shared is None else ClampedGLUSpec(hidden, shared, limit * 0.8, 1.702), shared_gate=shared is not None)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = {k: torch.tensor(v, dtype=torch.float32).to(td).cuda() for k, v in w.items()}
    part = MoE(spec, "", tensors, rt)
    rng = np.random.default_rng(rows)
    x = torch.tensor(rng.standard_normal((rows, hidden)), dtype=torch.float32).to(td).cuda()
    out = torch.zeros((rows, hidden), dtype=torch.float32, device="cuda:0")

    class Batch:
        pass
    part.forward(Batch(), x, out)
    torch.cuda.synchronize()
    want = P.mixture(x.double().cpu().numpy(), w, "", mlp)
    close(out.cpu().numpy(), want, 3e-5 if dtype == "float32" else 4e-2, MOST[dtype])


# ---- generation through the entry point, the trace program, the command line ----------------------
def test_greedy_generation_through_the_entry_point(models):
    import gophonic_b200 as g
    cfg, w, d = models["mix"]
    prompts = [tokens_for(cfg, 40, 9), tokens_for(cfg, 41, 1), tokens_for(cfg, 42, 75)]
    model = g.Open(d, g.Options(Format=g.FormatF32, CacheTokens=2048, Batch=4))
    got = g.Lane(model, g.TokensGenerator).Generate(prompts, g.ChatOptions(MaxTokens=10))
    model.Close()
    for p, out in zip(prompts, got):
        want, margins = P.greedy_generate(cfg, w, p, 10)
        for a, b, m in zip(out, want, margins):
            if m < 1e-3:
                break           # a near-tie of the plain logits: from here on either token is right
            assert a == b


def test_trace_program_on_a_folder(models, tmp_path):
    cfg, w, d = models["mix"]
    a, b = tokens_for(cfg, 50, 70), tokens_for(cfg, 51, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": []}, {"id": "b", "tokens": b[3:4], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": [0]}, {"id": "b", "tokens": b[4:5], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:70], "want": [1]}], "end": ["a"]}]
    out = tmp_path / "out"
    for dtype in ("float32", "bfloat16"):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                           timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        wa, wb = P.forward(cfg, w, a), P.forward(cfg, w, b)
        read = lambda n: np.fromfile(str(out / f"{n}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        close(read(0), np.stack([wa[0], wa[65], wb[2]]), TOL[dtype], MOST[dtype])
        close(read(1), wb[3:4], TOL[dtype], MOST[dtype])
        close(read(2), np.stack([wa[67], wb[4]]), TOL[dtype], MOST[dtype])
        close(read(3), wa[69:70], TOL[dtype], MOST[dtype])


def test_the_command_line_writes_and_runs_a_named_configuration(tmp_path):
    """-random-config NAME -write-model DIR, then -model DIR: the plain model reads the written folder
    and would have chosen the same tokens."""
    out = tmp_path / "written"
    run = lambda *a: subprocess.run([sys.executable, "-m", "gophonic_b200", *a], cwd=ROOT, capture_output=True, text=True, timeout=600)
    r = run("-random-config", "kimilix-tiny", "-weights-seed", "4", "-write-model", str(out))
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = P.read_model(str(out))
    assert cfg["architecture"] == "Kimilix" and {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
    r = run("-model", str(out), "-format", "f32", "-max-tokens", "6", "3,9,27", "100")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["prompt"] for l in lines] == [[3, 9, 27], [100]]
    for l in lines:
        ids = list(l["prompt"])
        assert len(l["tokens"]) == 6
        for t in l["tokens"]:
            logits = P.forward(cfg, w, ids)[-1]
            assert logits.max() - logits[t] <= 1e-5
            ids.append(t)
