"""The Kalonex design on the GPU against the plain implementation (tests/plain/kalonex_plain.py): each mechanism
alone, whole prompts against token-by-token decoding, prompts in portions down to two tokens, batches of unequal
requests, slots and pages that are used again, the edges of the window in prompts and in decoding, the first
tokens, keys far back, long decoding, odd sizes, the kernels by themselves, and greedy generation through the
entry point.  Every model here is made by the test (its own sizes, random weights that bfloat16 holds exactly)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.plain import kalonex_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(heads=4, kv_heads=2, dim=32, vdim=None, size=24, rot=16, base=100.0, scale=0.2, mlp=None):
    m = {"heads": heads, "dim": dim, "scale": scale}
    if kv_heads is not None:
        m["kv_heads"] = kv_heads
    if vdim is not None:
        m["vdim"] = vdim
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def config(layers, width=64, vocab=96, loop=None, logit_scale=0.7, eps=1e-5):
    cfg = {"architecture": "Kalonex", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


CONFIGS = {
    # each mechanism alone
    "attention": config([layer()]),
    "dense": config([layer(mlp=dense(96))]),
    "moe": config([layer(mlp=moe(6, 2, 24, shared=40))]),
    "loop": config([layer(mlp=dense(48))], loop=(0, 1, 3)),
    # all together: a repeated stretch in the middle, windows shorter and longer than a page, rotation of a part
    # of a head and of all of it, value heads of another size
    "mix": config([layer(mlp=dense(96)), layer(heads=6, kv_heads=3, dim=16, vdim=24, size=100, rot=16, scale=0.3, mlp=moe(5, 2, 40, shared=24)),
                   layer(mlp=None), layer(heads=2, kv_heads=1, dim=64, size=70, rot=32, base=5000.0, scale=0.12, mlp=moe(3, 1, 16)),
                   layer(mlp=dense(40))], loop=(1, 4, 2), logit_scale=1.3),
    # head sizes the tensor-core attention kernels take in bfloat16; one kv head for all heads; windows around a page
    "tensor": config([layer(heads=4, kv_heads=1, dim=128, size=70, rot=64, scale=0.09, mlp=dense(64)),
                      layer(heads=4, kv_heads=2, dim=64, size=64, rot=64, scale=0.12, mlp=moe(8, 1, 32, shared=64)),
                      layer(heads=6, kv_heads=2, dim=32, size=36, rot=8, mlp=moe(4, 2, 32)),
                      layer(heads=2, kv_heads=2, dim=96, size=129, rot=48, scale=0.1)], width=128, vocab=80, loop=(2, 4, 2), logit_scale=0.25),
    # what a file may leave out: no loop, no factor on the logits, no grouping, no window, no rotation, no shared
    # expert, values as wide as keys; sizes that are odd, equal or 1: one head, one expert of which one is used,
    # all experts used, a window of 1, a stretch that runs once, head sizes that are not multiples of 8
    "odd": config([layer(heads=3, kv_heads=None, dim=24, size=None, rot=None, scale=0.31, mlp=moe(1, 1, 56)),
                   layer(heads=1, kv_heads=1, dim=20, vdim=17, size=1, rot=20, scale=1.0),
                   layer(heads=6, kv_heads=1, dim=8, vdim=40, size=5, rot=2, scale=0.5, mlp=moe(3, 3, 8, shared=8)),
                   layer(heads=2, kv_heads=2, dim=12, size=200, rot=4, mlp=dense(24))], width=48, vocab=61, loop=None, logit_scale=None,
                  eps=1e-6),
    "once": config([layer(mlp=dense(40)), layer(size=7, mlp=moe(4, 2, 24))], loop=(0, 2, 1), width=40),
    "last": config([layer(mlp=dense(40)), layer(size=33, mlp=moe(4, 1, 24, shared=16))], loop=(1, 2, 3), width=40),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = P.random_weights(cfg, seed=170 + i)
        d = P.write_model(str(tmp_path_factory.mktemp(f"kalonex_{name}")), cfg, w)
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
    plain model where two scores nearly tie, and the rows that follow carry the difference."""
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
    toks = tokens_for(cfg, 1, 230)      # from 192 rows on the output projections run on the paired tensor-core kernel
    close(feed(engine_for(models, name, dtype), toks), P.forward(cfg, w, toks), TOL[dtype], MOST[dtype])


def test_the_residual_after_every_layer_run(models):
    import torch
    from gophonic_b200.parts.block import PreNormBlock
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", "float32", graphs=False)
    toks = tokens_for(cfg, 2, 70)
    seen, orig = [], PreNormBlock.forward

    def spy(self, batch, h, pending, cache, next_norm=None):
        out = orig(self, batch, h, pending, cache, next_norm=next_norm)
        seen.append((h + out if isinstance(out, torch.Tensor) else h).cpu().numpy())
        return out
    PreNormBlock.forward = spy
    try:
        feed(eng, toks)
    finally:
        PreNormBlock.forward = orig
    _, runs = P.forward(cfg, w, toks, return_layers=True)
    assert len(seen) == len(runs) == 8          # three layers twice, one before and one after
    for got, want in zip(seen, runs):
        close(got, want, 2e-5)


# ---- prompts against decoding, portions, batches ----------------------------------------------
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["mix", "odd", "tensor", "last"])
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
    """A sequence that takes over the slot and the pages of one that ended sees nothing of it, in any pass's cache."""
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
def test_long_decoding_past_windows_and_pages(models, name):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 5, 40 + 230)
    want = P.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        got = feed(engine_for(models, name, dtype), toks, cuts=[40] + [1] * 230)
        close(got, want, TOL[dtype], MOST[dtype])


# ---- the window's edge, a far key and the sink, through a whole model ---------------------------
def _standout_model(tmp_path, size, sink):
    """One layer whose attention picks out one far key: every query is one fixed direction u (its bias, with the
    projection scaled down), an ordinary key points anywhere, and the token ``mark`` has an embedding that the key
    projection turns into a key along u.  Whoever sees that token puts most of its weight on it; whoever does not,
    spreads it.  The sink is set low or high."""
    cfg = config([layer(heads=2, kv_heads=1, dim=16, size=size, rot=None, scale=0.5)], width=32, vocab=50, logit_scale=None)
    w = P.random_weights(cfg, seed=5)
    rng = np.random.default_rng(6)
    u = rng.standard_normal(16)
    u /= np.linalg.norm(u)
    w["l0.mix.q"] *= 0.02
    for n in ("q", "k"):
        w[f"l0.mix.{n}.norm"][:] = 1.0
    w["l0.mix.q.b"][:] = np.tile(2.0 * u, 2)       # every query is, after its norm, four times u
    w["l0.mix.k.b"][:] = 0.0                       # an ordinary key points anywhere
    mark = 7
    e = w["embed"][mark] / np.linalg.norm(w["embed"][mark])
    w["l0.mix.k"] += np.outer(u, e) * 3.0          # the marked token's key points along u
    w["l0.mix.sink"][:] = sink
    w = {k: P.from_bf16_bits(P.to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    return cfg, w, P.write_model(str(tmp_path), cfg, w), mark


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [37, 64, 65, 130, None])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path, size, dtype):
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    cfg, w, d, mark = _standout_model(tmp_path / "edge", size, sink=-4.0)
    rng = np.random.default_rng(8)
    toks = [int(t) for t in rng.integers(8, cfg["vocab"], size=300)]
    far = 3                                        # the marked token far back: at position 3
    toks[far] = mark
    want = P.forward(cfg, w, toks)
    if size is not None:
        inside, outside = far + size - 1, far + size
        # the plain model itself must tell the two positions apart by much more than the tolerance
        gone = P.forward(cfg, w, toks[:far] + [9] + toks[far + 1:])
        assert np.abs(want[inside] - gone[inside]).max() > 0.1 and np.abs(want[outside] - gone[outside]).max() < 1e-9
    else:
        gone = P.forward(cfg, w, toks[:far] + [9] + toks[far + 1:])
        assert np.abs(want[-1] - gone[-1]).max() > 0.05         # without a window the far key is still seen at the end
    eng = Engine(Model.from_dir(d, dtype=dtype), max_tokens=1024)
    tol = TOL[dtype] if dtype == "float32" else 3e-2
    close(feed(eng, toks), want, tol)                                          # in a prompt
    edge = far + (size or 200) - 2
    close(feed(eng, toks, cuts=[edge] + [1] * 6), want, tol)                   # decoded across the edge
    close(feed(eng, toks, cuts=[edge - 1, 2, 2, 2, 70]), want, tol)            # in portions across the edge


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share(tmp_path, dtype):
    """A sink of a high score takes most of the weight; the output shrinks accordingly.  Left out, counted twice or
    scaled like a key's score, it would show."""
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    cfg, w, d, mark = _standout_model(tmp_path / "sink", 50, sink=3.0)
    w["l0.mix.sink"][:] = [3.0, -1.0]
    d = P.write_model(d, cfg, w)
    toks = tokens_for(cfg, 12, 150)
    want = P.forward(cfg, w, toks)
    none = dict(w)
    none["l0.mix.sink"] = np.full(2, -30.0)
    assert np.abs(P.forward(cfg, none, toks) - want).max() > 0.2
    eng = Engine(Model.from_dir(d, dtype=dtype), max_tokens=512)
    tol = TOL[dtype] if dtype == "float32" else 3e-2
    close(feed(eng, toks), want, tol)
    close(feed(eng, toks, cuts=[100] + [1] * 50), want, tol)


# ---- the attention kernels by themselves: edges of the window, pages, key splits, the sink --------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 1, 16, 16, 37), (4, 4, 24, 24, 70), (3, 1, 8, 40, 64), (4, 2, 32, 32, 65), (2, 1, 64, 64, 1),
                                   (3, 3, 128, 128, 130), (2, 2, 16, 16, 0), (8, 2, 64, 64, 150), (2, 1, 128, 128, 300)])
def test_attention_kernels_with_a_learned_sink(shape, dtype):
    import torch
    from gophonic_b200 import ops
    heads, kv_heads, d, dv, window = shape
    T, scale = 330, 0.5
    rng = np.random.default_rng(sum(shape))
    q = 0.3 * rng.standard_normal((T, heads, d))
    k = 0.3 * rng.standard_normal((T, kv_heads, d))
    v = rng.standard_normal((T, kv_heads, dv))
    for i in range(window + 2, T, 7):          # one key stands out for some rows: at the window's edges, at page borders, at the start
        j = [i - window + 1, i - window, 0, 63, 64, 1, i, i - 1][(i // 7) % 8]
        if 0 <= j <= i:
            u = rng.standard_normal(d)
            u /= np.linalg.norm(u)
            k[j, :, :] = 6.0 * u
            q[i, :, :] = 4.0 * u
    sinks = 2.0 * rng.standard_normal(heads) + 1.0
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    ops.use_device(0)
    as_t = lambda a: torch.tensor(a, dtype=torch.float32).to(td).to(dev)
    qt, kt, vt = as_t(q), as_t(k), as_t(v)
    q, k, v = (t.float().cpu().numpy().astype(np.float64) for t in (qt, kt, vt))      # what the kernel sees
    want = P.sink_window_attention(q, k, v, scale, window or None, sinks)
    pages = (T + 63) // 64
    perm = [3, 0, 5, 1, 4, 2][:pages]                                                  # physical pages in another order
    k_plane = torch.zeros((pages, kv_heads, 64, d), dtype=td, device=dev)
    v_plane = torch.zeros((pages, kv_heads, 64, dv), dtype=td, device=dev)
    for lp, pp in enumerate(perm):
        n = min(64, T - lp * 64)
        k_plane[pp, :, :n] = kt[lp * 64:lp * 64 + n].transpose(0, 1)
        v_plane[pp, :, :n] = vt[lp * 64:lp * 64 + n].transpose(0, 1)
    table = torch.tensor([[0] * pages, perm], dtype=torch.int32, device=dev)
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device=dev)
    st = torch.tensor(sinks, dtype=torch.float32, device=dev)
    tol = 2e-5 if dtype == "float32" else 2e-2

    def run(rows, first, kv_len, splits=1, algo="auto"):
        qq = qt[first:first + rows].reshape(rows, heads * d).contiguous()
        out = torch.zeros((rows, heads * dv), dtype=td, device=dev)
        scratch = torch.zeros(ops.attention_scratch_floats(1, heads, dv, splits), dtype=torch.float32, device=dev) if splits > 1 else None
        used = ops.attention(qq, out, k_plane, v_plane, table, i32(1), i32(0), i32(rows), i32(kv_len), 1, rows, heads, kv_heads, d, scale,
                             window, splits, scratch, algo=algo, value_dim=dv, sinks=st)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy().reshape(rows, heads, dv)
        err = np.abs(got - want[first:first + rows]).max()
        assert err < tol, f"{used}: rows {first}..{first + rows}: {err:.3e}"
        return used

    used = {run(T, 0, T), run(130, 200, T), run(2, 201, 203), run(40, 0, 40)}
    for pos in (0, 1, 63, 64, 65, window, window + 1, 127, 128, 200, 329):
        if pos < T:
            used.add(run(1, pos, pos + 1))
            used.add(run(1, pos, pos + 1, splits=3))
    used.add(run(T, 0, T, algo="simt"))
    used.add(run(1, 300, 301, splits=4, algo="simt"))
    if dtype == "bfloat16" and d == dv and d % 16 == 0:
        assert used & {"decode_mma", "prefill_mma", "prefill_tc5"}, used     # the tensor-core kernels did run


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(3, 2, 8, 8, 4), (4, 1, 32, 16, 32), (8, 8, 128, 128, 128), (2, 1, 20, 17, 0), (5, 5, 16, 16, 2)])
def test_norm_over_the_projection_rotation_and_cache_write(shape, dtype):
    """The row-wise kernel in its whole-projection form against the plain functions, rows of several sequences at
    scattered positions and pages."""
    import torch
    from gophonic_b200 import ops
    heads, kv_heads, d, dv, rot = shape
    rng = np.random.default_rng(sum(shape) + 1)
    positions = [0, 1, 63, 64, 65, 130, 5]
    seqs = [0, 0, 0, 1, 1, 1, 2]
    rows = len(positions)
    nq, nk, nv = heads * d, kv_heads * d, kv_heads * dv
    x = rng.standard_normal((rows, nq + nk + nv + 3))
    bq, bk, bv = rng.standard_normal(nq), rng.standard_normal(nk), rng.standard_normal(nv)
    wq, wk = 1 + 0.3 * rng.standard_normal(nq), 1 + 0.3 * rng.standard_normal(nk)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    ops.use_device(0)
    xt = torch.tensor(x, dtype=torch.float32).to(td).to(dev)
    x = xt.float().cpu().numpy().astype(np.float64)
    eps, base = 1e-5, 50.0
    qn = P.rms_norm(x[:, :nq] + bq, wq, eps).reshape(rows, heads, d)
    kn = P.rms_norm(x[:, nq:nq + nk] + bk, wk, eps).reshape(rows, kv_heads, d)
    vn = (x[:, nq + nk:nq + nk + nv] + bv).reshape(rows, kv_heads, dv)
    want_q = np.stack([P.rotate_half(qn[r:r + 1], [positions[r]], rot, base)[0] for r in range(rows)]) if rot else qn
    want_k = np.stack([P.rotate_half(kn[r:r + 1], [positions[r]], rot, base)[0] for r in range(rows)]) if rot else kn
    f32 = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    cos = sin = None
    if rot:
        ang = np.arange(256)[:, None] * base ** (-2.0 * np.arange(rot // 2) / rot)[None, :]
        cos, sin = f32(np.cos(ang)), f32(np.sin(ang))
    pages = 9
    table = i32([[7, 2, 5], [1, 8, 0], [3, 4, 6]])
    k_plane = torch.zeros((pages, kv_heads, 64, d), dtype=td, device=dev)
    v_plane = torch.zeros((pages, kv_heads, 64, dv), dtype=td, device=dev)
    ops.qk_norm_rope_kv_write(xt, heads, kv_heads, d, f32(wq), f32(wk), eps, cos, sin, rot, i32(positions), i32(seqs), i32([2, 0, 1]),
                              table, k_plane, v_plane, True, biases=(f32(bq), f32(bk), f32(bv)), value_dim=dv, span=True)
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == "float32" else 2e-2
    got_q = xt[:, :nq].float().cpu().numpy().reshape(rows, heads, d)
    assert np.abs(got_q - want_q).max() < tol * max(1.0, np.abs(want_q).max())
    assert np.array_equal(xt[:, nq + nk + nv:].float().cpu().numpy(), x[:, nq + nk + nv:])       # what follows q, k, v is left alone
    slots = [2, 0, 1]
    tb = table.cpu().numpy()
    for r in range(rows):
        page = tb[slots[seqs[r]], positions[r] // 64]
        gk = k_plane[page, :, positions[r] % 64].float().cpu().numpy()
        gv = v_plane[page, :, positions[r] % 64].float().cpu().numpy()
        assert np.abs(gk - want_k[r]).max() < tol * max(1.0, np.abs(want_k).max())
        assert np.abs(gv - vn[r]).max() < tol * max(1.0, np.abs(vn).max())
    assert int((k_plane != 0).any(-1).sum()) == rows * kv_heads                                   # nothing else was written


# ---- the mixture in all its row ranges ---------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 3, 16, 17, 100, 230])
@pytest.mark.parametrize("sizes", [(6, 2, 24, 40), (12, 1, 48, None), (3, 3, 8, 16), (5, 4, 32, 8)])
def test_mixture_rows(rows, sizes, dtype):
    """The part by itself against the plain mixture: sigmoid scores as weights on the experts' inputs, gated
    experts, a shared expert, in the ranges of rows that take different paths."""
    import torch
    from types import SimpleNamespace
    from gophonic_b200 import ops
    from gophonic_b200.config.spec import MoESpec, SwiGLUSpec
    from gophonic_b200.parts.base import Runtime
    from gophonic_b200.parts.moe import MoE
    experts, top, ff, shared = sizes
    W = 64
    mlp = moe(experts, top, ff, shared)
    cfg = config([layer(mlp=mlp)], width=W)
    w = {k[len("l0.mlp."):]: v for k, v in P.random_weights(cfg, seed=rows + experts).items() if k.startswith("l0.mlp.")}
    w["router"] = w["router"] * 4.0            # scores that differ: weights between 0 and 1 that matter
    w = {k: P.from_bf16_bits(P.to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    ops.use_device(0)
    rng = np.random.default_rng(rows)
    xt = torch.tensor(rng.standard_normal((rows, W)), dtype=torch.float32).to(td).to(dev)
    x = xt.float().cpu().numpy().astype(np.float64)
    want = P.mixture(x, w, "", mlp)
    spec = MoESpec(hidden=W, experts=experts, top=top, intermediate=ff, score="sigmoid", renorm=False, weight_on="input", act="swiglu",
                   shared=None if shared is None else SwiGLUSpec(hidden=W, intermediate=shared, names=("gate", "up", "down")))
    tensors = {k: torch.tensor(v, dtype=torch.float32).to(td).to(dev) for k, v in w.items()}
    part = MoE(spec, "", tensors, Runtime(device=dev, act_dtype=td, ops=ops))
    out = torch.zeros((rows, W), dtype=torch.float32, device=dev)
    part.forward(SimpleNamespace(), xt, out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    if dtype == "float32":
        close(got, want, 2e-5)
    else:
        # a row whose last chosen score nearly ties with the next may take another expert in bfloat16
        s = np.sort(P.sigmoid(x @ w["router"].T), axis=-1)[:, ::-1]
        sure = np.ones(rows, bool) if top == experts else (s[:, top - 1] - s[:, top]) > 0.02
        if sure.any():
            close(got[sure], want[sure], 3e-2)


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 72, 40, [0, 3, 130, 0, 257]), (3, 300, 64, [1, 128, 129]), (7, 128, 200, [40, 0, 0, 9, 300, 64, 2]),
                                   (1, 8, 8, [5]), (4, 520, 152, [127, 1, 256, 70])])
def test_products_of_groups_of_rows_in_one_launch(shape, out_dtype):
    """Rows sorted by group, every group times its own block of the weights (blocks of rows, gated blocks with a
    weight a row, blocks of columns, rows written through a map), against one float64 product a group.  Groups that
    are empty, smaller and larger than a tile, ending one row before and after a tile's edge."""
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    dev = torch.device("cuda:0")
    groups, N, K, counts = shape
    assert len(counts) == groups
    rng = np.random.default_rng(N + K)
    P_rows = sum(counts)
    bf = lambda a: torch.tensor(a, dtype=torch.float32).to(torch.bfloat16).to(dev)
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    td = torch.float32 if out_dtype == "float32" else torch.bfloat16
    tol = 2e-3 if out_dtype == "float32" else 1.2e-2
    a = bf(rng.standard_normal((P_rows + 3, K)))[:P_rows]            # rows beyond the last group exist and are not used
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=dev)
    lo = np.concatenate([[0], np.cumsum(counts)])
    # blocks of rows
    w = bf(rng.standard_normal((groups * N, K)) / np.sqrt(K))
    out = torch.full((P_rows, N), 7.0, dtype=td, device=dev)
    ops.gemm_grouped(a, w, out, offsets, groups)
    want = np.concatenate([f64(a[lo[e]:lo[e + 1]]) @ f64(w[e * N:(e + 1) * N]).T for e in range(groups)])
    close(out.float().cpu().numpy(), want, tol)
    # gated blocks (N gate rows, then N up rows) with a weight on every row's input
    wg = bf(rng.standard_normal((groups * 2 * N, K)) / np.sqrt(K))
    f = torch.tensor(rng.uniform(0.2, 1.0, size=P_rows), dtype=torch.float32, device=dev)
    for weights in (f, None):
        out = torch.full((P_rows, N), 7.0, dtype=td, device=dev)
        ops.gemm_grouped(a, wg, out, offsets, groups, gated=True, row_weight=weights)
        rows = []
        for e in range(groups):
            x = f64(a[lo[e]:lo[e + 1]]) * (1.0 if weights is None else f64(f[lo[e]:lo[e + 1]])[:, None])
            g, u = x @ f64(wg[e * 2 * N:e * 2 * N + N]).T, x @ f64(wg[e * 2 * N + N:(e + 1) * 2 * N]).T
            rows.append(g * P.sigmoid(g) * u)
        close(out.float().cpu().numpy(), np.concatenate(rows), tol)
    # blocks of columns, rows written through a map (a permutation into a taller output)
    wc = bf(rng.standard_normal((N, groups * K)) / np.sqrt(K))
    perm = torch.tensor(rng.permutation(P_rows + 2)[:P_rows], dtype=torch.int32, device=dev)
    want = np.concatenate([f64(a[lo[e]:lo[e + 1]]) @ f64(wc[:, e * K:(e + 1) * K]).T for e in range(groups)])
    out = torch.full((P_rows, N), 7.0, dtype=td, device=dev)
    ops.gemm_grouped(a, wc, out, offsets, groups, by_cols=True)
    close(out.float().cpu().numpy(), want, tol)
    out = torch.full((P_rows + 2, N), 7.0, dtype=td, device=dev)
    ops.gemm_grouped(a, wc, out, offsets, groups, by_cols=True, row_map=perm)
    got = out.float().cpu().numpy()
    close(got[perm.cpu().numpy()], want, tol)
    untouched = np.setdiff1d(np.arange(P_rows + 2), perm.cpu().numpy())
    assert (got[untouched] == 7.0).all()
    assert ops.tc5_status() == 0


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
    cfg, w, d = models["last"]
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
    r = run("-random-config", "kalonex-tiny", "-weights-seed", "4", "-write-model", str(out))
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = P.read_model(str(out))
    assert cfg["architecture"] == "Kalonex" and {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
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
