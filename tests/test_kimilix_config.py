"""The Kimilix configuration without a GPU: reading config.json, the registry, the declared tensors, the constants
the specs carry, what a file may leave out, refusals, random weights, the frequencies of a stretched rotation, and
the cache's storage (one value head for two key heads; values that are channels of the keys)."""
import copy
import json

import numpy as np
import pytest
import torch

from tests.plain import kimilix_plain as P
from tests.test_gpu_kimilix import CONFIGS, SCALING


def test_the_registry_finds_the_design_by_its_name(tmp_path):
    from gophonic_b200 import registry
    from gophonic_b200.config import KimilixConfig
    cfg = CONFIGS["mix"]
    assert registry.architecture_of(cfg) == "Kimilix"
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    read = registry.read_config(str(tmp_path))
    assert isinstance(read, KimilixConfig) and read.num_layers == len(cfg["layers"])
    assert read.to_dict() == cfg                                       # nothing lost, nothing added
    assert KimilixConfig.from_dict(read.to_dict()) == read
    assert read.with_layers(3).to_dict()["layers"] == cfg["layers"][:3]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from gophonic_b200.config import KimilixConfig
    from gophonic_b200.weights import declare_model
    cfg = CONFIGS[name]
    decls = declare_model(KimilixConfig.from_dict(cfg).model_spec())
    assert {d.name: tuple(d.shape) for d in decls if not d.optional} == P.tensor_shapes(cfg)
    assert [d.name for d in decls if d.optional] == ["head"]          # the head is the embedding table


def test_the_spec_carries_the_designs_constants():
    from gophonic_b200.config import KimilixConfig
    spec = KimilixConfig.from_dict(CONFIGS["mix"]).model_spec()
    assert spec.head.tied_to == "embed" and spec.embedding.scale == 0.7 and spec.final_norm.offset == 1.0
    assert all(l.block == "postnorm" and l.residual_mult == 0.4 and l.mixer_norm.offset == 1.0 for l in spec.layers)
    a = spec.layers[1].mixer
    assert a.kind == "diff_attention" and (a.heads, a.kv_heads, a.head_dim, a.value_dim, a.chunk, a.window) == (4, 2, 16, 24, 40, 0)
    assert (a.scale, a.lambda_init, a.eps, a.qk_norm.eps, a.qk_norm.size) == (0.3, 0.25, 1e-5, 1e-5, 16)
    assert a.position.kind == "rope" and (a.position.rotary_dim, a.position.theta, a.position.scaling) == (8, 100.0, None)
    assert spec.layers[4].mixer.position.scaling == (4.0, 1.0, 3.0, 64.0)
    b = spec.layers[2].mixer
    assert b.kind == "latent_attention" and (b.heads, b.head_dim, b.rot_dim, b.value_dim, b.q_rank, b.kv_rank, b.window, b.chunk) == (2, 24, 16, 8, 24, 48, 100, 0)
    assert b.position.kind == "rope_pairs" and (b.position.rotary_dim, b.position.scaling) == (16, (4.0, 1.0, 3.0, 64.0))
    f = spec.layers[1].feed_forward
    assert f.kind == "moe" and (f.experts, f.top, f.intermediate, f.act, f.act_limit, f.act_slope) == (5, 2, 40, "glu_clamp", 1.5, 1.702)
    assert (f.score, f.renorm, f.renorm_eps, f.weight_on, f.router_bias, f.shared_gate) == ("softmax", True, 0.0, "output", True, True)
    assert f.shared.kind == "glu_clamp" and (f.shared.intermediate, f.shared.limit, f.shared.slope) == (24, 1.5 * 0.8, 1.702)
    assert spec.layers[3].feed_forward is None and spec.layers[0].feed_forward.kind == "relu2_ff"


def test_what_a_file_leaves_out_is_not_there():
    from gophonic_b200.config import KimilixConfig
    cfg = KimilixConfig.from_dict(CONFIGS["odd"])
    spec = cfg.model_spec()
    bare = spec.layers[0].mixer
    assert (bare.kv_heads, bare.value_dim, bare.chunk, bare.window) == (3, 12, 0, 0) and bare.position.kind == "none"
    assert cfg.embedding_scale == 1.0 and cfg.residual_mult == 1.0
    lat = spec.layers[1].mixer
    assert (lat.rot_dim, lat.value_dim, lat.window) == (0, 20, 0) and lat.position.kind == "none"
    f = spec.layers[0].feed_forward
    assert f.shared is None and not f.shared_gate


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="gla"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][4]["mixer"]["rot"]["scaling"].update(high=1.0), "high"),
    (lambda c: c.update(residual_mult="big"), "residual_mult"),
])
def test_a_wrong_file_is_refused(change, message):
    from gophonic_b200.config import ConfigError, KimilixConfig
    cfg = copy.deepcopy(CONFIGS["mix"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        KimilixConfig.from_dict(cfg)


def test_random_weights_write_a_model_the_plain_reader_takes(tmp_path):
    from gophonic_b200.config import KimilixConfig
    from gophonic_b200.weights import write_random_model
    cfg = CONFIGS["mix"]
    d = write_random_model(KimilixConfig.from_dict(cfg), seed=1, out_dir=str(tmp_path / "m"))
    read, w = P.read_model(d)
    assert {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
    assert abs(w["l0.norm1"]).max() < 0.5 and abs(w["l1.mix.q.norm"] - 1).max() < 0.5 and abs(w["l1.ls2"] - 1).max() < 0.5
    assert np.isfinite(P.forward(read, w, [1, 2, 3])).all()


def test_stretched_frequencies_against_the_plain_ones():
    from gophonic_b200.parts.rope import scaled_frequencies
    for dims, base in ((8, 100.0), (32, 3000.0), (64, 1e6)):
        plain = P.rotary_frequencies(dims, base)
        sc = (SCALING["factor"], SCALING["low"], SCALING["high"], SCALING["original"])
        got = scaled_frequencies(plain.copy(), sc)
        assert np.allclose(got, P.rotary_frequencies(dims, base, SCALING), rtol=1e-14, atol=0)
        assert np.array_equal(scaled_frequencies(plain.copy(), None), plain)
    f = P.rotary_frequencies(32, 3000.0, SCALING)
    p = P.rotary_frequencies(32, 3000.0)
    assert (f == p).any() and np.isclose(f, p / 4.0).any() and ((f < p * 0.999) & (f > p / 4.0 * 1.001)).any()     # all three ranges occur


def test_the_cache_keeps_values_once():
    """Differential attention: two key heads a value head.  Latent attention: no value plane at all, the values are
    the first channels of the keys."""
    from gophonic_b200.cache import Cache
    from gophonic_b200.config import KimilixConfig
    from gophonic_b200 import parts, registry  # noqa: F401
    spec = KimilixConfig.from_dict(CONFIGS["mix"]).model_spec()
    reqs = [(registry.part_class("block", spec.layers[e.layer].block).cache_request(spec.layers[e.layer]), e.cache_of) for e in spec.schedule]
    cache = Cache(reqs, max_tokens=256, device="cpu", dtype=torch.float32, max_slots=2)
    d = cache.view(1)                          # 4 heads over 2 key groups of two maps of 16, values of 24
    assert tuple(d.k.shape[1:]) == (4, 64, 16) and tuple(d.v.shape[1:]) == (2, 64, 24)
    l = cache.view(2)                          # a latent of 48 and 16 rotated channels
    assert tuple(l.k.shape[1:]) == (1, 64, 64) and tuple(l.v.shape[1:]) == (1, 64, 48)
    assert l.v.data_ptr() == l.k.data_ptr() and l.v.stride(2) == 64
    per_token = {(g["kv_heads"], g["head_dim"]): g["bytes_per_token"] // len(g["planes"]) for g in cache.groups() if g["kind"] == "kv"}
    assert per_token[(4, 16)] == 4 * (4 * 16 + 2 * 24) and per_token[(1, 64)] == 4 * 64
    assert len({cache.view(i).k.data_ptr() for i in range(5)}) == 5
    slot = cache.alloc_slot()
    cache.reserve([(slot, 70)])
    cache.commit([(slot, 70)])
    cache.free_slot(slot)
    cache.check()
