"""The Kalonex configuration without a GPU: reading config.json, the registry, the declared tensors, the schedule
of a repeated stretch with its junctions, what a file may leave out, refusals, random weights, and a cache plane
of its own for every pass."""
import copy
import json

import numpy as np
import pytest
import torch

from tests.plain import kalonex_plain as P
from tests.test_gpu_kalonex import CONFIGS


def test_the_registry_finds_the_design_by_its_name(tmp_path):
    from gophonic_b200 import registry
    from gophonic_b200.config import KalonexConfig
    cfg = CONFIGS["mix"]
    assert registry.architecture_of(cfg) == "Kalonex"
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    read = registry.read_config(str(tmp_path))
    assert isinstance(read, KalonexConfig) and read.num_layers == len(cfg["layers"])
    assert read.to_dict() == cfg                                       # nothing lost, nothing added
    assert KalonexConfig.from_dict(read.to_dict()) == read
    cut = read.with_layers(3)
    assert cut.to_dict()["layers"] == cfg["layers"][:3] and cut.loop == (1, 3, 2)      # the stretch ends with the layers
    assert read.with_layers(1).loop is None


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from gophonic_b200.config import KalonexConfig
    from gophonic_b200.weights import declare_model
    cfg = CONFIGS[name]
    decls = declare_model(KalonexConfig.from_dict(cfg).model_spec())
    assert {d.name: tuple(d.shape) for d in decls} == P.tensor_shapes(cfg)
    assert not any(d.optional for d in decls)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_schedule_runs_the_stretch_with_a_junction_ahead_of_every_pass(name):
    from gophonic_b200.config import KalonexConfig
    cfg = CONFIGS[name]
    spec = KalonexConfig.from_dict(cfg).model_spec()
    runs = P.layer_runs(cfg)
    assert [e.layer for e in spec.schedule] == [i for i, _ in runs]
    assert all(e.cache_of is None for e in spec.schedule)              # every pass keeps keys of its own
    for e, (i, t) in zip(spec.schedule, runs):
        if t >= 0 and i == cfg["loop"]["start"]:
            assert e.enter.kind == "reinject" and (e.enter.index, e.enter.passes, e.enter.hidden) == (t, cfg["loop"]["times"], cfg["width"])
        else:
            assert e.enter is None


def test_the_spec_carries_the_designs_constants():
    from gophonic_b200.config import KalonexConfig
    spec = KalonexConfig.from_dict(CONFIGS["mix"]).model_spec()
    assert spec.final_norm.gain == 1.3 and spec.head.tied_to is None and spec.streams == 1
    a = spec.layers[1].mixer
    assert a.kind == "gated_attention" and (a.heads, a.kv_heads, a.head_dim, a.value_dim, a.window, a.scale) == (6, 3, 16, 24, 100, 0.3)
    assert a.sink and a.sink_learned and a.bias and a.out_bias and not a.gate and a.qk_norm_span and a.qk_norm.eps == 1e-5
    assert a.position.kind == "rope" and (a.position.rotary_dim, a.position.theta) == (16, 100.0)
    f = spec.layers[1].feed_forward
    assert f.kind == "moe" and (f.experts, f.top, f.intermediate) == (5, 2, 40)
    assert (f.score, f.renorm, f.weight_on, f.act) == ("sigmoid", False, "input", "swiglu") and f.shared.intermediate == 24
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.kind == "swiglu"
    assert spec.layers[3].feed_forward.shared is None


def test_what_a_file_leaves_out_is_not_there():
    from gophonic_b200.config import KalonexConfig
    cfg = KalonexConfig.from_dict(CONFIGS["odd"])
    spec = cfg.model_spec()
    bare = spec.layers[0].mixer
    assert (bare.kv_heads, bare.value_dim, bare.window) == (3, 24, 0) and bare.position.kind == "none"
    assert cfg.loop is None and cfg.logit_scale == 1.0 and spec.final_norm.gain == 1.0
    assert all(e.enter is None for e in spec.schedule)
    assert "loop.in" not in P.tensor_shapes(CONFIGS["odd"])


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="gla"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=4), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=17), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c.update(logit_scale="big"), "logit_scale"),
])
def test_a_wrong_file_is_refused(change, message):
    from gophonic_b200.config import ConfigError, KalonexConfig
    cfg = copy.deepcopy(CONFIGS["mix"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        KalonexConfig.from_dict(cfg)


def test_random_weights_write_a_model_the_plain_reader_takes(tmp_path):
    from gophonic_b200.config import KalonexConfig
    from gophonic_b200.weights import write_random_model
    cfg = CONFIGS["mix"]
    d = write_random_model(KalonexConfig.from_dict(cfg), seed=1, out_dir=str(tmp_path / "m"))
    read, w = P.read_model(d)
    assert {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
    assert abs(w["l0.norm1"] - 1).max() < 0.5 and abs(w["l1.mix.q.norm"] - 1).max() < 0.5
    assert np.isfinite(P.forward(read, w, [1, 2, 3])).all()


def test_every_pass_has_a_cache_plane_of_its_own():
    from gophonic_b200.cache import Cache
    from gophonic_b200.config import KalonexConfig
    from gophonic_b200 import parts, registry  # noqa: F401
    spec = KalonexConfig.from_dict(CONFIGS["last"]).model_spec()
    reqs = [(registry.part_class("block", spec.layers[e.layer].block).cache_request(spec.layers[e.layer]), e.cache_of) for e in spec.schedule]
    assert len(reqs) == 4                                              # one layer, then one layer three times
    cache = Cache(reqs, max_tokens=256, device="cpu", dtype=torch.float32, max_slots=2)
    planes = {cache.view(i).k.data_ptr() for i in range(4)}
    assert len(planes) == 4
    cache.check()
