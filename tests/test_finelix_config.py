"""The Finelix configuration, its model spec and what the cache manager is asked for; no GPU."""
import copy
import json
import os

import pytest
import torch

from helpers import TINY_FINELIX, make_finelix_folder
from photon_infer_b200.cache.manager import CacheManager
from photon_infer_b200.config import load_config
from photon_infer_b200.config.finelix_config import FinelixConfig
from photon_infer_b200.errors import ErrorCode, PhotonError
from photon_infer_b200.models.model import _Skeleton, declared_tensors
from photon_infer_b200.parts.base import PagedCacheSpec, TensorSpec
from photon_infer_b200.weights.loader import check_names_and_shapes


def _cfg(name):
    return copy.deepcopy(TINY_FINELIX[name]["config"])


def test_round_trip_and_registry(tmp_path):
    for name in TINY_FINELIX:
        cfg = FinelixConfig.from_dict(_cfg(name))
        assert FinelixConfig.from_dict(cfg.to_dict()) == cfg
    folder = make_finelix_folder(str(tmp_path / "m"), "fx_a")
    arch, cfg = load_config(folder)
    assert arch.name == "Finelix" and cfg.width == 64 and cfg.loop.times == 2
    # the other way of naming the class is read too
    d = _cfg("fx_b"); d["architectures"] = [d.pop("architecture")]
    assert FinelixConfig.from_dict(d).architecture == "Finelix"


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("norm", "eps"), None, "norm.eps"), (("layers", 1, "type"), "conv", "layers[1].type"),
    (("layers", 1, "mixer", "kv_rank"), None, "kv_rank"), (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "tau"), "x", "tau"), (("layers", 1, "mlp", "router", "top"), 9, "router.top"),
    (("layers", 0, "mlp", "kind"), "conv", "mlp.kind"), (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop.times"),
])
def test_errors_name_the_key(path, value, word):
    d = _cfg("fx_a")
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(PhotonError) as e:
        FinelixConfig.from_dict(d)
    assert e.value.code == ErrorCode.INVALID_CONFIG and word in str(e.value)


def test_run_list_follows_the_loop():
    arch_spec = lambda name: load_spec(name)
    run = [(e.layer, e.before) for e in load_spec("fx_a").run]
    assert run == [(0, None), (1, ("loop", 0)), (2, None), (1, ("loop", 1)), (2, None), (3, None)]
    assert [(e.layer, e.before) for e in load_spec("fx_b").run] == [(0, None), (1, None)]
    assert [(e.layer, e.before) for e in load_spec("fx_c").run] == \
        [(0, ("loop", 0)), (1, None), (0, ("loop", 1)), (1, None), (0, ("loop", 2)), (1, None)]
    assert [(e.layer, e.before) for e in load_spec("fx_d").run] == [(0, None), (1, ("loop", 0))]
    assert not load_spec("fx_b").stream_parts and "loop" in load_spec("fx_a").stream_parts


def load_spec(name):
    from photon_infer_b200.config import get_architecture
    arch = get_architecture("Finelix")
    return arch.build_spec(arch.config_class.from_dict(_cfg(name)))


def test_declared_tensors():
    d = declared_tensors(load_spec("fx_a"))
    for n in ("embed", "head", "final.norm", "loop.in", "loop.step", "l0.norm1", "l0.mix.a2.b", "l0.mlp.gate",
              "l1.mix.dkv.norm", "l1.mix.uk", "l1.mlp.router.b", "l1.mlp.e3.down", "l1.mlp.shared.up", "l2.mix.norm"):
        assert n in d, n
    assert not any(n.startswith("l2.mlp.") for n in d)                    # that layer has no feed-forward
    assert d["loop.in"].shape == (64, 128) and d["loop.step"].shape == (2, 64)
    assert d["l1.mix.dkv"].shape == (32 + 8, 64) and d["l1.mix.uq"].shape == (3 * (16 + 8), 24)
    assert d["l0.mix.a1"].shape == (-1, 64)                               # the file decides the rank ...
    assert declared_tensors(load_spec("fx_c"))["l1.mix.a1"].shape == (6, 48)   # ... unless the configuration does
    b = declared_tensors(load_spec("fx_b"))
    assert "l0.mlp.shared.gate" not in b and "l1.mlp.shared.gate" in b and "loop.in" not in b


def test_a_size_the_file_decides():
    spec = {"a": TensorSpec("a", (-1, 8)), "b": TensorSpec("b", (4, -1))}
    check_names_and_shapes(spec, {"a": (3, 8), "b": (4, 11)}, {"a": torch.bfloat16, "b": torch.bfloat16}, "x")
    with pytest.raises(PhotonError):
        check_names_and_shapes(spec, {"a": (3, 9), "b": (4, 11)}, {"a": torch.bfloat16, "b": torch.bfloat16}, "x")
    assert spec["a"].concrete_shape() == (16, 8)


def test_cache_needs_latent_rows_and_state_slots():
    sk = _Skeleton(load_spec("fx_a"))
    needs = []
    for e in sk.spec.run:
        m = sk.blocks[e.layer].mixer()
        needs.append((m.cache_spec(), m.state_spec()))
    # run list: gla, [latent, gla_2] x 2, latent
    assert [n[0] is not None for n in needs] == [False, True, False, True, False, True]
    assert needs[1][0] == PagedCacheSpec(1, 40, None, values=False) and needs[1][0].planes == 1
    assert needs[0][1].shape == (2, 16, 24) and needs[2][1].shape == (1, 32, 16) and needs[0][1].dtype == torch.float32
    cm = CacheManager(needs, [None] * len(needs), 16, 6, 4, torch.bfloat16, None)
    # two passes of layer 1 share one group (equal needs) with a pool of their own each; the last layer has another row width
    assert [(g.spec.head_dim, g.entries) for g in cm.groups] == [(40, [1, 3]), (40, [5])] or \
        [(g.spec.head_dim, g.entries) for g in cm.groups] == [(40, [1, 3, 5])]
    assert sorted(cm.states.specs) == [0, 2, 4]
    assert cm.groups[0].bytes_per_token(2) == len(cm.groups[0].entries) * 40 * 2


def test_pages_and_slots_come_back():
    sk = _Skeleton(load_spec("fx_d"))
    needs = [(sk.blocks[e.layer].mixer().cache_spec(), sk.blocks[e.layer].mixer().state_spec()) for e in sk.spec.run]
    cm = CacheManager(needs, [None, None], 16, 4, 2, torch.float32, None)
    a = cm.add_request("a"); cm.extend("a", 40); cm.commit("a", 40)
    b = cm.add_request("b"); cm.extend("b", 16); cm.commit("b", 16)
    assert {a, b} == {0, 1} and cm.free_pages() == [0]
    with pytest.raises(PhotonError):
        cm.add_request("c")
    cm.free_request("a")
    assert cm.add_request("c") == a and cm.free_pages() == [3]
    cm.check_consistency()
