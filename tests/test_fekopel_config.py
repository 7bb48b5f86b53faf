"""The Fekopel configuration, its model spec, what the cache manager is asked for, and the pages of a window that
keeps its first tokens; no GPU."""
import copy

import pytest
import torch

from helpers import TINY_FEKOPEL, make_fekopel_folder
from photon_infer_b200.cache.manager import CacheManager
from photon_infer_b200.cache.groups import NO_PAGE
from photon_infer_b200.config import load_config
from photon_infer_b200.config.fekopel_config import FekopelConfig
from photon_infer_b200.errors import ErrorCode, PhotonError
from photon_infer_b200.models.model import _Skeleton, declared_tensors
from photon_infer_b200.parts.base import PagedCacheSpec


def _cfg(name):
    return copy.deepcopy(TINY_FEKOPEL[name]["config"])


def load_spec(name_or_dict):
    from photon_infer_b200.config import get_architecture
    arch = get_architecture("Fekopel")
    d = _cfg(name_or_dict) if isinstance(name_or_dict, str) else name_or_dict
    return arch.build_spec(arch.config_class.from_dict(d))


def test_round_trip_and_registry(tmp_path):
    for name in TINY_FEKOPEL:
        cfg = FekopelConfig.from_dict(_cfg(name))
        assert FekopelConfig.from_dict(cfg.to_dict()) == cfg
    folder = make_fekopel_folder(str(tmp_path / "m"), "fk_a")
    arch, cfg = load_config(folder)
    assert arch.name == "Fekopel" and cfg.width == 64 and cfg.loop.times == 2
    d = _cfg("fk_b"); d["architectures"] = [d.pop("architecture")]
    assert FekopelConfig.from_dict(d).architecture == "Fekopel"


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("vocab",), 0, "vocab"), (("norm", "eps"), None, "norm.eps"), (("norm",), None, "norm"),
    (("layers", 1, "type"), "conv", "layers[1].type"), (("layers", 0, "mixer", "dim"), None, "dim"),
    (("layers", 0, "mixer", "scale"), "x", "scale"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 128, "rot.dims"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"), (("layers", 0, "mixer", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 0, "mlp", "router", "top"), 9, "router.top"), (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4, "groups"), (("layers", 0, "mlp", "kind"), "dense", "mlp.kind"),
    (("layers", 0, "mlp", "expert"), None, "expert"), (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop.times"),
])
def test_errors_name_the_key(path, value, word):
    d = _cfg("fk_a")
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(PhotonError) as e:
        FekopelConfig.from_dict(d)
    assert e.value.code == ErrorCode.INVALID_CONFIG and word in str(e.value)


def test_groups_that_cannot_hold_the_choice_are_refused():
    d = _cfg("fk_a")
    d["layers"][0]["mlp"]["router"].update(top=3, groups=dict(count=3, keep=1))      # one group of two experts for three choices
    with pytest.raises(PhotonError):
        FekopelConfig.from_dict(d)


def test_what_the_file_leaves_out_does_not_exist():
    d = _cfg("fk_a")
    m = d["layers"][0]["mixer"]
    for k in ("kv_heads", "vdim", "mask", "rot", "softcap"):
        m.pop(k)
    d["layers"][0]["mlp"]["router"].pop("groups"); d["layers"][0]["mlp"]["router"].pop("scale"); d["layers"][0]["mlp"].pop("shared")
    d["loop"] = None
    spec = load_spec(d)
    p = spec.layers[0].mixer.params
    assert p["n_kv_heads"] == p["n_q_heads"] == 2 and p["value_dim"] == 64 and p["window"] is None and p["rot_dims"] == 0
    assert p["softcap"] is None and p["keep_first"] == 0 and p["output_gate"] and p["norm_weight"] and not p.get("sink")
    f = spec.layers[0].feed_forward.params
    assert f["groups"] == 1 and f["route_scale"] == 1.0 and f["shared_size"] is None and not f["shared_gate"]
    assert not spec.stream_parts and "loop.step" not in declared_tensors(spec)


def test_the_two_mixers_are_one_part_with_other_parameters():
    spec = load_spec("fk_a")
    a2, a1 = spec.layers[0].mixer, spec.layers[1].mixer
    assert a1.kind == a2.kind == "normed_attention"
    assert a1.params["sink"] and not a1.params["norm_weight"] and not a1.params.get("output_gate") and not a1.params.get("rot_dims")
    assert a2.params["rot_dims"] == 16 and a2.params["rot_base"] == 5000.0 and a2.params["softcap"] == 6.0
    assert a2.params["window"] == 40 and a2.params["keep_first"] == 5 and a2.params["scale"] == 0.2
    ff = spec.layers[0].feed_forward.params
    assert (ff["experts"], ff["top"], ff["groups"], ff["keep_groups"], ff["route_scale"]) == (6, 2, 3, 2, 0.06)
    assert ff["activation"] == "gelu" and not ff["gated"] and not ff["router_bias"] and ff["scoring"] == "softmax_all"


def test_run_list_follows_the_loop():
    run = lambda name: [(e.layer, e.before) for e in load_spec(name).run]
    assert run("fk_a") == [(0, ("loop", 0)), (1, None), (0, ("loop", 1)), (1, None), (2, None)]
    assert run("fk_b") == [(0, None), (1, None), (2, None)]
    assert run("fk_c") == [(0, ("loop", 0)), (1, None), (0, ("loop", 1)), (1, None), (0, ("loop", 2)), (1, None)]
    assert run("fk_d") == [(0, None), (1, ("loop", 0)), (2, None)]
    assert run("fk_e") == [(0, None), (1, ("loop", 0)), (2, None), (1, ("loop", 1)), (2, None)]
    assert load_spec("fk_a").stream_parts["loop"].kind == "loop_add"


def test_declared_tensors():
    d = declared_tensors(load_spec("fk_a"))
    for n in ("embed", "head", "final.norm", "final.norm.b", "loop.step", "l0.norm1", "l0.norm1.b", "l0.norm2.b", "l0.mix.q.norm",
              "l0.mix.k.norm", "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.e5.up", "l0.mlp.e5.down", "l0.mlp.shared.up",
              "l0.mlp.shared.sg", "l1.mix.q", "l2.norm1.b"):
        assert n in d, n
    for n in ("l1.mix.g", "l1.mix.q.norm", "l0.mlp.router.b", "l0.mlp.e0.gate", "l1.mlp.shared.up", "l2.norm2", "l2.mlp.router", "loop.in"):
        assert n not in d, n
    assert d["loop.step"].shape == (2, 64) and d["l0.mix.q"].shape == (128, 64) and d["l0.mix.k"].shape == (64, 64)
    assert d["l0.mix.g"].shape == (128, 64) and d["l0.mlp.shared.sg"].shape == (1, 64) and d["l0.mix.q.norm"].shape == (64,)
    b = declared_tensors(load_spec("fk_b"))
    assert b["l0.mix.v"].shape == (40, 96) and b["l0.mix.o"].shape == (96, 120) and b["l1.mix.g"].shape == (32, 96)


def test_cache_needs_and_groups():
    sk = _Skeleton(load_spec("fk_a"))
    needs = [(sk.blocks[e.layer].mixer().cache_spec(), sk.blocks[e.layer].mixer().state_spec()) for e in sk.spec.run]
    assert needs[0][0] == PagedCacheSpec(1, 64, 40, value_dim=64, keep_first=5) and all(s is None for _, s in needs)
    cm = CacheManager(needs, [None] * len(needs), 16, 12, 4, torch.bfloat16, None)
    # the two passes of a looped layer have equal needs: one group, a pool of their own each
    assert [g.entries for g in cm.groups] == [[0, 2], [1, 3], [4]]
    sk = _Skeleton(load_spec("fk_b"))
    spec = sk.blocks[0].mixer().cache_spec()
    assert spec.split_planes and spec.row_width == 16 + 40 and spec.keep_first == 0
    assert sk.blocks[2].mixer().cache_spec().keep_first == 0 and sk.blocks[1].mixer().cache_spec().keep_first == 11


@pytest.mark.parametrize("page,window,keep", [(8, 19, 11), (16, 40, 5), (4, 3, 1), (8, 8, 0), (16, 24, 16), (4, 6, 9)])
def test_a_window_gives_pages_back_but_keeps_the_first_tokens(page, window, keep):
    """Tokens arrive in portions of changing size.  After every step the request holds exactly the pages of the kept
    first tokens and of the keys the next token can see; everything else is back in the pool and may be taken by
    another request at once."""
    spec = PagedCacheSpec(1, 8, window, keep_first=keep)
    cm = CacheManager([(spec, None)], [None], page, 40, 2, torch.float32, None)
    cm.add_request("a")
    n = 0
    for step, cnt in enumerate([5, 1, 1, 30, 2, 1, 1, 1, 17, 1, 64, 1, 1, 3]):
        cm.extend("a", cnt)
        table = cm.groups[0].tables["a"]
        first_needed = max(0, n - window + 1)
        for p in list(range(min(keep, n + cnt))) + list(range(first_needed, n + cnt)):
            assert table[p // page] != NO_PAGE, f"step {step}: position {p} has no page"
        cm.commit("a", cnt)
        n += cnt
        held = {i for i, pg in enumerate(cm.groups[0].tables["a"]) if pg != NO_PAGE}
        want = {p // page for p in range(min(keep, n))} | {p // page for p in range(max(0, n - window + 1), n)}
        assert held == want, f"after {n} tokens"
        cm.check_consistency()
    free_before = cm.free_pages()[0]
    cm.add_request("b"); cm.extend("b", 3 * page); cm.commit("b", 3 * page)
    assert cm.free_pages()[0] < free_before
    cm.free_request("a"); cm.free_request("b")
    assert cm.free_pages() == [40]


def test_keys_and_values_of_other_widths_live_in_two_tensors():
    from photon_infer_b200.cache.groups import CacheGroup
    g = CacheGroup(PagedCacheSpec(2, 16, 8, value_dim=40), [0, 1], 4, 6, torch.float32, torch.device("cpu"))
    assert g.kv.shape == (2, 1, 6, 2, 4, 16) and g.v_only.shape == (2, 6, 2, 4, 40)
    assert g.bytes_per_token(2) == 2 * 2 * (16 + 40) * 2
    g2 = CacheGroup(PagedCacheSpec(2, 16, 8, value_dim=16), [0], 4, 6, torch.float32, torch.device("cpu"))
    assert g2.kv.shape == (1, 2, 6, 2, 4, 16) and g2.v_only is None
