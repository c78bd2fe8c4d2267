"""Gipozen on the CPU: the configuration class, the spec it emits, the tensors the assembled model asks for, and the
cache manager's part of the design (pages of kept first keys, a state besides the pages)."""
import copy

import pytest
import torch

import gipozen_models as gm
from cisr_b200.cache import CacheManager
from cisr_b200.config import CacheUse, ConfigError, architecture_for
from cisr_b200.engine.model import Model


def spec_of(cfg):
    return architecture_for(cfg).config_class.from_dict(cfg).to_spec()


@pytest.mark.parametrize("case", sorted(gm.CASES))
def test_the_model_asks_for_exactly_the_designs_tensors(case):
    cfg, _ = gm.CASES[case]
    model = Model(spec_of(cfg), "float32", config=cfg, device=None)
    assert {k: tuple(v.shape) for k, v in model.tensor_needs().items()} == {k: tuple(v) for k, v in gm.tensor_shapes(cfg).items()}


def test_spec_carries_every_constant_of_the_configuration():
    spec = spec_of(gm.GA)
    assert spec.stream.kind == "depth_average" and spec.stream["entries"] == 4
    assert [e.cache_of for e in spec.run] == [None, 0, None, 2]
    m0, m1, m3 = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[3].mixer
    assert (m0["num_heads"], m0["num_kv_heads"], m0["key_dim"], m0["value_dim"], m0["conv"]) == (4, 2, 24, 40, 3)
    assert (m0["window"], m0["keep_first"], m0["scale"], m0["diff"], m0["shared_kv"]) == (21, 5, 0.21, 0.55, False)
    assert (m1["window"], m1["keep_first"], m1["shared_kv"], m1["conv"]) == (13, 18, True, 2)
    assert m3["conv"] == 1 and m3["keep_first"] == 1
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    ff1 = spec.layers[1].feed_forward
    assert (ff1.kind, ff1["experts"], ff1["identity"], ff1["top"], ff1["limit"], ff1["scores"]) == ("routed_experts", 5, 2, 2, 1.5, "softmax")
    assert ff1["shared"] == {"size": 24, "limit": 0.8} and spec.layers[3].feed_forward["shared"] is None
    assert spec.layers[0].feed_forward.kind == "polynorm_mlp" and spec.layers[0].feed_forward["eps"] == gm.GA["norm"]["eps"]
    assert spec.head["scale"] == 0.5 and spec.layers[3].extras["depth"]["count"] == 5
    no_mask = spec_of(gm.GC).layers[0].mixer
    assert no_mask["window"] is None and no_mask["keep_first"] == 0


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="delta"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(dim=130), "do not fit"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "must come earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no keys and values of its own"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=48), "other key/value heads or widths"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="swiglu"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "lacks"),
    (lambda c: c["norm"].pop("eps"), "lacks"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "at least 1"),
])
def test_refusals_come_before_any_weight_is_read(change, message):
    cfg = copy.deepcopy(gm.GA)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_of(cfg)


def test_pages_with_kept_first_keys_stay_while_the_window_moves_on():
    use = CacheUse("pages", kv_heads=1, head_dim=16, window=20, keep_first=18)
    plain = CacheUse("pages", kv_heads=1, head_dim=16, window=20)
    assert use.group_key() != plain.group_key()
    cache = CacheManager([use, plain], n_pages=12, page_size=8, max_slots=2, max_positions=256)
    cache.create("a")
    for n in (30, 1, 1, 40, 3):
        cache.reserve([("a", n)])
        cache.commit("a", n)
        cache.check()
    kept, moving = (cache.requests["a"].tables[g.index] for g in cache.page_groups)
    # 75 tokens: the next query (position 75) sees keys from 56 on, and the first 18 keys: pages 0..2 stay
    assert [p >= 0 for p in kept] == [True, True, True, False, False, False, False, True, True, True]
    assert [p >= 0 for p in moving] == [False] * 7 + [True] * 3
    cache.release("a")
    assert all(g.pool.n_free == g.pool.n_pages for g in cache.page_groups)


def test_a_state_besides_the_pages_is_the_entrys_own():
    pages = CacheUse("pages", kv_heads=2, head_dim=16, window=None)
    side = [CacheUse("state", state_shape=(2, 10)), CacheUse("state", state_shape=(2, 4)), None]
    cache = CacheManager([pages, 0, pages], n_pages=4, page_size=8, max_slots=2, max_positions=64, dtype=torch.float32,
                         device=torch.device("cpu"), side_states=side)
    own, reader, none = cache.binding(0), cache.binding(1, reads_from=0), cache.binding(2)
    assert own.state.shape == (3, 2, 10) and reader.state.shape == (3, 2, 4) and none.state is None
    assert own.write and not reader.write and reader.k.data_ptr() == own.k.data_ptr()
    own.state[:] = 1.0
    reader.state[:] = 2.0
    slot = cache.create("a")
    assert float(own.state[slot].abs().sum()) == 0.0 and float(reader.state[slot].abs().sum()) == 0.0      # a new request starts from zeros
    assert float(own.state[1 - slot].sum()) == 20.0
    with pytest.raises(ValueError):
        CacheManager([pages], 4, 8, 2, 64, side_states=[pages])


def test_pages_that_another_layer_reads_stay_while_either_mask_sees_them():
    """A layer that reads another's keys and values masks them by its own window and kept first keys: the owner's pages
    are kept by the wider of the two windows and the larger count of kept keys."""
    uses = Model(spec_of(gm.GA), "float32", config=gm.GA, device=None).cache_uses()
    assert uses[1] == 0 and uses[3] == 2
    assert (uses[0].window, uses[0].keep_first) == (21, 18) and (uses[2].window, uses[2].keep_first) == (40, 1)
    uses = Model(spec_of(gm.GC), "float32", config=gm.GC, device=None).cache_uses()
    assert uses[0].window is None and uses[2] == 0
    reader_without_window = copy.deepcopy(gm.GA)
    reader_without_window["layers"][1]["mixer"].pop("mask")
    uses = Model(spec_of(reader_without_window), "float32", config=reader_without_window, device=None).cache_uses()
    assert uses[0].window is None and uses[0].keep_first == 0
