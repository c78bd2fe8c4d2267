"""Vilodra on the CPU: the configuration class, the spec it emits, the tensors the assembled model asks for, the cache
groups of its layers, the launch plan of the recurrence, and the stretched rotary frequencies against the plain ones."""
import copy

import pytest
import torch

import plain_vilodra as pv
import vilodra_models as vm
from cisr_b200.cache import CacheManager
from cisr_b200.config import ConfigError, architecture_for, preset
from cisr_b200.engine.model import Model


def spec_of(cfg):
    return architecture_for(cfg).config_class.from_dict(cfg).to_spec()


@pytest.mark.parametrize("case", sorted(vm.CASES))
def test_the_model_asks_for_exactly_the_designs_tensors(case):
    cfg, _ = vm.CASES[case]
    model = Model(spec_of(cfg), "float32", config=cfg, device=None)
    needs = model.tensor_needs()
    assert {k: tuple(v.shape) for k, v in needs.items() if v.alias is None} == {k: tuple(v) for k, v in vm.tensor_shapes(cfg).items()}
    assert [k for k, v in needs.items() if v.alias is not None] == ["head"] and needs["head"].alias == "embed"


def test_spec_carries_every_constant_of_the_configuration():
    spec = spec_of(vm.VA)
    assert [e.cache_of for e in spec.run] == [None, None, None, 1, None]
    assert [l.mixer.kind for l in spec.layers] == ["lightning", "latent_attention", "diff_attention", "latent_attention", "lightning"]
    l0, a1, d2, a3 = (spec.layers[i].mixer for i in range(4))
    assert (l0["num_heads"], l0["key_dim"], l0["value_dim"], l0["decay"], l0["eps"]) == (3, 20, 12, (0.7, 0.93, 1.0), 1e-5)
    assert (a1["num_heads"], a1["plain_dim"], a1["rot_dim"], a1["value_dim"], a1["kv_rank"], a1["window"], a1["sink"], a1["shared_kv"]) == (3, 24, 8, 20, 40, 19, True, False)
    assert a1["position"].kind == "rotary_interleaved" and a1["position"]["scaling"] == {"kind": "yarn", "factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}
    assert (a3["window"], a3["shared_kv"], a3["scale"]) == (33, True, 0.25)
    assert (d2["num_heads"], d2["num_kv_heads"], d2["key_dim"], d2["value_dim"], d2["diff"], d2["conv"], d2["gate"]) == (4, 2, 24, 40, 0.55, 0, False)
    assert d2["position"]["dim"] == 12 and d2["position"]["scaling"]["kind"] == "wavelength"
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None and "feed_forward_scale" not in spec.layers[2].extras
    ff = spec.layers[1].feed_forward
    assert (ff.kind, ff["experts"], ff["top"], ff["route_scale"], ff["scores"], ff["renormalize"], ff["activation"]) == ("routed_experts", 5, 2, 1.7, "softmax", True, "gelu")
    assert spec.layers[0].feed_forward.kind == "swiglu" and spec.layers[0].mixer_norm.kind == "rms_norm_offset"
    assert all(l.extras["mixer_scale"]["value"] == 0.6 for l in spec.layers) and spec.head["tied_to"] == "embed"
    plain = spec_of(vm.VC)
    assert plain.layers[0].mixer["window"] is None and plain.layers[0].mixer["position"].get("scaling") is None
    assert preset("vilodra-small").to_spec().layers[3].mixer["shared_kv"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="delta"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "one decay"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5, 1.5]), "one decay"),
    (lambda c: c["layers"][0]["mixer"].update(dim=300), "not supported"),
    (lambda c: c["layers"][2]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"].update(dim=130), "do not fit"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=26), "must not exceed"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "must equal rot_dim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=250), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "must come earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "no down projection"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=24), "another kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "at least 1"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "not a feed-forward"),
    (lambda c: c["layers"][2]["mixer"].pop("scale"), "lacks"),
    (lambda c: c.pop("residual_mult"), "lacks"),
    (lambda c: c["norm"].pop("eps"), "lacks"),
])
def test_refusals_come_before_any_weight_is_read(change, message):
    cfg = copy.deepcopy(vm.VA)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_for(cfg).config_class.from_dict(cfg)


def test_cache_groups_states_and_shared_rows():
    """Lightning layers hold one state row per request and no pages; a latent layer's rows are one plane; a reader shares
    its owner's rows, and the owner keeps the wider of the two windows."""
    model = Model(spec_of(vm.VA), "float32", config=vm.VA, device=None)
    uses = model.cache_uses()
    assert uses[0].kind == "state" and uses[0].state_shape == (3 * 20 * 12,) and uses[4].state_shape == (2 * 40 * 24,)
    assert (uses[1].kind, uses[1].planes, uses[1].kv_heads, uses[1].head_dim, uses[1].window) == ("pages", 1, 1, 48, 33)
    assert uses[3] == 1 and (uses[2].planes, uses[2].kv_heads, uses[2].head_dim, uses[2].window) == (2, 2, 48, None)
    assert model.side_states() == [None] * 5
    narrow = Model(spec_of(vm.VB), "float32", config=vm.VB, device=None).cache_uses()
    assert narrow[2].window == 150 and narrow[3] == 2                  # the reader's window of 70 lies inside the owner's
    cache = CacheManager(uses, n_pages=6, page_size=16, max_slots=2, max_positions=256, device=None)
    cache.create("a")
    cache.reserve([("a", 70)])
    cache.commit("a", 70)
    cache.check()
    windowed = next(g for g in cache.page_groups if g.use.window == 33)
    assert windowed.pool.n_used == 3 and next(g for g in cache.page_groups if g.use.window is None).pool.n_used == 5
    cache.release("a")
    assert all(g.pool.n_free == g.pool.n_pages for g in cache.page_groups)


def test_the_recurrences_launch_plan_lists_the_chunks_of_long_portions():
    from cisr_b200.parts.lightning import CHUNKED_FROM, chunk_plan
    C = CHUNKED_FROM
    chunk_req, chunk_t0, req_chunk0, short = chunk_plan([1, C - 1, C, 2 * C + 5, 2])
    assert (chunk_req, chunk_t0, req_chunk0, short) == ([2, 3, 3, 3], [0, 0, C, 2 * C], [0, 0, 0, 1, 4], 3)
    assert chunk_plan([1, 1]) == ([], [], [0, 0], 2)


@pytest.mark.parametrize("base, dims, scaling", [(10000.0, 24, (8.0, 1.0, 4.0, 1024)), (500.0, 16, (8.0, 1.0, 2.0, 40)), (10000.0, 64, (3.0, 2.0, 16.0, 300))])
def test_frequencies_stretched_by_wavelength(base, dims, scaling):
    from cisr_b200.parts.rotary import scaled_frequencies
    s = dict(zip(("factor", "low", "high", "original"), scaling))
    plain = pv.plain_frequencies(base, dims)
    want = pv.stretched_by_wavelength(plain, s)
    got, magnitude = scaled_frequencies(plain.clone(), base, dims, {"kind": "wavelength", **s})
    assert magnitude == 1.0 and torch.allclose(got, want, rtol=1e-14, atol=0)
    assert (want < plain).any() and (want == plain).any(), "the constants would not show the rule"


@pytest.mark.parametrize("base, dims, scaling", [(50000.0, 8, vm.YARN_A), (1000.0, 64, vm.YARN_B), (1000000.0, 16, (8.0, 512, 32.0, 1.0))])
def test_frequencies_stretched_by_a_ramp(base, dims, scaling):
    from cisr_b200.parts.rotary import scaled_frequencies
    s = dict(zip(("factor", "original", "fast", "slow"), scaling))
    plain = pv.plain_frequencies(base, dims)
    want, want_magnitude = pv.stretched_by_ramp(plain, base, dims, s)
    got, magnitude = scaled_frequencies(plain.clone(), base, dims, {"kind": "yarn", **s})
    assert magnitude == pytest.approx(want_magnitude, rel=1e-15) and torch.allclose(got, want, rtol=1e-14, atol=0)
