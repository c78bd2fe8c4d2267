"""Vilodra through the engine against the plain implementation (tests/plain_vilodra.py).

Each mechanism alone (the recurrence token by token and chunk by chunk with state slots used again, its output norm and
gate, the turned rows of the two attention maps, the softmax sink per head on every attention kernel, the renormalised
router and the gelu experts on both of their paths, the norm whose weight is an offset from one), one-layer models, then
whole models under every way of cutting and batching: whole prompts, prefill against token-by-token decoding, portions
down to two and one tokens, unequal requests side by side with pages and slots used again, a request alone and in a
crowd, long decoding, the first tokens of a sequence, tokens made to stand out just inside and just outside a window and
far back in the recurrence, peaked attention, and greedy generation through the scheduler, the command line and the
trace program.
"""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vilodra as pv
import replay
import vilodra_models as vm

pytestmark = pytest.mark.gpu
F = torch.float64
LENGTHS = {"a": 150, "b": 70, "c": 33, "d": 200, "e": 90, "f": 3, "g": 129, "h": 64, "i": 47, "j": 1}
_cache = {}


# ------------------------------------------------------------------ helpers
def plain(cfg, weights, tokens):
    return pv.forward(cfg, weights, tokens).numpy()


def setup(case, dtype, tmp_path_factory, gain=1.0, lengths=None, choice=None):
    """`choice` False: the same model with routers that take every expert (bfloat16 runs of whole models: a close call
    between two experts would send a token down another path than the plain implementation's)."""
    choice = dtype == "float32" if choice is None else choice
    key = (case, dtype, gain, choice, None if lengths is None else tuple(sorted(lengths.items())))
    if key not in _cache:
        from cisr_b200 import Model

        cfg, seed = vm.CASES[case]
        if not choice:
            cfg = vm.no_choice(cfg)
        weights = vm.make_weights(cfg, seed, gain=gain)
        path = vm.write_model_dir(tmp_path_factory.mktemp(f"{case}_{dtype}"), cfg, weights)
        model = Model.from_pretrained(path, dtype=dtype)
        requests = {rid: vm.random_tokens(cfg, n, 100 + i) for i, (rid, n) in enumerate((lengths or LENGTHS).items())}
        reference = {rid: plain(cfg, weights, tokens) for rid, tokens in requests.items()}
        _cache[key] = (cfg, weights, path, model, requests, reference)
    return _cache[key]


def compare(got, requests, reference, dtype, scale=4.0):
    """float32: every logit within the replay tests' bound.  bfloat16: every row's relative RMS error below twice the
    replay tests' bound, and at most one row in a hundred (or one) above the bound itself.  The lightning mixer divides a
    token's read-out by its root mean square, and the differential attention divides the difference of its two maps by
    its root mean square per head; where such a vector of a few numbers is nearly zero (a position among hundreds, the
    same under every cut) the rounding of the layer's input is magnified there, in the plain implementation's arithmetic
    as in the engine's, while the float32 run of the same model stays inside its bound."""
    if dtype == "float32":
        return replay.compare(got, requests, reference, dtype, scale=scale)
    assert got, "nothing was compared"
    errors = {key: replay.relative_rms(row, reference[key[0]][key[1]]) for key, row in got.items()}
    assert all(np.isfinite(row).all() for row in got.values())
    worst = max(errors, key=errors.get)
    assert errors[worst] < 2 * replay.RRMS16, f"bfloat16 logits differ for request {worst[0]} at position {worst[1]}: {errors[worst]:.4f}"
    over = sorted(k for k, e in errors.items() if e >= replay.RRMS16)
    assert len(over) <= max(1, len(errors) // 100), f"bfloat16 rows over the bound: {over[:10]}"


def stepper_for(model, steps, slack_pages=0):
    from cisr_b200 import Stepper
    return Stepper(model, n_pages=replay.max_live_tokens(steps) // 16 + slack_pages, page_size=16, max_slots=4)


def model_of(cfg, weights, tmp_path, dtype="float32"):
    from cisr_b200 import Model
    return Model.from_pretrained(vm.write_model_dir(tmp_path, cfg, weights), dtype=dtype)


def dev(a):
    return torch.from_numpy(np.asarray(a, dtype=np.int32)).cuda()


# ------------------------------------------------------------------ each mechanism alone: kernels
@pytest.mark.parametrize("heads, dk, dv, columns", [(3, 20, 12, 0), (2, 64, 64, 16), (1, 10, 7, 0), (2, 100, 40, 32), (1, 160, 24, 0),
                                                    (2, 32, 128, 64), (1, 256, 16, 0)])
def test_recurrence_token_by_token_and_chunk_by_chunk(heads, dk, dv, columns):
    """Two requests in portions of every kind (one token, a few, a whole chunk, several chunks with a tail), rows of a step
    not in slot order, slots that held another request's state before, both forms side by side in one step: read-outs
    and the state left behind against the plain recurrence in float64."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(heads * 1000 + dk)
    decay = torch.tensor([0.6, 0.97, 1.0][:heads] if heads <= 3 else np.linspace(0.5, 0.999, heads), dtype=torch.float32)
    nqk, nv = heads * dk, heads * dv
    cols = 2 * nqk + 2 * nv + 5
    lengths = {0: 64 + 130 + 1 + 9 + 63, 1: 3 + 1 + 200 + 64}
    us = {r: 0.7 * torch.randn(n, cols, generator=g) for r, n in lengths.items()}
    want = {}
    for r, u in us.items():
        x = u.to(F)
        q, k = pv.silu(x[:, :nqk]).view(-1, heads, dk), pv.silu(x[:, nqk:2 * nqk]).view(-1, heads, dk)
        v = pv.silu(x[:, 2 * nqk:2 * nqk + nv]).view(-1, heads, dv)
        want[r] = pv.lightning_recurrence(q, k, v, decay.to(F)).reshape(-1, nv)
    slot = {0: 3, 1: 1}
    state = torch.randn(5, heads * dk * dv, generator=g).cuda()          # what other requests left in the slots
    for s in slot.values():
        state[s].zero_()                                                 # what the cache manager does at `create`
    cuts = {0: [64, 130, 1, 9, 63], 1: [3, 1, 200, 64]}
    at, got = {0: 0, 1: 0}, {0: [], 1: []}
    while any(cuts.values()):
        batch = [r for r in (1, 0) if cuts[r]]
        sizes = [cuts[r].pop(0) for r in batch]
        proj = torch.cat([us[r][at[r]:at[r] + n] for r, n in zip(batch, sizes)]).cuda().contiguous()
        q_start = np.cumsum([0] + sizes[:-1]).astype(np.int32)
        chunk_req, chunk_t0, req_chunk0 = [], [], []          # the chunks of the portions that are long enough, request by request
        for i, n in enumerate(sizes):
            req_chunk0.append(len(chunk_req))
            if n >= kernels.LIGHTNING_CHUNK:
                for t0 in range(0, n, kernels.LIGHTNING_CHUNK):
                    chunk_req.append(i)
                    chunk_t0.append(t0)
        n_short = sum(n < kernels.LIGHTNING_CHUNK for n in sizes)
        o = torch.full((proj.shape[0], nv), 7.0, device="cuda")
        kernels.lightning_recurrence(proj, 0, nqk, 2 * nqk, decay.cuda(), state, dev([slot[r] for r in batch]), dev(q_start), dev(sizes),
                                     len(batch), o, heads, dk, dv, least=kernels.LIGHTNING_CHUNK if chunk_req else 0, n_short=n_short,
                                     chunks=(dev(chunk_req), dev(chunk_t0), dev(req_chunk0), len(chunk_req)) if chunk_req else None,
                                     columns_per_cta=columns)
        for i, (r, n) in enumerate(zip(batch, sizes)):
            got[r].append(o[q_start[i]:q_start[i] + n].double().cpu())
            at[r] += n
    for r in lengths:
        out = torch.cat(got[r])
        err = (out - want[r]).abs().max() / want[r].abs().max()
        assert err < 2e-5, f"request {r}: read-outs differ by {float(err)}"
    # the same tokens, all token by token, leave the same state up to rounding
    walked = torch.zeros_like(state)
    for r, u in us.items():
        o = torch.empty((u.shape[0], nv), device="cuda")
        kernels.lightning_recurrence(u.cuda().contiguous(), 0, nqk, 2 * nqk, decay.cuda(), walked, dev([slot[r]]), dev([0]), dev([u.shape[0]]), 1, o,
                                     heads, dk, dv)
        assert (o.double().cpu() - want[r]).abs().max() / want[r].abs().max() < 2e-5
        assert torch.allclose(walked[slot[r]], state[slot[r]], rtol=2e-4, atol=2e-4 * float(state[slot[r]].abs().max()))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, width, out_cols", [(7, 36, 40), (1, 7, 8), (130, 1024, 1024), (3, 128, 128)])
def test_output_norm_and_gate_of_the_recurrence(out_dtype, tokens, width, out_cols):
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(width)
    o, gate, w = torch.randn(tokens, width, generator=g), torch.randn(tokens, width + 9, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
    out = torch.full((tokens, out_cols), 5.0, dtype=out_dtype, device="cuda")
    kernels.lightning_output(o.cuda(), gate.cuda(), 4, w.cuda(), 1e-5, out)
    want = pv.rms(o.to(F), 1e-5) * w.to(F) * torch.sigmoid(gate.to(F)[:, 4:4 + width])
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert torch.allclose(out[:, :width].double().cpu(), want, rtol=tol, atol=tol)
    assert (out[:, width:] == 5.0).all(), "padding columns belong to the caller"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, dk, dv, rot_dims, write", [(4, 2, 24, 40, 12, True), (2, 1, 32, 64, 32, True), (1, 1, 10, 25, 4, True),
                                                              (2, 2, 64, 128, 16, True), (4, 2, 24, 40, 0, True), (6, 3, 16, 24, 8, False)])
def test_turned_rows_of_the_two_maps(dtype, hq, hkv, dk, dv, rot_dims, write):
    """Each map's leading coordinates turn in neighbouring pairs, the rest pass; query rows of map m lie where the key row
    holds k_m; key and value rows land in the token's place in scattered pages."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(hq * 100 + dk)
    width = -(-max(2 * dk, dv) // 16) * 16
    nq, nk, nv = hq * 2 * dk, hkv * 2 * dk, hkv * dv
    tokens, page, n_pages = 21, 8, 9
    proj = torch.randn(tokens, nq + nk + nv + 3, generator=g)
    positions = np.arange(40, 40 + tokens, dtype=np.int32)
    freq = pv.plain_frequencies(300.0, rot_dims) if rot_dims else torch.zeros(0, dtype=F)
    angle = torch.tensor(positions, dtype=F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle).float().cuda().contiguous(), torch.sin(angle).float().cuda().contiguous()
    table = np.full((2, 10), -1, dtype=np.int32)
    table[1, 5:8] = [6, 2, 7]                                   # positions 40 .. 63 of slot 1
    q = torch.full((tokens, 2 * hq, width), 7.0, dtype=dtype, device="cuda")
    k_cache = torch.full((n_pages, hkv, page, width), 9.0, dtype=dtype, device="cuda")
    v_cache = torch.full((n_pages, hkv, page, width), 9.0, dtype=dtype, device="cuda")
    kernels.diff_rope_rows(proj.cuda(), nq, nq + nk, cos=cos if rot_dims else None, sin=sin if rot_dims else None, rot_half=rot_dims // 2,
                           interleaved=True, token_req=dev([0] * tokens), req_slot=dev([1]), positions=dev(positions), q_out=q,
                           k_cache=k_cache if write else None, v_cache=v_cache if write else None, block_table=dev(table), page_size=page,
                           hq=hq, hkv=hkv, key_dim=dk, value_dim=dv)

    def turned(x):              # x [tokens, heads, 2, dk] at the test's positions
        out = x.clone()
        for i in range(rot_dims // 2):
            c, s = torch.cos(angle[:, i]).view(-1, 1, 1), torch.sin(angle[:, i]).view(-1, 1, 1)
            out[..., 2 * i], out[..., 2 * i + 1] = x[..., 2 * i] * c - x[..., 2 * i + 1] * s, x[..., 2 * i + 1] * c + x[..., 2 * i] * s
        return out

    tol = 1e-5 if dtype == torch.float32 else 1e-2
    want_q = turned(proj[:, :nq].to(F).view(tokens, hq, 2, dk))
    got_q = q.double().cpu().view(tokens, hq, 2, width)
    for m in range(2):
        assert torch.allclose(got_q[:, :, m, m * dk:(m + 1) * dk], want_q[:, :, m], rtol=tol, atol=tol)
        rest = torch.cat((got_q[:, :, m, :m * dk], got_q[:, :, m, (m + 1) * dk:]), dim=-1)
        assert (rest == 0).all(), "a query row is zero outside its own map"
    if not write:
        assert (k_cache == 9.0).all() and (v_cache == 9.0).all()
        return
    want_k = turned(proj[:, nq:nq + nk].to(F).view(tokens, hkv, 2, dk)).reshape(tokens, hkv, 2 * dk)
    want_v = proj[:, nq + nk:nq + nk + nv].to(F).view(tokens, hkv, dv)
    for t, pos in enumerate(positions):
        p, off = table[1, pos // page], pos % page
        assert torch.allclose(k_cache[p, :, off, :2 * dk].double().cpu(), want_k[t], rtol=tol, atol=tol)
        assert torch.allclose(v_cache[p, :, off, :dv].double().cpu(), want_v[t], rtol=tol, atol=tol)
        assert (k_cache[p, :, off, 2 * dk:] == 0).all() and (v_cache[p, :, off, dv:] == 0).all()
    untouched = [p for p in range(n_pages) if p not in (6, 2, 7)]
    assert (k_cache[untouched] == 9.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, hq, dv, width", [(5, 4, 40, 48), (130, 2, 96, 128), (3, 3, 25, 32)])
def test_combination_of_the_two_maps_without_a_gate(dtype, tokens, hq, dv, width):
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(tokens + dv)
    mixed = torch.randn(tokens, 2 * hq, width, generator=g).to(dtype)
    out = torch.empty((tokens, hq * dv), dtype=dtype, device="cuda")
    kernels.diff_combine(mixed.cuda(), None, 0, out, hq, dv, 0.37, 1e-5, 0.6)
    a = mixed.to(F).view(tokens, hq, 2, width)[..., :dv]
    want = (pv.rms(a[:, :, 0] - 0.37 * a[:, :, 1], 1e-5) * 0.6).reshape(tokens, hq * dv)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("experts, top, scale, hidden", [(5, 2, 1.7, 80), (3, 1, 0.8, 72), (12, 4, 2.0, 176), (4, 4, 1.0, 64)])
def test_renormalised_softmax_router(experts, top, scale, hidden):
    """The chosen experts are the `top` largest softmax scores; their weights are those scores over their sum, times the
    scale (so they add up to the scale, and top 1 always weighs exactly the scale)."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(experts)
    logits = 2.0 * torch.randn(37, experts, generator=g)
    chosen = torch.empty((37, top), dtype=torch.int32, device="cuda")
    weight = torch.empty((37, top), dtype=torch.float32, device="cuda")
    kernels.moe_select(logits.cuda(), top, 0, 0, scale, chosen, weight, scores="softmax", renormalize=True)
    s = torch.softmax(logits.to(F), dim=-1)
    best = torch.topk(s, top, dim=-1)
    want = best.values / (best.values.sum(-1, keepdim=True) + 1e-20) * scale
    assert (chosen.cpu().long() == best.indices).all()
    assert torch.allclose(weight.double().cpu(), want, rtol=1e-5, atol=1e-6)
    assert torch.allclose(weight.double().cpu().sum(-1), torch.full((37,), scale, dtype=F), rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, experts, top, ff, hidden", [(6, 5, 2, 40, 72), (1, 3, 1, 24, 64), (700, 4, 2, 64, 128), (40, 3, 3, 20, 52)])
def test_gelu_experts_on_both_paths(dtype, tokens, experts, top, ff, hidden):
    """A routed feed-forward alone against the plain one: few tokens and float32 run the row kernels, many bfloat16 tokens
    the sorted, grouped tensor-core products.  The inputs are the same to the bit, so the choice is the same too."""
    from cisr_b200.config import PartSpec
    from cisr_b200.parts import FEED_FORWARDS, build_part
    g = torch.Generator().manual_seed(tokens + experts)
    bf = lambda x: x.to(torch.bfloat16).to(F)
    w = {"mlp.router": bf(3.0 / hidden ** 0.5 * torch.randn(experts, hidden, generator=g))}
    for e in range(experts):
        w[f"mlp.e{e}.up"] = bf(torch.randn(ff, hidden, generator=g) / hidden ** 0.5)
        w[f"mlp.e{e}.down"] = bf(torch.randn(hidden, ff, generator=g) / ff ** 0.5)
    part = build_part(FEED_FORWARDS, PartSpec("routed_experts", {
        "hidden_size": hidden, "expert_size": ff, "experts": experts, "top": top, "scores": "softmax", "renormalize": True, "route_scale": 1.3,
        "activation": "gelu", "names": {"router": "router", "up": "e{}.up", "down": "e{}.down"}}), dtype, "feed-forward")
    part.load({k[4:]: v.to(dtype).cuda() for k, v in w.items()})
    h = bf(torch.randn(tokens, hidden, generator=g))
    got = part.forward(h.to(dtype).cuda(), None).double().cpu()
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": 1.3}}
    want = pv.routed_ff(w, "mlp.", mlp, h)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got, want, rtol=tol, atol=tol * float(want.abs().max()))


def test_norm_whose_weight_is_an_offset_from_one():
    from cisr_b200.config import PartSpec
    from cisr_b200.parts import NORMS, build_part
    g = torch.Generator().manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        part = build_part(NORMS, PartSpec("rms_norm_offset", {"size": 72, "eps": 1e-5, "weight_name": ""}), dtype, "norm")
        w = (0.3 * torch.randn(72, generator=g)).to(torch.bfloat16)
        part.load({"": w.to(dtype).cuda()})
        x, delta = torch.randn(9, 72, generator=g), torch.randn(9, 72, generator=g)
        xs = x.cuda()
        out = part.forward(xs, delta.cuda(), dtype)
        want = pv.layer_norm((x + delta).to(F), w.to(F), 1e-5)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol) and torch.allclose(xs.cpu(), x + delta)


@pytest.mark.parametrize("tokens, n, k", [(3, 72, 128), (16, 320, 192), (8, 4096, 1024), (200, 136, 256), (513, 72, 64)])
def test_products_add_into_the_stream_times_a_constant(tokens, n, k):
    """The in-place add of a sub-block's last product with the branch multiplier as its factor, on each product kernel
    that has it: the weight-streaming kernels for few tokens (small matrices, and the persistent one from 8 MB on) and
    the tcgen05 product for many.  out += 0.7 * (a w^T) against float64."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(tokens + n)
    a = torch.randn(tokens, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    x = torch.randn(tokens, n, generator=g)
    want = x.to(F) + 0.7 * (a.to(F) @ w.to(F).T)
    out = x.clone().cuda()
    if tokens <= 16:
        assert kernels.skinny_ok(tokens, w.cuda())
        kernels.skinny_gemm(w.cuda(), tokens, act=a.cuda(), epilogue=kernels.EPI_PLAIN, out=out, accumulate=True, out_mult=0.7)
    else:
        assert kernels.tcgen05_ok(a.cuda(), w.cuda())
        kernels.gemm_tcgen05(a.cuda(), w.cuda(), out, accumulate=True, out_mult=0.7)
    assert torch.allclose(out.double().cpu(), want, rtol=1e-4, atol=1e-4)
    plain = torch.empty(tokens, n, device="cuda")            # written, not added: the factor applies there too
    if tokens <= 16:
        kernels.skinny_gemm(w.cuda(), tokens, act=a.cuda(), epilogue=kernels.EPI_PLAIN, out=plain, out_mult=0.7)
    else:
        kernels.gemm_tcgen05(a.cuda(), w.cuda(), plain, out_mult=0.7)
    assert torch.allclose(plain.double().cpu(), want - x.to(F), rtol=1e-4, atol=1e-4)


# ------------------------------------------------------------------ one layer is the whole model
def one_latent(window, heads=3, dim=24, rot=8, vdim=20, rank=40, scale=0.3, width=64, scaling=vm.YARN_A, mlp=None):
    return vm.one_layer(vm.latent(heads, dim, rot, vdim, rank, scale, window=window, scaling=scaling), mlp, width=width)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank, rot, window", [(48, 16, 45), (96, 32, 131), (40, 8, 17), (13, 6, None), (64, 64, 300), (200, 24, 50)])
def test_every_attention_kernel_has_the_window_and_a_sink_per_head(dtype, rank, rot, window, tmp_path):
    """Cache rows of 64 and 128 (tcgen05 and tensor-map kernels in bfloat16), other widths up to 128 (`mma.sync`), wider
    ones and float32 (CUDA cores): prompts, single tokens and portions of one latent layer, whose sinks are spread so
    widely that a head without its own sink, or with its neighbour's, is far off."""
    cfg = one_latent(window, heads=4, dim=20, rot=rot, vdim=24, rank=rank, scale=0.1, scaling=None if rot == 6 else (4.0, 64, 8.0, 1.0))
    weights = vm.make_weights(cfg, 9)
    weights["l0.mix.sink"] = (3.0 * weights["l0.mix.sink"]).to(torch.bfloat16).to(F)      # sinks that take a large share of some heads' softmax
    model = model_of(cfg, weights, tmp_path, dtype)
    requests = {"p": vm.random_tokens(cfg, 333, 1), "q": vm.random_tokens(cfg, 40, 2)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    swapped = dict(weights)
    swapped["l0.mix.sink"] = weights["l0.mix.sink"].flip(0)
    assert replay.relative_rms(plain(cfg, swapped, requests["q"])[-1], reference["q"][-1]) > 1e-3, "the sinks would not show"
    for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 200), replay.trace_portions(requests, (100, 2, 129, 1, 31))):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=1), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mix", [vm.lightning(3, 20, 12, (0.7, 0.93, 1.0)), vm.lightning(2, 64, 64, (0.9, 0.999)), vm.lightning(1, 100, 7, (0.95,)),
                                 vm.attention(4, 2, 24, 40, 0.2, 0.55, 12, scaling=(4.0, 1.0, 4.0, 48)), vm.attention(2, 1, 32, 64, 0.18, 0.3, 32),
                                 vm.attention(2, 2, 64, 128, 0.12, 0.7, 16, base=500.0, scaling=(8.0, 1.0, 2.0, 40)), vm.attention(1, 1, 10, 25, 0.3, 0.45, 4)])
def test_one_layer_of_each_mixer_and_the_stream_after_it(mix, dtype, tmp_path):
    """The residual stream after the layer (the branch multiplier, the offset norm) and the logits, whole, decoded and in
    portions that cut inside chunks of the recurrence."""
    from cisr_b200 import StepEntry, Stepper
    cfg = vm.one_layer(mix, vm.dense(80), width=72, mult=0.45)
    weights = vm.make_weights(cfg, 11)
    model = model_of(cfg, weights, tmp_path, dtype)
    requests = {"p": vm.random_tokens(cfg, 210, 1), "q": vm.random_tokens(cfg, 70, 2)}
    streams = {}
    reference = {k: pv.forward(cfg, weights, t, after_layer=lambda i, x, k=k: streams.__setitem__(k, x.clone())).numpy() for k, t in requests.items()}
    seen = []
    model.layer_probe = lambda i, s: seen.append(s.total().double().cpu())
    stepper = Stepper(model, n_pages=20, page_size=16, max_slots=2)
    stepper.create("p")
    stepper.step([StepEntry("p", requests["p"], [])])
    model.layer_probe = None
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert torch.allclose(seen[0], streams["p"], rtol=tol, atol=tol * float(streams["p"].abs().max()))
    for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 40), replay.trace_portions(requests, (64, 2, 65, 1, 70, 3))):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=1), steps), requests, reference, dtype)


# ------------------------------------------------------------------ whole models under every cut
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(vm.CASES))
def test_whole_prompts(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_whole(requests)
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(vm.CASES))
def test_prefill_against_token_by_token_decoding(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_tail_decode(requests, 60)           # the windows of va and vc pass over decoded tokens only
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case, sizes", [("va", (16, 2, 15, 17, 3, 64, 33)), ("vb", (2, 2, 1, 5)), ("vc", (128, 7, 2, 130)), ("va", (1,)), ("vb", (2,)),
                                         ("vb", (65, 63, 2, 64))])
def test_portions_of_several_sizes(case, sizes, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    if max(sizes) <= 5:
        requests = {k: requests[k] for k in ("b", "c", "f", "j")}
    steps = replay.trace_portions(requests, sizes)
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(vm.CASES))
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_mixed(requests, seed=7, sizes=(9, 2, 17, 5, 3, 70, 2, 11))
    stepper = stepper_for(model, steps)
    compare(replay.run_steps(stepper, steps), requests, reference, dtype)
    assert not stepper.cache.requests and len(stepper.cache.free_slots) == 4
    assert all(g.pool.n_free == g.pool.n_pages for g in stepper.cache.page_groups)
    assert any(g.pool.taken > g.pool.n_pages for g in stepper.cache.page_groups), "no page was used twice"


def test_a_request_alone_and_in_a_crowd(tmp_path_factory):
    """The same request by itself and beside three others of other lengths, portion by portion and token by token:
    float32 logits agree far inside the comparison's bound (the products may choose another kernel by the step's token
    count; everything else is the same arithmetic in the same order)."""
    from cisr_b200 import StepEntry, Stepper
    cfg, weights, path, model, requests, reference = setup("va", "float32", tmp_path_factory)
    target = requests["e"]
    cuts = [30, 2, 17, 1, 1, 1, 20, 1, 1] + [1] * 16
    alone = Stepper(model, n_pages=40, page_size=16, max_slots=4)
    crowd = Stepper(model, n_pages=40, page_size=16, max_slots=4)
    alone.create("t")
    for key in ("x", "t", "y", "z"):
        crowd.create(key)
    others = {"x": requests["a"], "y": requests["d"], "z": requests["g"]}
    at, step = 0, 0
    for n in cuts:
        want = list(range(n))
        a = alone.step([StepEntry("t", target[at:at + n], want)]).cpu().numpy()
        entries = [StepEntry("x", others["x"][3 * step:3 * step + 3], []), StepEntry("t", target[at:at + n], want),
                   StepEntry("y", others["y"][step:step + 1], [0]), StepEntry("z", others["z"][4 * step:4 * step + 4], [])]
        b = crowd.step(entries).cpu().numpy()[:n]
        for i in range(n):
            assert replay.relative_rms(a[i], b[i].astype(np.float64)) < 2e-6, f"position {at + i} depends on its neighbours"
            compare({("e", at + i): a[i]}, requests, reference, "float32")
        at += n
        step += 1


def test_long_decoding(tmp_path_factory):
    """330 tokens one by one from the first: the recurrence runs far past its chunk length token by token, every window
    passes over decoded tokens many times, and pages behind the widest window that still reads them go back to their pool
    while the request lives."""
    cfg, weights, path, model, _, _ = setup("va", "float32", tmp_path_factory)
    requests = {"long": vm.random_tokens(cfg, 330, 77)}
    reference = {"long": plain(cfg, weights, requests["long"])}
    steps = replay.trace_portions(requests, (1,))
    stepper = stepper_for(model, steps)
    compare(replay.run_steps(stepper, steps), requests, reference, "float32")
    for g in stepper.cache.page_groups:
        if g.use.window is not None:
            assert g.pool.peak <= -(-g.use.window // 16) + 1, "a window kept pages it had passed"


def test_first_tokens_of_a_sequence(tmp_path_factory):
    """Positions 0, 1, 2, ...: a state that starts at zero, windows that are not full yet, a softmax over a single key
    and its sink; whole, in two-token portions and one by one, also with nothing wanted in a step."""
    cfg, weights, path, model, _, _ = setup("va", "float32", tmp_path_factory)
    requests = {f"s{n}": vm.random_tokens(cfg, n, 300 + n) for n in (1, 2, 3, 4, 6, 9)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (2,)), replay.trace_portions(requests, (1,))):
        compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32")
    nothing_wanted = [{"step": 0, "entries": [{"id": "s9", "tokens": requests["s9"][:5], "want": []}], "end": []},
                      {"step": 1, "entries": [{"id": "s9", "tokens": requests["s9"][5:], "want": [3]}], "end": ["s9"]}]
    got = replay.run_steps(stepper_for(model, nothing_wanted), nothing_wanted)
    assert list(got) == [("s9", 8)]
    compare(got, requests, reference, "float32")


def stands_out(cfg, weights, filler, place, seen):
    """The token of the vocabulary's last eight that moves the last position's plain logits most when put at `place`."""
    without = plain(cfg, weights, filler)[-1]
    effect = {}
    for b in range(cfg["vocab"] - 8, cfg["vocab"]):
        tokens = list(filler)
        tokens[place] = b
        effect[b] = replay.relative_rms(plain(cfg, weights, tokens)[-1], without)
    key = max(effect, key=effect.get)
    if seen:
        assert effect[key] > 1e-3, f"a token at {place} does not matter: the test would show nothing"
    else:
        assert effect[key] == 0.0, f"a token at {place}, beyond the window, moved the plain logits"
    return key


def test_tokens_just_inside_and_just_outside_the_window(tmp_path):
    """One latent layer is the whole model, so the last position sees exactly its window.  A token that occurs nowhere
    else is put at the window's oldest place (the plain implementation says it moves the last logits) and one place
    earlier (it does not move them at all); the engine must agree with the prompt whole, decoded (the window passing page
    borders on the way) and in portions that cut at the edge."""
    from cisr_b200 import Stepper
    window, n = 37, 150
    cfg = one_latent(window, scale=0.5)
    weights = vm.make_weights(cfg, 5, gain=2.0)
    model = model_of(cfg, weights, tmp_path)
    rng = np.random.default_rng(0)
    filler = [int(t) for t in rng.integers(0, cfg["vocab"] - 8, size=n)]
    oldest_seen = n - window
    for place, seen in ((oldest_seen, True), (oldest_seen - 1, False), (0, False), (n - 1, True)):
        tokens = list(filler)
        tokens[place] = stands_out(cfg, weights, filler, place, seen)
        requests, reference = {"r": tokens}, {"r": plain(cfg, weights, tokens)}
        for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 60),
                      replay.trace_portions(requests, (oldest_seen, 1, window - 2, 1)),
                      replay.trace_portions(requests, (oldest_seen - 1, 2, window - 1, 5))):
            compare(replay.run_steps(Stepper(model, n_pages=12, page_size=16, max_slots=2), steps), requests, reference, "float32", scale=1.0)


def test_a_token_far_back_in_the_recurrence_and_in_full_attention(tmp_path):
    """A head with a decay of 1 never forgets, and the differential attention has no window: a token that occurs once,
    hundreds of places back (behind several chunks, pages and key ranges), moves the last logits.  Among hundreds of
    random keys one would carry a six-hundredth of the weight, so the weights are made for it: the vocabulary's last
    eight tokens carry a large number in a channel that no other token uses and that every key row reads (and, for the
    softmax maps, every query has a constant part along the direction those keys take).  Whole, decoded from early on,
    and in portions."""
    from cisr_b200 import Stepper
    for mix in (vm.lightning(2, 24, 16, (1.0, 0.999)), vm.attention(2, 1, 32, 32, 0.6, 0.4, 8)):
        cfg = vm.one_layer(mix, None, width=64)
        weights = vm.make_weights(cfg, 6, gain=3.0)
        weights["embed"][:, 0] = 0.0
        weights["embed"][-8:, 0] = 8.0
        weights["l0.mix.k"][:, 0] = 1.0
        if mix[0] == "attention":
            weights["embed"][:, 1] = 1.0
            weights["l0.mix.q"][:, 1] = 0.5
        model = model_of(cfg, weights, tmp_path / mix[0])
        rng = np.random.default_rng(1)
        n = 600
        filler = [int(t) for t in rng.integers(0, cfg["vocab"] - 8, size=n)]
        for place in (3, 255, 256, 40):
            tokens = list(filler)
            tokens[place] = stands_out(cfg, weights, filler, place, True)
            requests, reference = {"r": tokens}, {"r": plain(cfg, weights, tokens)}
            for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 330), replay.trace_portions(requests, (250, 6, 1, 64, 130))):
                compare(replay.run_steps(Stepper(model, n_pages=40, page_size=16, max_slots=2), steps), requests, reference, "float32", scale=2.0)


def test_a_reader_with_a_wider_window_than_the_owner_of_its_rows(tmp_path):
    """The second layer reads the first one's cache rows through a wider window (and the fourth through a narrower one):
    rows that the owner's own window has passed must still be there for the reader, in long decoding, where pages go back
    one by one, as in whole prompts."""
    lat = lambda window, kv_from=None, heads=2: vm.latent(heads, 16, 8, 24, 24, 0.4, window=window, kv_from=kv_from)
    cfg = vm.model(89, 64, [vm.layer(lat(18), vm.dense(72)), vm.layer(lat(50, 0, heads=3), None),
                            vm.layer(lat(64), None), vm.layer(lat(20, 2), vm.dense(40))])
    weights = vm.make_weights(cfg, 21, gain=2.0)
    model = model_of(cfg, weights, tmp_path)
    requests = {"w": vm.random_tokens(cfg, 170, 8), "x": vm.random_tokens(cfg, 75, 9)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    narrow = json.loads(json.dumps(cfg))
    narrow["layers"][1]["mixer"]["mask"] = {"size": 18}
    assert replay.relative_rms(plain(narrow, weights, requests["w"])[-1], reference["w"][-1]) > 1e-3, "the wider window would not show"
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (1,)), replay.trace_mixed(requests, seed=1, max_live=2)):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=1), steps), requests, reference, "float32")


def test_sharp_attention_depends_on_single_keys(tmp_path_factory):
    """With the query projections scaled up the softmax is peaked: each query's weight sits on one or two keys somewhere
    in its sight (or on the sink), so a wrong, missing or stale cache row shows.  float32 only."""
    lengths = {"x": 300, "y": 170, "z": 61}
    cfg, weights, path, model, requests, reference = setup("vb", "float32", tmp_path_factory, gain=4.0, lengths=lengths)
    for steps in (replay.trace_whole(requests), replay.trace_mixed(requests, seed=3), replay.trace_tail_decode(requests, 160),
                  replay.trace_portions(requests, (16, 2, 15, 17, 3, 64, 33))):
        compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32", scale=8.0)


def test_repeated_step_shapes_replay_from_graphs_with_recurrent_state(tmp_path_factory):
    """Steps of the same shape recur: from the second time on the step is a graph replay.  The warm-up run in front of a
    capture must not advance any request's state twice."""
    from cisr_b200 import StepEntry, Stepper
    cfg, weights, path, model, _, _ = setup("va", "float32", tmp_path_factory)
    stepper = Stepper(model, n_pages=60, page_size=16, max_slots=4, graph=True)
    tokens = {k: vm.random_tokens(cfg, 131, 20 + i) for i, k in enumerate("abcd")}
    reference = {k: plain(cfg, weights, t) for k, t in tokens.items()}
    got = {}
    for k in "abcd":
        stepper.create(k)
    plan = [[("a", 0, 70)], [("b", 0, 70)], [("c", 0, 70)], [("d", 0, 70)], [("a", 70, 30)],
            [("b", 70, 20), ("a", 100, 1)], [("c", 70, 20), ("a", 101, 1)], [("d", 70, 20), ("b", 90, 1)],
            [("a", 102, 1), ("b", 91, 1)], [("a", 103, 1), ("b", 92, 1)], [("a", 104, 1), ("b", 93, 1)]]
    for step in plan:
        entries = [StepEntry(k, tokens[k][at:at + n], [n - 1, 0] if n > 1 else [0]) for k, at, n in step]
        logits = stepper.step(entries).cpu().numpy()
        row = 0
        for k, at, n in step:
            for w in ([n - 1, 0] if n > 1 else [0]):
                got[(k, at + w)] = logits[row].copy()
                row += 1
        stepper.cache.check()
    compare(got, tokens, reference, "float32")
    report = stepper.graphs.report()
    assert report["shape_entries"] >= 2 and report["hits"] >= 4


# ------------------------------------------------------------------ generation through the scheduler and the command line
@pytest.mark.parametrize("case, graph", [("va", False), ("va", True), ("vc", False)])
def test_greedy_generation_through_the_scheduler(case, graph, tmp_path_factory):
    """More requests than slots, few pages: requests wait, run in portions under a token budget, decode side by side,
    end, and their pages and slots serve the next ones.  float32 tokens equal the plain greedy choice."""
    from cisr_b200 import Engine, Request
    cfg, weights, path, model, _, _ = setup(case, "float32", tmp_path_factory)
    prompts = {f"g{i}": vm.random_tokens(cfg, n, 50 + i) for i, n in enumerate((19, 5, 40, 2, 27, 11))}
    new = 7

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(pv.forward(cfg, weights, seq)[-1].argmax()))
        return seq[len(prompt):]

    engine = Engine.for_model(model, pages=7, page_size=16, max_active=3, token_budget=24, prefill_chunk=9, policy="decode_first", graph=graph)
    for key, prompt in prompts.items():
        engine.submit(Request(key, prompt, max_new_tokens=new))
    got = {r.key: r.generated for r in engine.run()}
    assert got == {k: plain_greedy(p) for k, p in prompts.items()}
    assert not engine.stepper.cache.requests and all(g.pool.n_free == g.pool.n_pages for g in engine.stepper.cache.page_groups)


def test_command_line_and_trace_program(tmp_path_factory, tmp_path):
    cfg, weights, path, model, requests, reference = setup("vb", "float32", tmp_path_factory)
    short = {k: requests[k] for k in ("c", "f", "i", "j", "h")}
    steps = replay.trace_mixed(short, seed=5, max_live=4)
    got = replay.run_trace_program(path, "float32", steps, tmp_path / "out", replay.max_live_tokens(steps), cfg["vocab"])
    compare(got, short, reference, "float32")
    cfg16, weights16, path16, _, requests16, reference16 = setup("vb", "bfloat16", tmp_path_factory)
    short16 = {k: requests16[k] for k in short}
    got = replay.run_trace_program(path16, "bfloat16", steps, tmp_path / "out16", replay.max_live_tokens(steps), cfg["vocab"])
    compare(got, short16, reference16, "bfloat16")
    listing = tmp_path / "requests.json"
    listing.write_text(json.dumps([{"key": "only", "prompt": requests["c"][:9], "max_new_tokens": 4}]))
    proc = subprocess.run([sys.executable, "-m", "cisr_b200", "--config", "vilodra-small", "--dtype", "float32", "--requests", str(listing),
                           "--pages", "16"], capture_output=True, text=True, timeout=900, cwd=str(replay.ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout[proc.stdout.index("{"):])
    assert out["weights"] == "random-vilodra-small" and len(out["requests"][0]["generated"]) == 4
