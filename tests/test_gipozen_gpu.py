"""Gipozen through the engine against the plain implementation (tests/plain_gipozen.py).

Each mechanism alone (the rows of the convolved projections with their kept inputs, the combination of the two maps,
the seam kernel of the depth average, PolyNorm, the gated activation, the softmax router with its correction and
identity experts, one-layer models on every attention kernel), then whole models under every way of cutting and
batching: whole prompts, prefill against token-by-token decoding, portions down to one and two tokens, unequal requests
side by side with pages and slots used again, long decoding, the first tokens of a sequence, tokens made to stand out
just inside and just outside the window and the kept first keys, and greedy generation through the scheduler, the
command line and the trace program.
"""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import gipozen_models as gm
import plain_gipozen as pg
import replay

pytestmark = pytest.mark.gpu
F = torch.float64
LENGTHS = {"a": 150, "b": 70, "c": 33, "d": 200, "e": 90, "f": 3, "g": 129, "h": 64, "i": 47, "j": 1}
_cache = {}


# ------------------------------------------------------------------ helpers
def plain(cfg, weights, tokens):
    return pg.forward(cfg, weights, tokens).numpy()


def setup(case, dtype, tmp_path_factory, gain=1.0, lengths=None, choice=None):
    """`choice` False: the same model with routers that take every output (bfloat16 runs of whole models: a close call
    between two experts would send a token down another path than the plain implementation's)."""
    choice = dtype == "float32" if choice is None else choice
    key = (case, dtype, gain, choice, None if lengths is None else tuple(sorted(lengths.items())))
    if key not in _cache:
        from cisr_b200 import Model

        cfg, seed = gm.CASES[case]
        if not choice:
            cfg = gm.no_choice(cfg)
        weights = gm.make_weights(cfg, seed, gain=gain)
        path = gm.write_model_dir(tmp_path_factory.mktemp(f"{case}_{dtype}"), cfg, weights)
        model = Model.from_pretrained(path, dtype=dtype)
        requests = {rid: gm.random_tokens(cfg, n, 100 + i) for i, (rid, n) in enumerate((lengths or LENGTHS).items())}
        reference = {rid: plain(cfg, weights, tokens) for rid, tokens in requests.items()}
        _cache[key] = (cfg, weights, path, model, requests, reference)
    return _cache[key]


def compare(got, requests, reference, dtype, scale=4.0):
    return replay.compare(got, requests, reference, dtype, scale=scale)


def stepper_for(model, steps, slack_pages=0):
    from cisr_b200 import Stepper
    return Stepper(model, n_pages=replay.max_live_tokens(steps) // 16 + slack_pages, page_size=16, max_slots=4)


def model_of(cfg, weights, tmp_path, dtype="float32"):
    from cisr_b200 import Model
    return Model.from_pretrained(gm.write_model_dir(tmp_path, cfg, weights), dtype=dtype)


def dev(a):
    return torch.from_numpy(np.asarray(a, dtype=np.int32)).cuda()


# ------------------------------------------------------------------ each mechanism alone: kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, dk, dv, taps, write", [(4, 2, 24, 40, 3, True), (2, 1, 32, 64, 4, True), (3, 3, 10, 12, 1, True),
                                                          (2, 2, 6, 25, 2, True), (1, 1, 64, 96, 5, True), (4, 2, 24, 40, 3, False),
                                                          (6, 3, 16, 24, 2, False)])
def test_rows_of_the_convolved_projections(dtype, hq, hkv, dk, dv, taps, write):
    """The convolution with kept inputs, the layout of the two maps' query rows and the key and value rows in their
    pages: two requests in portions down to one token (shorter than the taps), rows of a step not in slot order, one
    request in a slot that held another's inputs before, pages scattered over the pool.  `write` False: a layer that
    reads another's keys and values convolves its queries only and touches no page."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(hq * 100 + dk)
    width = -(-max(2 * dk, dv) // 16) * 16
    nq, nk, nv = hq * 2 * dk, hkv * 2 * dk, hkv * dv
    channels = nq + (nk + nv if write else 0)
    extra = 7                                             # columns after the convolved ones (the gate's) stay untouched
    conv_w = torch.randn(channels, taps, generator=g)
    lengths = {0: 37, 1: 12}
    us = {r: torch.randn(n, channels + extra, generator=g) for r, n in lengths.items()}
    want = {r: pg.causal_conv(u[:, :channels].to(F), conv_w.to(F)) for r, u in us.items()}
    page, n_pages, table_width = 8, 11, 6
    slot = {0: 2, 1: 0}
    table = np.full((4, table_width), -1, dtype=np.int32)
    table[2, :5] = [9, 3, 7, 0, 5]
    table[0, :2] = [4, 10]
    state = torch.randn(4, max(taps - 1, 1), channels, generator=g).cuda()
    for s in slot.values():
        state[s].zero_()
    k_cache = torch.full((n_pages, hkv, page, width), 9.0, dtype=dtype, device="cuda")
    v_cache = torch.full((n_pages, hkv, page, width), 9.0, dtype=dtype, device="cuda")
    cuts = {0: [5, 1, 1, 2, 9, 1, 18], 1: [1, 1, 3, 7]}
    at, got = {0: 0, 1: 0}, {0: [], 1: []}
    while any(cuts.values()):
        batch = [r for r in (1, 0) if cuts[r]]
        sizes = [cuts[r].pop(0) for r in batch]
        proj = torch.cat([us[r][at[r]:at[r] + n] for r, n in zip(batch, sizes)]).cuda().contiguous()
        q_start = np.cumsum([0] + sizes[:-1]).astype(np.int32)
        token_req = np.concatenate([np.full(n, i, dtype=np.int32) for i, n in enumerate(sizes)])
        positions = np.concatenate([np.arange(at[r], at[r] + n, dtype=np.int32) for r, n in zip(batch, sizes)])
        q = torch.full((proj.shape[0], 2 * hq, width), 7.0, dtype=dtype, device="cuda")
        req_slot = dev([slot[r] for r in batch])
        kernels.diff_rows(proj, conv_w.t().contiguous().cuda(), taps, state, token_req=dev(token_req), req_slot=req_slot, q_start=dev(q_start),
                          positions=dev(positions), q_out=q, k_cache=k_cache if write else None, v_cache=v_cache if write else None,
                          block_table=dev(table), page_size=page, hq=hq, hkv=hkv, key_dim=dk, value_dim=dv)
        kernels.conv_keep(proj, state, req_slot, dev(q_start), dev(sizes), len(batch), taps, channels)
        for i, (r, n) in enumerate(zip(batch, sizes)):
            got[r].append(q[q_start[i]:q_start[i] + n].float().cpu())
            at[r] += n
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for r, n in lengths.items():
        q = torch.cat(got[r]).view(n, hq, 2, width)
        ref = want[r][:, :nq].view(n, hq, 2, dk)
        for m in (0, 1):
            assert (q[:, :, m, m * dk:(m + 1) * dk].to(F) - ref[:, :, m]).abs().max() < tol * ref.abs().max()
            outside = torch.ones(width, dtype=torch.bool)
            outside[m * dk:(m + 1) * dk] = False
            assert float(q[:, :, m, outside].abs().max()) == 0.0, "a query row has numbers where the other map's keys lie"
        if not write:
            continue
        pages = torch.tensor(table[slot[r]][: -(-n // page)].astype(np.int64))
        k = k_cache[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, hkv, width)[:n]        # [positions, kv heads, D]
        v = v_cache[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, hkv, width)[:n]
        ref_k = want[r][:, nq:nq + nk].view(n, hkv, 2 * dk)
        ref_v = want[r][:, nq + nk:].view(n, hkv, dv)
        assert (k[:, :, :2 * dk].to(F) - ref_k).abs().max() < tol * ref_k.abs().max()
        assert (v[:, :, :dv].to(F) - ref_v).abs().max() < tol * ref_v.abs().max()
        assert float(k[:, :, 2 * dk:].abs().sum()) == 0.0 and float(v[:, :, dv:].abs().sum()) == 0.0
    if write:
        assert float(k_cache[[1, 2, 6, 8]].float().min()) == 9.0, "a page of no request was written"
    else:
        assert float(k_cache.float().min()) == 9.0 and float(v_cache.float().min()) == 9.0
    assert float(state[1].abs().sum()) > 0 and float(state[3].abs().sum()) > 0        # other slots keep what they held


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, dk, dv, taps, first, second", [
    (16, 4, 8, 16, 4, [900, 1, 2, 1100], [1, 1500, 3, 500]),     # sixteen tokens per CTA
    (4, 2, 24, 40, 3, [400, 2, 1, 300], [2, 5, 350, 1]),          # a few tokens per CTA
    (16, 4, 7, 16, 8, [1000, 3, 1000], [7, 6, 2000]),             # as many taps as a lane carries; an odd key width
    (16, 4, 8, 16, 9, [1000, 3, 1000], [7, 6, 2000]),             # more taps than a lane carries
    (16, 4, 8, 16, 1, [1000, 3, 1000], [7, 6, 2000])])
def test_rows_of_a_large_step(dtype, hq, hkv, dk, dv, taps, first, second):
    """A step of many tokens gives a CTA several neighbouring tokens, of whichever requests: portions that begin in the
    middle of a CTA's tokens, portions shorter than the taps beside long ones, and a second step that goes on from the
    kept inputs of the first."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(taps * 10 + hq)
    width = -(-max(2 * dk, dv) // 16) * 16
    nq, nk, nv = hq * 2 * dk, hkv * 2 * dk, hkv * dv
    channels = nq + nk + nv
    conv_w = torch.randn(channels, taps, generator=g)
    lengths = [a + b for a, b in zip(first, second)]
    us = [torch.randn(n, channels + 3, generator=g) for n in lengths]
    want = [pg.causal_conv(u[:, :channels].to(F), conv_w.to(F)) for u in us]
    page = 16
    per = [-(-n // page) for n in lengths]
    n_pages = sum(per)
    order = torch.randperm(n_pages, generator=g).numpy().astype(np.int32)
    table = np.full((len(lengths), max(per)), -1, dtype=np.int32)
    used = 0
    for r, n in enumerate(per):
        table[r, :n] = order[used:used + n]
        used += n
    state = torch.zeros(len(lengths), max(taps - 1, 1), channels).cuda()
    k_cache = torch.zeros(n_pages, hkv, page, width, dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    at, got = [0] * len(lengths), [[] for _ in lengths]
    for sizes in (first, second):
        proj = torch.cat([us[r][at[r]:at[r] + n] for r, n in enumerate(sizes)]).cuda().contiguous()
        q_start = np.cumsum([0] + sizes[:-1]).astype(np.int32)
        token_req = np.concatenate([np.full(n, r, dtype=np.int32) for r, n in enumerate(sizes)])
        positions = np.concatenate([np.arange(at[r], at[r] + n, dtype=np.int32) for r, n in enumerate(sizes)])
        q = torch.full((proj.shape[0], 2 * hq, width), 7.0, dtype=dtype, device="cuda")
        req_slot = dev(np.arange(len(sizes)))
        kernels.diff_rows(proj, conv_w.t().contiguous().cuda(), taps, state, token_req=dev(token_req), req_slot=req_slot,
                          q_start=dev(q_start), positions=dev(positions), q_out=q, k_cache=k_cache, v_cache=v_cache,
                          block_table=dev(table), page_size=page, hq=hq, hkv=hkv, key_dim=dk, value_dim=dv)
        kernels.conv_keep(proj, state, req_slot, dev(q_start), dev(sizes), len(sizes), taps, channels)
        for r, n in enumerate(sizes):
            got[r].append(q[q_start[r]:q_start[r] + n].float().cpu())
            at[r] += n
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for r, n in enumerate(lengths):
        q = torch.cat(got[r]).view(n, hq, 2, width)
        ref = want[r][:, :nq].view(n, hq, 2, dk)
        for m in (0, 1):
            assert (q[:, :, m, m * dk:(m + 1) * dk].to(F) - ref[:, :, m]).abs().max() < tol * ref.abs().max()
            outside = torch.ones(width, dtype=torch.bool)
            outside[m * dk:(m + 1) * dk] = False
            assert float(q[:, :, m, outside].abs().max()) == 0.0
        pages = torch.tensor(table[r][:per[r]].astype(np.int64))
        k = k_cache[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, hkv, width)[:n]
        v = v_cache[pages].float().cpu().permute(0, 2, 1, 3).reshape(-1, hkv, width)[:n]
        ref_k = want[r][:, nq:nq + nk].view(n, hkv, 2 * dk)
        ref_v = want[r][:, nq + nk:].view(n, hkv, dv)
        assert (k[:, :, :2 * dk].to(F) - ref_k).abs().max() < tol * ref_k.abs().max()
        assert (v[:, :, :dv].to(F) - ref_v).abs().max() < tol * ref_v.abs().max()
        assert float(k[:, :, 2 * dk:].abs().sum()) == 0.0 and float(v[:, :, dv:].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, hq, dv, width", [(5, 4, 40, 48), (130, 2, 96, 128), (3, 3, 12, 32), (64, 1, 25, 32), (9, 8, 64, 64),
                                                   (7, 2, 320, 320), (33, 2, 250, 256)])
def test_combination_of_the_two_maps(dtype, tokens, hq, dv, width):
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(tokens + dv)
    mixed = torch.randn(tokens, 2 * hq, width, generator=g).to(dtype)
    cols, gate_col = 11 + hq * dv + 3, 11
    gate = torch.randn(tokens, cols, generator=g) * 2
    lam, eps, out_scale = 0.37, 1e-3, 0.45
    out = torch.empty((tokens, hq * dv), dtype=dtype, device="cuda")
    kernels.diff_combine(mixed.cuda(), gate.cuda(), gate_col, out, hq, dv, lam, eps, out_scale)
    a = mixed.to(F).view(tokens, hq, 2, width)[..., :dv]
    o = pg.rms(a[:, :, 0] - lam * a[:, :, 1], eps) * out_scale * torch.sigmoid(gate[:, gate_col:gate_col + hq * dv].to(F).view(tokens, hq, dv))
    err = (out.float().cpu().to(F).view(tokens, hq, dv) - o).abs().max()
    assert err < (2e-6 if dtype == torch.float32 else 8e-3) * o.abs().max()


@pytest.mark.parametrize("h_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("entries, tokens, hidden", [(4, 9, 80), (2, 1, 52), (7, 33, 128), (3, 5, 1000)])
def test_seam_of_the_depth_average(h_dtype, entries, tokens, hidden):
    """Layer after layer: the history gains the layer's result, the stream becomes the weighted sum of everything so far,
    and the next layer's normed input comes out of the same launch; with picked rows nothing is stored."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(entries * 10 + hidden)
    hist = torch.zeros(entries + 1, tokens, hidden, device="cuda")
    results = [torch.randn(tokens, hidden, generator=g)]
    hist[0].copy_(results[0])
    x = results[0].clone().cuda()
    eps = 1e-5
    tol = 2e-6 if h_dtype == torch.float32 else 8e-3
    for i in range(entries):
        delta_a, delta_b = torch.randn(tokens, hidden, generator=g), torch.randn(tokens, hidden, generator=g)
        x += delta_a.cuda()                                    # the mixer's output, added inside the layer
        w = torch.randn(i + 2, generator=g)
        norm_w = 1 + 0.2 * torch.randn(hidden, generator=g)
        results.append((x.cpu().to(F) + delta_b.to(F)))
        mixed = sum(w[j].to(F) * results[j].to(F) for j in range(i + 2))
        normed = pg.rms(mixed, eps) * norm_w.to(F)
        rows = dev([tokens - 1, 0])
        picked = torch.empty((2, hidden), dtype=h_dtype, device="cuda")
        before = (hist.clone(), x.clone())
        kernels.depth_mix_norm(hist, x, delta_b.cuda(), w.cuda(), i + 1, norm_w=norm_w.cuda(), eps=eps, h=picked, rows=rows)
        assert torch.equal(hist, before[0]) and torch.equal(x, before[1]), "picked rows must store nothing"
        assert (picked.float().cpu().to(F) - normed[[tokens - 1, 0]]).abs().max() < tol * normed.abs().max()
        h = torch.empty((tokens, hidden), dtype=h_dtype, device="cuda")
        also = torch.empty((tokens, hidden), device="cuda")
        kernels.depth_mix_norm(hist, x, delta_b.cuda(), w.cuda(), i + 1, norm_w=norm_w.cuda(), eps=eps, h=h, mixed_out=also)
        assert (hist[i + 1].cpu().to(F) - results[i + 1]).abs().max() < 2e-6 * results[i + 1].abs().max()
        assert (x.cpu().to(F) - mixed).abs().max() < 4e-6 * max(1.0, float(mixed.abs().max())) and torch.equal(also, x)
        assert (h.float().cpu().to(F) - normed).abs().max() < tol * normed.abs().max()
    assert float(hist[entries].abs().sum()) > 0


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, ff, out_cols", [(7, 136, 136), (1, 50, 56), (130, 1000, 1000), (3, 9, 16)])
def test_polynorm_kernel(out_dtype, tokens, ff, out_cols):
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(ff)
    z = torch.randn(tokens, ff, generator=g) * 1.7
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    out = torch.full((tokens, out_cols), 5.0, dtype=out_dtype, device="cuda")
    kernels.polynorm(z.cuda(), coef.cuda(), 1e-5, out)
    ref = pg.polynorm(z.to(F), coef.to(F), 1e-5)
    got = out.float().cpu().to(F)
    assert (got[:, :ff] - ref).abs().max() < (3e-6 if out_dtype == torch.float32 else 8e-3) * ref.abs().max()
    assert float(got[:, ff:].abs().sum()) == 0.0


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, ff, out_cols, scaled", [(6, 40, 40, False), (2, 24, 24, True), (257, 96, 96, True), (5, 9, 16, False)])
def test_gated_activation_kernel(out_dtype, rows, ff, out_cols, scaled):
    """Both clamps bite (the inputs reach well beyond the limit on both sides); the gate has no lower clamp."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(rows + ff)
    gu = torch.randn(rows, 2 * ff + 1, generator=g) * 2
    limit = 0.9
    out = torch.full((rows, out_cols), 5.0, dtype=out_dtype, device="cuda")
    kernels.gated_clamp(gu.cuda(), ff, limit, out, scale_col=2 * ff if scaled else -1)
    gate = torch.clamp(gu[:, :ff].to(F), max=limit)
    up = torch.clamp(gu[:, ff:2 * ff].to(F), -limit, limit)
    ref = gate * torch.sigmoid(pg.GELU_FREE_ALPHA * gate) * (up + 1.0)
    if scaled:
        ref = ref * torch.sigmoid(gu[:, 2 * ff:].to(F))
    assert float(gu[:, :ff].min()) < -2 * limit and float(gate.min()) < -2 * limit
    got = out.float().cpu().to(F)
    assert (got[:, :ff] - ref).abs().max() < (2e-6 if out_dtype == torch.float32 else 8e-3) * ref.abs().max()
    assert float(got[:, ff:].abs().sum()) == 0.0


def expert_part(dtype, hidden, ff, experts, top, identity, limit, shared, tensors):
    from cisr_b200.config import PartSpec
    from cisr_b200.config.gipozen import EXPERT_NAMES
    from cisr_b200.ops import build
    from cisr_b200.parts import FEED_FORWARDS, build_part
    part = build_part(FEED_FORWARDS, PartSpec("routed_experts", {
        "hidden_size": hidden, "expert_size": ff, "experts": experts, "top": top, "identity": identity, "scores": "softmax", "choice_bias": True,
        "activation": "gated_clamp", "limit": limit, "shared": shared, "names": EXPERT_NAMES}), dtype, "feed-forward")
    build.compile_many(part.kernel_jobs())
    part.load({k: v.to(dtype).cuda() for k, v in tensors.items()})
    return part


def expert_tensors(g, hidden, ff, experts, identity, shared, correction=0.2):
    outputs = experts + identity
    w = {"router": 3.0 / hidden ** 0.5 * torch.randn(outputs, hidden, generator=g), "correction": correction * torch.randn(outputs, generator=g)}
    for e in range(experts):
        w[f"e{e}.gate"] = 1.5 / hidden ** 0.5 * torch.randn(ff, hidden, generator=g)
        w[f"e{e}.up"] = 1.5 / hidden ** 0.5 * torch.randn(ff, hidden, generator=g)
        w[f"e{e}.down"] = torch.randn(hidden, ff, generator=g) / ff ** 0.5
    if shared:
        fs = shared["size"]
        w.update({"shared.gate": 1.5 / hidden ** 0.5 * torch.randn(fs, hidden, generator=g), "shared.up": 1.5 / hidden ** 0.5 * torch.randn(fs, hidden, generator=g),
                  "shared.down": torch.randn(hidden, fs, generator=g) / fs ** 0.5, "shared.sg": torch.randn(1, hidden, generator=g) / hidden ** 0.5})
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, identity, top, hidden", [(5, 2, 2, 80), (3, 0, 1, 72), (10, 3, 2, 176), (4, 1, 5, 64), (1, 3, 2, 40), (16, 0, 4, 128)])
def test_softmax_router_with_correction(dtype, experts, identity, top, hidden):
    """The choice is made by score + correction and the weights are the scores without it: the corrections are drawn
    wide enough that they change the choice for many tokens (checked), inputs equal to the bit."""
    g = torch.Generator().manual_seed(experts * 100 + top)
    tensors = expert_tensors(g, hidden, 8, experts, identity, None, correction=0.3)
    h = torch.randn(57, hidden, generator=g).to(dtype)
    w64 = {k: v.to(F) for k, v in tensors.items()}
    want_ids, scores = pg.route(w64, "", h.to(F), top)
    plain_ids = torch.argsort(scores, dim=-1, descending=True, stable=True)[:, :top]
    if top < experts + identity:
        assert not torch.equal(plain_ids.sort(dim=-1).values, want_ids.sort(dim=-1).values), "the correction changes no choice: the test would show nothing"
    part = expert_part(dtype, hidden, 8, experts, top, identity, 1.0, None, tensors)
    chosen, weight = part.route(h.cuda())
    assert torch.equal(chosen.cpu().long(), want_ids), "the router chose other outputs"
    assert torch.allclose(weight.cpu().to(F), torch.gather(scores, 1, want_ids), rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, experts, identity, top, ff, hidden, shared", [
    (1, 4, 2, 2, 40, 72, None), (13, 5, 2, 2, 40, 80, (24, 0.8)), (150, 3, 0, 1, 56, 64, None), (400, 4, 1, 2, 64, 128, (32, 2.0)),
    (700, 3, 2, 5, 24, 56, (20, 1.0)), (3, 10, 3, 2, 80, 176, (48, 2.0)), (2, 1, 3, 4, 9, 20, None),
    (512, 2, 1, 2, 200, 128, None), (2048, 4, 0, 2, 520, 128, (64, 1.5))])
def test_gated_experts_with_identity_and_shared_experts(dtype, tokens, experts, identity, top, ff, hidden, shared):
    """The whole feed-forward part against the plain one with the part's own choice of experts handed to the plain sum (so
    no close call decides): few tokens (a warp per output feature) and many (sorted by expert, grouped tensor-core
    products in bfloat16 with the activation as the first one's epilogue: one column tile, several with a ragged last
    one, and enough row tiles for the wide tile form), identity experts among the chosen, the shared expert with its
    per-token factor."""
    g = torch.Generator().manual_seed(tokens + experts)
    limit = 0.7
    shared_spec = {"size": shared[0], "limit": shared[1]} if shared else None
    tensors = expert_tensors(g, hidden, ff, experts, identity, shared_spec)
    part = expert_part(dtype, hidden, ff, experts, top, identity, limit, shared_spec, tensors)
    h = torch.randn(tokens, hidden, generator=g).to(dtype)
    chosen, weight = part.route(h.cuda())
    got = part.forward(h.cuda(), None).cpu().to(F)
    w64 = {k: v.to(F) for k, v in tensors.items()}
    h64 = h.to(F)
    want = torch.zeros(tokens, hidden, dtype=F)
    took_identity = 0
    for t in range(tokens):
        for k in range(top):
            e = int(chosen[t, k])
            took_identity += e >= experts
            y = pg.gated_expert(w64, f"e{e}.", h64[t:t + 1], limit)[0] if e < experts else h64[t]
            want[t] += float(weight[t, k]) * y
    if shared:
        want += torch.sigmoid(h64 @ w64["shared.sg"].T) * pg.gated_expert(w64, "shared.", h64, shared[1])
    assert identity == 0 or took_identity > 0 or tokens < 4
    err = (got - want).abs().max() / want.abs().max()
    assert err < (3e-6 if dtype == torch.float32 else 1.2e-2), f"relative error {err:.2e}"
    from cisr_b200.ops import kernels
    kernels.raise_if_kernel_gave_up()


# ------------------------------------------------------------------ each mechanism alone: one-layer models
def one_attention(dim, vdim, window, keep_first, heads=4, kv_heads=2, conv=3, diff=0.4, scale=None, width=128):
    return gm.one_layer(gm.mixer(heads, kv_heads, dim, vdim, scale or dim ** -0.5, conv=conv, diff=diff, window=window, keep_first=keep_first),
                        width=width)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim, vdim, window, keep_first, conv", [(32, 64, 45, 7, 3), (64, 128, 131, 20, 2), (24, 40, 17, 3, 3), (48, 80, None, None, 4),
                                                                 (80, 160, 64, 70, 1), (32, 30, 3, 2, 2), (16, 112, 150, 1, 3), (128, 8, 33, 0, 2)])
def test_every_attention_kernel_has_the_window_and_the_kept_first_keys(dtype, dim, vdim, window, keep_first, conv, tmp_path):
    """One layer is the whole model; prompts long enough for every prompt kernel (128-query tensor-memory tiles at row
    widths 64 and 128, 64-query tiles at the others, the CUDA cores in float32 and beyond 128) and decoding for the split
    kernels and their merge.  Keys kept first that a kernel forgot show directly: the test first makes sure that the
    plain logits without them differ far beyond the bound."""
    cfg = one_attention(dim, vdim, window, keep_first)
    weights = gm.make_weights(cfg, dim + vdim)
    model = model_of(cfg, weights, tmp_path, dtype)
    requests = {"p": gm.random_tokens(cfg, 300, 1), "q": gm.random_tokens(cfg, 140, 2)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    if keep_first:
        other_cfg = json.loads(json.dumps(cfg))
        other_cfg["layers"][0]["mixer"]["mask"]["keep_first"] = 0
        moved = replay.relative_rms(plain(other_cfg, weights, requests["p"])[-1], reference["p"][-1])
        if dtype == "float32" or window <= 3:
            assert moved > (1e-3 if dtype == "float32" else 0.06), "the kept first keys would not show in this test"
    for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 20), replay.trace_portions(requests, (130, 2, 64, 1))):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=2), steps), requests, reference, dtype, scale=2.0)


@pytest.mark.parametrize("mlp", [gm.dense(136), gm.dense(50), gm.moe(40, 1.5, 5, 7, identity=2, shared=(24, 0.8)), gm.moe(56, 0.7, 3, 1), None])
def test_one_layer_with_each_feed_forward_and_the_stream_after_it(mlp, tmp_path):
    """The stream that the layer hands on (after the depth average, which also weights the embedding) against the plain
    one, through the engine's layer probe; then the logits."""
    from cisr_b200 import StepEntry, Stepper
    cfg = gm.model(101, 72, [gm.layer(gm.mixer(3, 1, 12, 20, 0.3, conv=2, diff=0.35, window=19, keep_first=4), mlp),
                             gm.layer(gm.mixer(3, 1, 12, 20, 0.25, conv=3, diff=0.5, window=8, keep_first=0, kv_from=0), mlp)])
    weights = gm.make_weights(cfg, 11)
    model = model_of(cfg, weights, tmp_path)
    tokens = gm.random_tokens(cfg, 45, 5)
    want = pg.layers_of(cfg, weights, tokens)
    got = []
    model.layer_probe = lambda i, stream: got.append(stream.total().cpu().to(F))
    stepper = Stepper(model, n_pages=4, page_size=16, max_slots=1)
    stepper.create("s")
    logits = stepper.step([StepEntry("s", tokens, list(range(45)))]).cpu().numpy()
    model.layer_probe = None
    assert len(got) == 2
    for i in range(2):
        assert (got[i] - want[i]).abs().max() < 1e-5 * want[i].abs().max(), f"the stream after layer {i} differs"
    compare({("s", p): logits[p] for p in range(45)}, {"s": tokens}, {"s": plain(cfg, weights, tokens)}, "float32")


# ------------------------------------------------------------------ whole models under every cut
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(gm.CASES))
def test_whole_prompts(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_whole(requests)
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(gm.CASES))
def test_prefill_against_token_by_token_decoding(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_tail_decode(requests, 60)           # the windows of ga and gc pass over decoded tokens only
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case, sizes", [("ga", (16, 2, 15, 17, 3, 64, 33)), ("gb", (2, 2, 1, 5)), ("gc", (128, 7, 2, 130)), ("ga", (1,)), ("gb", (2,))])
def test_portions_of_several_sizes(case, sizes, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    if max(sizes) <= 5:
        requests = {k: requests[k] for k in ("b", "c", "f", "j")}
    steps = replay.trace_portions(requests, sizes)
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(gm.CASES))
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_mixed(requests, seed=7)
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
    cfg, weights, path, model, requests, reference = setup("ga", "float32", tmp_path_factory)
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


def test_long_decoding_through_windows(tmp_path_factory):
    """330 tokens one by one from the first: every window passes over decoded tokens many times, pages behind the
    windows go back to their pools while the request lives, and the pages of the kept first keys stay."""
    cfg, weights, path, model, _, _ = setup("ga", "float32", tmp_path_factory)
    requests = {"long": gm.random_tokens(cfg, 330, 77)}
    reference = {"long": plain(cfg, weights, requests["long"])}
    steps = replay.trace_portions(requests, (1,))
    stepper = stepper_for(model, steps)
    compare(replay.run_steps(stepper, steps), requests, reference, "float32")
    for g in stepper.cache.page_groups:
        assert g.pool.peak <= -(-g.use.window // 16) + 1 + -(-g.use.keep_first // 16), "a window kept pages it had passed"


def test_first_tokens_of_a_sequence(tmp_path_factory):
    """Positions 0, 1, 2, ...: the convolution's zeros before the sequence, windows that are not full yet, kept first
    keys that are still inside the window, a softmax over a single key; whole, in two-token portions and one by one,
    also with nothing wanted in a step."""
    cfg, weights, path, model, _, _ = setup("ga", "float32", tmp_path_factory)
    requests = {f"s{n}": gm.random_tokens(cfg, n, 300 + n) for n in (1, 2, 3, 4, 6, 9)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (2,)), replay.trace_portions(requests, (1,))):
        compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32")
    nothing_wanted = [{"step": 0, "entries": [{"id": "s9", "tokens": requests["s9"][:5], "want": []}], "end": []},
                      {"step": 1, "entries": [{"id": "s9", "tokens": requests["s9"][5:], "want": [3]}], "end": ["s9"]}]
    got = replay.run_steps(stepper_for(model, nothing_wanted), nothing_wanted)
    assert list(got) == [("s9", 8)]
    compare(got, requests, reference, "float32")


@pytest.mark.parametrize("taps", [1, 3])
def test_tokens_just_inside_and_just_outside_the_window_and_the_kept_first_keys(taps, tmp_path):
    """One layer is the whole model, so the last position sees exactly its window and the kept first keys.  A token
    reaches the keys of its own place and of the next taps - 1 places.  A token that occurs nowhere else is put where
    only the oldest tap of the window's oldest key sees it, and one place earlier (nothing sees it); at the last kept
    place, and one place later.  The plain implementation says that the first of each pair moves the last logits and
    the second does not move them at all; the engine must agree with the prompt whole, decoded (the window passing page
    borders on the way) and in portions that cut at the edges."""
    from cisr_b200 import Stepper
    window, keep, n = 37, 21, 150
    cfg = one_attention(32, 32, window, keep, conv=taps, scale=0.1, width=64)
    weights = gm.make_weights(cfg, 5)
    model = model_of(cfg, weights, tmp_path)
    rng = np.random.default_rng(0)
    filler = [int(t) for t in rng.integers(0, cfg["vocab"] - 8, size=n)]
    without = plain(cfg, weights, filler)[-1]
    oldest_seen = n - window                              # the oldest key inside the last position's window
    for place, seen in ((oldest_seen - (taps - 1), True), (oldest_seen - taps, False), (keep - 1, True), (keep, False), (0, True), (n - 1, True)):
        effect = {}
        for b in range(cfg["vocab"] - 8, cfg["vocab"]):
            tokens = list(filler)
            tokens[place] = b
            effect[b] = replay.relative_rms(plain(cfg, weights, tokens)[-1], without)
        key = max(effect, key=effect.get)
        if seen:
            assert effect[key] > 1e-3, f"a token at {place} does not matter: the test would show nothing"
        else:
            assert effect[key] == 0.0, f"a token at {place}, beyond the window and the kept keys, moved the plain logits"
        tokens = list(filler)
        tokens[place] = key
        requests, reference = {"r": tokens}, {"r": plain(cfg, weights, tokens)}
        for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 60),
                      replay.trace_portions(requests, (keep, 1, oldest_seen - keep - 1, 2, window - 2, 1)),
                      replay.trace_portions(requests, (keep - 1, 2, oldest_seen - keep, window - 1, 5))):
            compare(replay.run_steps(Stepper(model, n_pages=12, page_size=16, max_slots=2), steps), requests, reference, "float32", scale=1.0)


def test_a_reader_with_a_wider_mask_than_the_owner_of_its_keys(tmp_path):
    """The second layer reads the first one's keys and values through a wider window and more kept first keys (and the
    fourth through a narrower one): pages that the owner's own mask has passed must still be there for the reader, in
    long decoding, where pages go back one by one, as in whole prompts."""
    mix = lambda window, keep, kv_from=None: gm.mixer(2, 1, 16, 32, 0.3, conv=2, diff=0.4, window=window, keep_first=keep, kv_from=kv_from)
    cfg = gm.model(89, 64, [gm.layer(mix(18, 3), gm.dense(72)), gm.layer(mix(50, 35, 0), None),
                            gm.layer(mix(64, 40), None), gm.layer(mix(20, 2, 2), gm.dense(40))])
    weights = gm.make_weights(cfg, 21, gain=2.0)
    model = model_of(cfg, weights, tmp_path)
    requests = {"w": gm.random_tokens(cfg, 170, 8), "x": gm.random_tokens(cfg, 75, 9)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    narrow = json.loads(json.dumps(cfg))
    narrow["layers"][1]["mixer"]["mask"] = {"size": 18, "keep_first": 3}
    assert replay.relative_rms(plain(narrow, weights, requests["w"])[-1], reference["w"][-1]) > 1e-3, "the wider mask would not show"
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (1,)), replay.trace_mixed(requests, seed=1, max_live=2)):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=1), steps), requests, reference, "float32")


def test_sharp_attention_depends_on_single_keys(tmp_path_factory):
    """With the query and key projections scaled up the softmax is peaked: each query's weight sits on one or two keys
    somewhere in its window or among the kept first ones, so a wrong, missing or stale cache row shows.  float32 only."""
    lengths = {"x": 300, "y": 170, "z": 61}
    cfg, weights, path, model, requests, reference = setup("gb", "float32", tmp_path_factory, gain=4.0, lengths=lengths)
    for steps in (replay.trace_whole(requests), replay.trace_mixed(requests, seed=3), replay.trace_tail_decode(requests, 160),
                  replay.trace_portions(requests, (16, 2, 15, 17, 3, 64, 33))):
        compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32", scale=8.0)


def test_repeated_step_shapes_replay_from_graphs_with_kept_inputs(tmp_path_factory):
    """Steps of the same shape recur: from the second time on the step is a graph replay.  The warm-up run in front of a
    capture must not move any request's kept convolution inputs twice."""
    from cisr_b200 import StepEntry, Stepper
    cfg, weights, path, model, _, _ = setup("ga", "float32", tmp_path_factory)
    stepper = Stepper(model, n_pages=60, page_size=16, max_slots=4, graph=True)
    tokens = {k: gm.random_tokens(cfg, 131, 20 + i) for i, k in enumerate("abcd")}
    reference = {k: plain(cfg, weights, t) for k, t in tokens.items()}
    got = {}
    for k in "abcd":
        stepper.create(k)
    plan = [[("a", 0, 50)], [("b", 0, 50)], [("c", 0, 50)], [("d", 0, 50)], [("a", 50, 50)],
            [("b", 50, 40), ("a", 100, 1)], [("c", 50, 40), ("a", 101, 1)], [("d", 50, 40), ("b", 90, 1)],
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
@pytest.mark.parametrize("case, graph", [("ga", False), ("ga", True), ("gc", False)])
def test_greedy_generation_through_the_scheduler(case, graph, tmp_path_factory):
    """More requests than slots, few pages: requests wait, run in portions under a token budget, decode side by side,
    end, and their pages and slots serve the next ones.  float32 tokens equal the plain greedy choice."""
    from cisr_b200 import Engine, Request
    cfg, weights, path, model, _, _ = setup(case, "float32", tmp_path_factory)
    prompts = {f"g{i}": gm.random_tokens(cfg, n, 50 + i) for i, n in enumerate((19, 5, 40, 2, 27, 11))}
    new = 7

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(pg.forward(cfg, weights, seq)[-1].argmax()))
        return seq[len(prompt):]

    engine = Engine.for_model(model, pages=7, page_size=16, max_active=3, token_budget=24, prefill_chunk=9, policy="decode_first", graph=graph)
    for key, prompt in prompts.items():
        engine.submit(Request(key, prompt, max_new_tokens=new))
    got = {r.key: r.generated for r in engine.run()}
    assert got == {k: plain_greedy(p) for k, p in prompts.items()}
    assert not engine.stepper.cache.requests and all(g.pool.n_free == g.pool.n_pages for g in engine.stepper.cache.page_groups)


def test_command_line_and_trace_program(tmp_path_factory, tmp_path):
    cfg, weights, path, model, requests, reference = setup("gb", "float32", tmp_path_factory)
    short = {k: requests[k] for k in ("c", "f", "i", "j", "h")}
    steps = replay.trace_mixed(short, seed=5, max_live=4)
    got = replay.run_trace_program(path, "float32", steps, tmp_path / "out", replay.max_live_tokens(steps), cfg["vocab"])
    compare(got, short, reference, "float32")
    cfg16, weights16, path16, _, requests16, reference16 = setup("gb", "bfloat16", tmp_path_factory)
    short16 = {k: requests16[k] for k in short}
    got = replay.run_trace_program(path16, "bfloat16", steps, tmp_path / "out16", replay.max_live_tokens(steps), cfg["vocab"])
    compare(got, short16, reference16, "bfloat16")
    listing = tmp_path / "requests.json"
    listing.write_text(json.dumps([{"key": "only", "prompt": requests["c"][:9], "max_new_tokens": 4}]))
    proc = subprocess.run([sys.executable, "-m", "cisr_b200", "--config", "gipozen-small", "--dtype", "float32", "--requests", str(listing),
                           "--pages", "16"], capture_output=True, text=True, timeout=900, cwd=str(replay.ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout[proc.stdout.index("{"):])
    assert out["weights"] == "random-gipozen-small" and len(out["requests"][0]["generated"]) == 4
