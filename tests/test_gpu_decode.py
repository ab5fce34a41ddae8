"""GPU parity tests of the decode path, through the C ABI, against the CPU oracle.

Bars: dequantized weights and int8 activations bit-exact; router ids exact on the GPU's own logits,
weights within 1e-6; expert and layer outputs within 1e-3 relative L2 per token row
(the metric of tests/cpu/test_expert_pool.cpp:166-188 of the reference), measured at ~1e-6.
"""
import numpy as np
import pytest

from fngine_b200 import synth
from oracle import oracle as O
import patterns

pytestmark = pytest.mark.gpu

IQ3_S, IQ4_NL = 21, 20
H = 2560
TOL = 1e-3  # relative L2 per row, the bar stated for fp32 expert outputs


def _torch():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def fast_lib():
    """The reference build where it runs (AVX-512 hosts), else the scalar port: same results."""
    return O.ref()


def q8k_sums32(blocks, k):
    """Sums of every 32 codes of ggml Q8_K blocks: block_q8_K's bsums (16-code groups) added in pairs,
    int16 [k / 32]; the planar workspace rows keep them behind the scales (64 bytes after the codes)."""
    b = blocks.reshape(k // 256, 292)
    bs = b[:, 260:292].copy().view(np.int16).astype(np.int32).reshape(-1, 8, 2).sum(axis=2)
    return bs.reshape(-1).astype(np.int16)


def planar_from_blocks(act, blocks, k):
    """ggml activation blocks -> (codes int8 [k] in the workspace order, scales float32)."""
    if act == O.ACT_Q8_K:
        b = blocks.reshape(k // 256, 292)
        return b[:, 4:260].reshape(-1).view(np.int8), b[:, :4].copy().view(np.float32).reshape(-1)
    b = blocks.reshape(k // 32, 34)
    d = b[:, :2].copy().view(np.float16).astype(np.float32).reshape(-1)
    q = b[:, 2:].view(np.int8)
    order = np.array([2 * (e % 16) + e // 16 for e in range(32)])
    inter = np.empty_like(q)
    inter[:, order] = q
    return inter.reshape(-1), d


# ---------------------------------------------------------------------------------- probes
IQ3_XXS, IQ2_S, IQ4_XS, Q2_0 = O.IQ3_XXS, O.IQ2_S, O.IQ4_XS, O.Q2_0


@pytest.mark.parametrize("fmt", [IQ3_S, IQ4_NL, IQ3_XXS, IQ2_S, IQ4_XS, Q2_0])
def test_synth_device_equals_host(fmt):
    torch = _torch()
    from fngine_b200 import moe
    fmt, fd = (IQ4_NL, Q2_0) if fmt == Q2_0 else (fmt, fmt if fmt in (IQ3_S, IQ4_NL) else IQ4_NL)
    layer = moe.synth_layer(fmt, fd, 512, 3, 77)
    torch.cuda.synchronize()
    dev = layer.slots.cpu().numpy()
    for e in range(3):
        host = synth.expert_blob(fmt, fd, 512, 77, e)
        assert np.array_equal(dev[e * len(host):(e + 1) * len(host)], host)


@pytest.mark.parametrize("fmt,k", [(IQ3_S, 2560), (IQ3_S, 512), (IQ4_NL, 2560), (IQ4_NL, 640), (IQ3_XXS, 2560),
                                   (IQ2_S, 2560), (IQ4_XS, 2560), (Q2_0, 512), (Q2_0, 640)])
def test_dequant_bit_exact(fmt, k):
    torch = _torch()
    from fngine_b200 import moe
    nrows = 96
    rows = synth.fill_blocks(fmt, nrows * k // synth.BLOCK_ELEMS[fmt], 5, 31)
    got = moe.dequant_rows(fmt, torch.from_numpy(rows).cuda(), nrows, k).cpu().numpy()
    want = O.dequant_rows(fmt, rows, nrows, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("act", [O.ACT_Q8_K, O.ACT_Q8_0])
@pytest.mark.parametrize("bf16", [False, True])
def test_quantize_act_bit_exact(act, bf16):
    torch = _torch()
    from fngine_b200 import moe
    x = patterns.all_inputs(trials=64, seed=4321)
    if bf16:
        bits = synth.to_bf16_bits(x)
        x = synth.bf16_bits_to_f32(bits)
        xd = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        xd = torch.from_numpy(x).cuda()
    got = moe.quantize_act(act, xd).cpu().numpy()
    want = O.quantize_act(act, x)
    assert np.array_equal(got, want)


# ---------------------------------------------------------------------------------- router + select
def run_layer(torch, moe, layer, ws, wr, x, tokens, slot_of=None, logits=None):
    if logits is None:
        moe.router_logits(wr, x, ws.logits)
        logits = ws.logits
    moe.moe_select_publish(logits, x, slot_of, 0, None, None, tokens, ws)
    moe.moe_hot_gate_up(layer, tokens, ws)
    moe.moe_hot_down(layer, tokens, ws)
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_combine(ws, None, None, 0, None, None, None, y, tokens)
    torch.cuda.synchronize()
    return y


def check_work_list(work, ids, w, tokens, slot_of=None):
    """Invariants of the sorted work list (moe.h:87-105 of the reference)."""
    slots = ids if slot_of is None else slot_of[ids]
    distinct = sorted(set(slots.reshape(-1).tolist()))
    assert work.n_items == len(distinct) and work.n_pairs == tokens * 10 and work.n_cold == 0
    assert list(work.item_slot[:work.n_items]) == distinct
    assert work.item_pair_begin[0] == 0 and work.item_pair_begin[work.n_items] == work.n_pairs
    for it, s in enumerate(distinct):
        b, e = work.item_pair_begin[it], work.item_pair_begin[it + 1]
        toks = [t for t in range(tokens) if s in slots[t]]
        assert list(work.pair_token[b:e]) == toks  # tokens ascending inside an item
        for p, t in zip(range(b, e), toks):
            k = list(slots[t]).index(s)
            assert abs(work.pair_weight[p] - w[t, k]) <= 1e-6
    for t in range(tokens):
        assert work.token_pair_count[t] == 10
        pairs = list(work.token_pairs[t])
        assert pairs == sorted(pairs)  # slot order == pair order
        assert sorted(work.pair_token[p] for p in pairs) == [t] * 10


@pytest.mark.parametrize("tokens,bf16", [(1, False), (4, False), (16, False), (9, True)])
def test_router_and_select(tokens, bf16):
    torch = _torch()
    from fngine_b200 import moe
    wr_bits = synth.router_weights(101, rows=513)
    wr = torch.from_numpy(wr_bits.view(np.int16)).cuda().view(torch.bfloat16)
    x = synth.activations(202, tokens)
    if bf16:
        xb = synth.to_bf16_bits(x)
        x = synth.bf16_bits_to_f32(xb)
        xd = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        xd = torch.from_numpy(x).cuda()
    layer = moe.synth_layer(IQ3_S, IQ3_S, 512, 8, 1)  # only the formats matter here
    ws = moe.DecodeWorkspace(layer)
    moe.router_logits(wr, xd, ws.logits)
    logits = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)
    want = x.astype(np.float64) @ synth.bf16_bits_to_f32(wr_bits).astype(np.float64).T
    assert np.max(np.abs(logits - want)) <= 1e-4 * np.sqrt(np.mean(want ** 2))
    moe.moe_select_publish(ws.logits, xd, None, 0, None, None, tokens, ws)
    torch.cuda.synchronize()
    ids, w = O.topk(logits[:, :512])
    work = ws.work()
    got_ids = np.array([list(work.topk_expert[t]) for t in range(tokens)])
    got_w = np.array([list(work.topk_weight[t]) for t in range(tokens)])
    assert np.array_equal(got_ids, ids)
    assert np.max(np.abs(got_w - w)) <= 1e-6
    check_work_list(work, ids, w, tokens)
    # int8 activations: bit-identical to the host quantizer
    xq = ws.xq(tokens)
    for t in range(tokens):
        blocks = O.quantize_act(O.ACT_Q8_K, x[t])
        codes, scales = planar_from_blocks(O.ACT_Q8_K, blocks, H)
        assert np.array_equal(xq[t, :H].view(np.int8), codes)
        assert np.array_equal(xq[t, H:H + 40].copy().view(np.float32), scales)
        assert np.array_equal(xq[t, H + 64:H + 64 + 160].copy().view(np.int16), q8k_sums32(blocks, H))
    assert ws.status() == 0


@pytest.mark.parametrize("tokens", [1, 3, 4, 16])
def test_fused_route_agrees_with_the_separate_router(tokens):
    """The fused layer call projects the router in eight K slices met through distributed shared memory, the
    separate fb_router_logits sums 80 values per lane and then the lanes: the two agree to fp32 rounding (stated
    tolerance: 2e-6 of the logits' rms), and on these seeded inputs they select the same experts with weights
    equal to 1e-6. Row 512 (the shared-expert gate) is produced by the separate call only."""
    torch = _torch()
    from fngine_b200 import moe
    wr = torch.from_numpy(synth.router_weights(111, rows=513).view(np.int16)).cuda().view(torch.bfloat16)
    xd = torch.from_numpy(synth.activations(212 + tokens, tokens)).cuda()
    layer = moe.synth_layer(IQ3_S, IQ3_S, 512, 512, 3)
    ws = moe.DecodeWorkspace(layer)
    moe.router_logits(wr, xd, ws.logits)
    moe.moe_select_publish(ws.logits, xd, None, 0, None, None, tokens, ws)
    torch.cuda.synchronize()
    sep = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513).copy()
    w1 = ws.work()
    ids1 = np.array([list(w1.topk_expert[t]) for t in range(tokens)])
    wt1 = np.array([list(w1.topk_weight[t]) for t in range(tokens)])
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, layer, xd, ws, y)
    torch.cuda.synchronize()
    fused = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)
    w2 = ws.work()
    ids2 = np.array([list(w2.topk_expert[t]) for t in range(tokens)])
    wt2 = np.array([list(w2.topk_weight[t]) for t in range(tokens)])
    rms = float(np.sqrt(np.mean(sep[:, :512] ** 2)))
    assert np.max(np.abs(fused[:, :512] - sep[:, :512])) <= 2e-6 * rms
    assert np.array_equal(ids1, ids2) and np.max(np.abs(wt1 - wt2)) <= 1e-6
    assert ws.status() == 0


def test_select_ties_nan_and_slot_map():
    torch = _torch()
    from fngine_b200 import moe
    tokens = 3
    logits = (synth.normal(5, tokens * 513) * 0.5).astype(np.float32).reshape(tokens, 513)
    logits[0, [7, 300, 40]] = 3.0       # ties -> lower id first
    logits[1, 11] = np.nan              # NaN never wins
    logits[2, :] = 0.0                  # all equal: ids 0..9
    logits[2, 3] = -0.0
    ids, w = O.topk(logits[:, :512])
    assert list(ids[0][:3]) == [7, 40, 300] and 11 not in ids[1] and list(ids[2]) == list(range(10))
    perm = np.random.default_rng(3).permutation(512).astype(np.int32)
    layer = moe.synth_layer(IQ3_S, IQ3_S, 512, 8, 1)
    ws = moe.DecodeWorkspace(layer)
    x = torch.from_numpy(synth.activations(1, tokens)).cuda()
    for slot_of in (None, perm):
        sd = None if slot_of is None else torch.from_numpy(slot_of).cuda()
        moe.moe_select_publish(torch.from_numpy(logits).cuda(), x, sd, 0, None, None, tokens, ws)
        torch.cuda.synchronize()
        work = ws.work()
        got_ids = np.array([list(work.topk_expert[t]) for t in range(tokens)])
        assert np.array_equal(got_ids, ids)
        check_work_list(work, ids, w, tokens, slot_of)


# ---------------------------------------------------------------------------------- experts
def forced_logits(tokens, experts_per_token):
    """Router logits that make token t pick exactly experts_per_token[t] (descending preference)."""
    l = np.full((tokens, 513), -30.0, dtype=np.float32)
    for t, es in enumerate(experts_per_token):
        for r, e in enumerate(es):
            l[t, e] = 4.0 - 0.37 * r
    return l


@pytest.mark.parametrize("fg,fd,inter", [(IQ3_S, IQ3_S, 512), (IQ4_NL, IQ4_NL, 512), (IQ3_S, IQ4_NL, 640),
                                         (IQ4_NL, IQ4_NL, 640)])
def test_single_expert_rows(fg, fd, inter):
    """One token through ten experts: every h row and every weighted partial row against the CPU
    expert path on identical bytes (the single-expert case of the benchmark definition, ten times)."""
    torch = _torch()
    from fngine_b200 import moe
    n_exp = 16
    layer = moe.synth_layer(fg, fd, inter, n_exp, 4242)
    ws = moe.DecodeWorkspace(layer)
    x = synth.activations(9, 1)
    xd = torch.from_numpy(x).cuda()
    chosen = [[12, 3, 5, 0, 9, 15, 1, 7, 8, 2]]
    logits = torch.from_numpy(forced_logits(1, chosen)).cuda()
    y = run_layer(torch, moe, layer, ws, None, xd, 1, logits=logits).cpu().numpy()
    work = ws.work()
    ids, w = O.topk(forced_logits(1, chosen)[:, :512])
    hs, parts = ws.h(10), ws.partial(10)
    y_ref = np.zeros(H, dtype=np.float64)
    worst_h = worst_y = 0.0
    for it in range(work.n_items):
        e = work.item_slot[it]
        p = work.item_pair_begin[it]
        blob = synth.expert_blob(fg, fd, inter, 4242, e)
        h_ref, ye = O.expert_ffn(fg, fd, H, inter, blob, x, lib=fast_lib())
        wt = float(w[0][list(ids[0]).index(e)])
        worst_h = max(worst_h, rel_l2(hs[p], h_ref[0]))
        worst_y = max(worst_y, rel_l2(parts[p], wt * ye[0]))
        y_ref += wt * ye[0].astype(np.float64)
    assert worst_h <= TOL and worst_y <= TOL, (worst_h, worst_y)
    assert rel_l2(y[0], y_ref) <= TOL
    assert ws.status() == 0
    print("single expert rows: max rel h %.2e, partial %.2e, y %.2e" % (worst_h, worst_y, rel_l2(y[0], y_ref)))


def oracle_layer(fg, fd, inter, seed, x, ids, w):
    """CPU layer over only the experts that were selected (blobs regenerated on the host)."""
    used = sorted(set(ids.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    blobs = np.concatenate([synth.expert_blob(fg, fd, inter, seed, e) for e in used])
    ids2 = np.vectorize(remap.get)(ids).astype(np.int32)
    stride = synth.blob_bytes(fg, fd, inter)
    return O.moe_layer(fg, fd, H, inter, blobs, stride, x, ids2, w, threads=8, lib=fast_lib())


@pytest.mark.parametrize("fg,fd,inter,tokens", [(IQ3_S, IQ3_S, 512, 1), (IQ3_S, IQ3_S, 512, 4),
                                                (IQ3_S, IQ3_S, 512, 16), (IQ4_NL, IQ4_NL, 512, 1),
                                                (IQ4_NL, IQ4_NL, 512, 8), (IQ3_S, IQ4_NL, 640, 5)])
def test_moe_layer_decode(fg, fd, inter, tokens):
    """The MoE layer of the benchmark definition: 512 experts, bf16 router ~ N(0, 0.02), top-10."""
    torch = _torch()
    from fngine_b200 import moe
    seed = 1000 + inter + fg
    layer = moe.synth_layer(fg, fd, inter, 512, seed)
    ws = moe.DecodeWorkspace(layer)
    wr_bits = synth.router_weights(303, rows=512)
    wr = torch.from_numpy(wr_bits.view(np.int16)).cuda().view(torch.bfloat16)
    x = synth.activations(404 + tokens, tokens)
    xd = torch.from_numpy(x).cuda()
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, layer, xd, ws, y)
    torch.cuda.synchronize()
    y1 = y.cpu().numpy()
    logits = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)[:, :512]
    ids, w = O.topk(logits)
    work = ws.work()
    assert np.array_equal(np.array([list(work.topk_expert[t]) for t in range(tokens)]), ids)
    want = oracle_layer(fg, fd, inter, seed, x, ids, w)
    errs = [rel_l2(y1[t], want[t]) for t in range(tokens)]
    assert max(errs) <= TOL, errs
    assert ws.status() == 0
    # repeated calls are bitwise identical (fixed reduction order)
    moe.moe_layer_decode(wr, layer, xd, ws, y)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy().view(np.uint32), y1.view(np.uint32))
    # the fused layer call equals the reference's five-call sequence on the same logits
    y5 = run_layer(torch, moe, layer, ws, None, xd, tokens, logits=ws.logits.clone())
    assert np.array_equal(y5.cpu().numpy().view(np.uint32), y1.view(np.uint32))
    print("layer fmt %d/%d inter %d T=%d: distinct experts %d, max rel L2 %.2e" %
          (fg, fd, inter, tokens, work.n_items, max(errs)))


@pytest.mark.parametrize("fg,fd,inter,tokens", [(IQ3_XXS, IQ4_NL, 512, 3), (IQ2_S, IQ4_NL, 640, 9), (IQ4_XS, Q2_0, 512, 16),
                                                (IQ2_S, Q2_0, 640, 1), (IQ3_S, Q2_0, 512, 5), (IQ4_NL, Q2_0, 640, 7)])
def test_moe_layer_decode_in_the_other_formats(fg, fd, inter, tokens):
    """The reference's other expert formats (IQ3_XXS / IQ2_S / IQ4_XS gate/up, Q2_0 down) through the same layer
    call, against the CPU expert path on identical bytes (the oracle is pinned to the reference build for them)."""
    torch = _torch()
    from fngine_b200 import moe
    seed = 2000 + inter + fg
    layer = moe.synth_layer(fg, fd, inter, 512, seed)
    ws = moe.DecodeWorkspace(layer)
    wr = torch.from_numpy(synth.router_weights(305, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    x = synth.activations(504 + tokens, tokens)
    xd = torch.from_numpy(x).cuda()
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, layer, xd, ws, y)
    torch.cuda.synchronize()
    y1 = y.cpu().numpy()
    logits = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)[:, :512]
    ids, w = O.topk(logits)
    work = ws.work()
    assert np.array_equal(np.array([list(work.topk_expert[t]) for t in range(tokens)]), ids)
    want = oracle_layer(fg, fd, inter, seed, x, ids, w)
    errs = [rel_l2(y1[t], want[t]) for t in range(tokens)]
    assert max(errs) <= TOL, errs
    assert ws.status() == 0
    # the fused layer call equals the reference's five-call sequence on the same logits
    y5 = run_layer(torch, moe, layer, ws, None, xd, tokens, logits=ws.logits.clone())
    assert np.array_equal(y5.cpu().numpy().view(np.uint32), y1.view(np.uint32))
    print("layer fmt %d/%d inter %d T=%d: distinct experts %d, max rel L2 %.2e" % (fg, fd, inter, tokens, work.n_items, max(errs)))


@pytest.mark.parametrize("fg,fd", [(IQ3_S, IQ3_S), (IQ4_NL, IQ4_NL)])
def test_crowded_experts_and_h_requantization(fg, fd):
    """All 16 tokens on the same ten experts (more tokens per expert than one pass holds), and the
    re-quantized h of every pair bit-identical to the host quantizer applied to the GPU's own h."""
    torch = _torch()
    from fngine_b200 import moe
    tokens, inter = 16, 512
    layer = moe.synth_layer(fg, fd, inter, 32, 77)
    ws = moe.DecodeWorkspace(layer)
    chosen = [[(3 * i + r) % 32 for i in range(10)] for r in (0,) * 11 + (1, 1, 1, 2, 2)]
    lg = forced_logits(tokens, chosen)
    x = synth.activations(55, tokens)
    y = run_layer(torch, moe, layer, ws, None, torch.from_numpy(x).cuda(), tokens,
                  logits=torch.from_numpy(lg).cuda()).cpu().numpy()
    ids, w = O.topk(lg[:, :512])
    want = oracle_layer(fg, fd, inter, 77, x, ids, w)
    errs = [rel_l2(y[t], want[t]) for t in range(tokens)]
    assert max(errs) <= TOL, errs
    work = ws.work()
    assert max(work.item_pair_begin[i + 1] - work.item_pair_begin[i] for i in range(work.n_items)) >= 11
    act = O.ACT_OF[fd]
    hs, hq = ws.h(work.n_pairs), ws.hq(work.n_pairs)
    nscale = inter // (256 if act == O.ACT_Q8_K else 32)
    for p in range(work.n_pairs):
        blocks = O.quantize_act(act, hs[p])
        codes, scales = planar_from_blocks(act, blocks, inter)
        assert np.array_equal(hq[p, :inter].view(np.int8), codes)
        assert np.array_equal(hq[p, inter:inter + 4 * nscale].copy().view(np.float32), scales)
        if act == O.ACT_Q8_K:
            assert np.array_equal(hq[p, inter + 64:inter + 64 + inter // 16].copy().view(np.int16), q8k_sums32(blocks, inter))
    assert ws.status() == 0


def test_combine_shared_residual_and_ablation():
    """y_shared, the 4-stream residual write X += inj * y and the rank-1 ablation of the routed part
    (moe.h:144-158 of the reference)."""
    torch = _torch()
    from fngine_b200 import moe
    tokens = 3
    layer = moe.synth_layer(IQ3_S, IQ3_S, 512, 16, 5)
    ws = moe.DecodeWorkspace(layer)
    lg = forced_logits(tokens, [[(t + i) % 16 for i in range(10)] for t in range(tokens)])
    x = torch.from_numpy(synth.activations(3, tokens)).cuda()
    y0 = run_layer(torch, moe, layer, ws, None, x, tokens, logits=torch.from_numpy(lg).cuda())
    ysh = torch.from_numpy(synth.activations(4, tokens) * 1e5).cuda()
    inj = torch.from_numpy(synth.normal(6, tokens * 4).astype(np.float32).reshape(tokens, 4)).cuda()
    X0 = torch.from_numpy(synth.normal(7, tokens * 4 * H).astype(np.float32).reshape(tokens, 4, H)).cuda()
    X = X0.clone()
    r = torch.from_numpy(synth.normal(8, H).astype(np.float32)).cuda()
    r = r / r.norm()
    yo = torch.empty_like(y0)
    moe.moe_combine(ws, ysh, None, 0, None, inj, X, yo, tokens, 0, r, 0.75)
    torch.cuda.synchronize()
    routed = y0.double() - 0.75 * r.double()[None, :] * (y0.double() @ r.double())[:, None]
    want = routed + ysh.double()
    assert rel_l2(yo.cpu().numpy(), want.cpu().numpy()) <= 1e-5
    wantX = X0.double() + inj.double()[:, :, None] * want[:, None, :]
    assert rel_l2(X.cpu().numpy(), wantX.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("tokens,aux", [(1, False), (5, True), (16, True)])
def test_forward_moe_decode_with_shared_expert(tokens, aux):
    """The whole decode branch of Forward::moe (src/model/forward.cpp:333,356-376 of the reference):
    513-row router, routed experts, the FP8-row shared expert (SwiGlu, then SharedScale with the
    shared-gate logit) on a side stream, combine with the residual write. Checked against the CPU
    expert path plus an fp64 shared expert over the represented weights, 1e-3 relative per token."""
    torch = _torch()
    from fngine_b200 import linear, moe
    seed, inter = 4242, 512
    layer = moe.synth_layer(IQ3_S, IQ3_S, inter, 512, seed)
    ws = moe.DecodeWorkspace(layer)
    wr = torch.from_numpy(synth.router_weights(909, rows=513).view(np.int16)).cuda().view(torch.bfloat16)
    gu_c, gu_s = synth.fp8_row_weight(31, 1280, H)
    dn_c, dn_s = synth.fp8_row_weight(32, H, 640)
    gu_s = gu_s * np.float32(10.0)  # gate and up values of order one, so that the shared part matters
    shared = moe.SharedExpert(
        linear.Fp8RowWeight(torch.from_numpy(gu_c).cuda(), torch.from_numpy(gu_s).cuda().to(torch.bfloat16)),
        linear.Fp8RowWeight(torch.from_numpy(dn_c).cuda(), torch.from_numpy(dn_s).cuda().to(torch.bfloat16)))
    xb = synth.to_bf16_bits(synth.activations(77 + tokens, tokens))
    x = synth.bf16_bits_to_f32(xb)
    xd = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    inj = torch.from_numpy(synth.normal(61, tokens * 4).astype(np.float32).reshape(tokens, 4)).cuda()
    X0 = torch.from_numpy(synth.normal(62, tokens * 4 * H).astype(np.float32).reshape(tokens, 4, H)).cuda()
    X = X0.clone()
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    side = torch.cuda.Stream() if aux else None
    moe.forward_moe_decode(wr, shared, layer, xd, ws, inj, X, y, aux_stream=side)
    torch.cuda.synchronize()
    assert ws.status() == 0
    logits = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)
    ids, w = O.topk(logits[:, :512])
    routed = oracle_layer(IQ3_S, IQ3_S, inter, seed, x, ids, w).astype(np.float64)
    widen = lambda sc: synth.bf16_bits_to_f32(synth.to_bf16_bits(sc))  # the row scales as the GPU holds them (bf16)
    h = O.linear_fp8_a16(xb, gu_c, widen(gu_s), kind="swiglu")
    hb = synth.to_bf16_bits(h.astype(np.float32))  # h is stored as bf16 between the two projections
    ysh = O.linear_fp8_a16(hb, dn_c, widen(dn_s), kind="shared_scale", gate_logit=logits[:, 512])
    # the shared expert on its own (it is small beside the routed sum of these synthetic experts)
    h_gpu = synth.bf16_bits_to_f32(shared.h[:tokens].view(torch.int16).cpu().numpy().view(np.uint16))
    assert float(np.mean(h_gpu == synth.bf16_bits_to_f32(hb))) >= 0.99
    ysh_gpu = shared.y[:tokens].cpu().numpy()
    assert max(rel_l2(ysh_gpu[t], ysh[t]) for t in range(tokens)) <= TOL
    want = routed + ysh
    got = y.cpu().numpy()
    errs = [rel_l2(got[t], want[t]) for t in range(tokens)]
    assert max(errs) <= TOL, errs
    wantX = X0.cpu().numpy().astype(np.float64) + inj.cpu().numpy().astype(np.float64)[:, :, None] * want[:, None, :]
    assert rel_l2(X.cpu().numpy(), wantX) <= 1e-5
    print("forward moe decode T=%d: shared/routed norm %.2f, max rel L2 %.2e" %
          (tokens, float(np.linalg.norm(ysh) / np.linalg.norm(routed)), max(errs)))


@pytest.mark.parametrize("fg,fd,inter", [(IQ3_S, IQ3_S, 512), (IQ3_S, IQ4_NL, 640)])
def test_layers_read_from_a_pack_and_from_gguf(fg, fd, inter, tmp_path):
    """Expert bytes written as a pack (manifest.json + experts.bin, 4096-aligned stride) and as GGUF expert
    tensors, read back by fngine_b200.pack and put in HBM, give the decode layer's result bit for bit as
    the same bytes generated in place, and match the CPU expert path."""
    torch = _torch()
    from fngine_b200 import moe, pack
    n_exp, tokens, seed = 16, 3, 606
    blobs = np.stack([synth.expert_blob(fg, fd, inter, seed, e) for e in range(n_exp)])
    info = pack.layer_info(fg, fd, H, inter, 0)
    assert blobs.shape[1] == info.blob_bytes and info.blob_stride > info.blob_bytes
    pack.write_expert_pack(str(tmp_path / "pack"), H, inter, [(fg, fd, blobs)])
    gate, up, down = blobs[:, :info.gate_bytes], blobs[:, info.gate_bytes:2 * info.gate_bytes], blobs[:, 2 * info.gate_bytes:]
    pack.write_gguf(str(tmp_path / "experts.gguf"),
                    [("blk.0.ffn_gate_exps.weight", [H, inter, n_exp], fg, np.ascontiguousarray(gate)),
                     ("blk.0.ffn_up_exps.weight", [H, inter, n_exp], fg, np.ascontiguousarray(up)),
                     ("blk.0.ffn_down_exps.weight", [inter, H, n_exp], fd, np.ascontiguousarray(down))])
    lg = forced_logits(tokens, [[(5 * t + i) % n_exp for i in range(10)] for t in range(tokens)])
    x = synth.activations(17, tokens)
    xd, ld = torch.from_numpy(x).cuda(), torch.from_numpy(lg).cuda()
    results = []
    for layer in (moe.synth_layer(fg, fd, inter, n_exp, seed),
                  pack.ExpertPack.open(str(tmp_path / "pack")).load_layer(0),
                  pack.GgufExperts(str(tmp_path / "experts.gguf")).load_layer(0)):
        ws = moe.DecodeWorkspace(layer)
        results.append(run_layer(torch, moe, layer, ws, None, xd, tokens, logits=ld).cpu().numpy())
        assert ws.status() == 0
    assert np.array_equal(results[1].view(np.uint32), results[0].view(np.uint32))
    assert np.array_equal(results[2].view(np.uint32), results[0].view(np.uint32))
    ids, w = O.topk(lg[:, :512])
    want = oracle_layer(fg, fd, inter, seed, x, ids, w)
    assert max(rel_l2(results[1][t], want[t]) for t in range(tokens)) <= TOL
    # a shard of the pack: experts 8..15 as slots 0..7
    shard = pack.ExpertPack.open(str(tmp_path / "pack")).load_layer(0, first=8, count=8)
    assert shard.n_slots == 8 and shard.layout.blob_stride == info.blob_stride


def test_host_entry_point_matches_device_path():
    torch = _torch()
    from fngine_b200 import moe
    tokens = 4
    layer = moe.synth_layer(IQ3_S, IQ3_S, 512, 512, 9)
    ws = moe.DecodeWorkspace(layer)
    wr = torch.from_numpy(synth.router_weights(303, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    xh = torch.from_numpy(synth.activations(12, tokens)).pin_memory()
    yh = torch.empty(tokens, H, dtype=torch.float32).pin_memory()
    xd = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    yd = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode_host(wr, layer, xh, ws, xd, yd, yh)
    y2 = torch.empty_like(yd)
    moe.moe_layer_decode(wr, layer, xh.cuda(), ws, y2)
    torch.cuda.synchronize()
    assert np.array_equal(yh.numpy().view(np.uint32), y2.cpu().numpy().view(np.uint32))
    # a pageable result buffer takes the copy instead of the direct write: same bits
    yp = torch.empty(tokens, H, dtype=torch.float32)
    moe.moe_layer_decode_host(wr, layer, xh, ws, xd, yd, yp)
    assert np.array_equal(yp.numpy().view(np.uint32), y2.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("world", [2, 8])
def test_expert_parallel_shards_on_one_gpu(world):
    """The expert-parallel entry points, with the ranks played one after another on a single GPU:
    each rank's shard (its own slot array and slot map) gives partial rows, the rank-order sum equals
    the single-GPU layer (same routing) within summation-order noise and the CPU oracle within 1e-3."""
    torch = _torch()
    from fngine_b200 import ep, moe
    tokens, seed = 16, 5000
    wr = torch.from_numpy(synth.router_weights(303, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    x = synth.activations(77, tokens)
    xd = torch.from_numpy(x).cuda()
    full = moe.synth_layer(IQ3_S, IQ3_S, 512, 512, seed)
    ws = moe.DecodeWorkspace(full)
    y_full = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, full, xd, ws, y_full)
    torch.cuda.synchronize()
    parts = torch.empty(world, tokens, H, dtype=torch.float32, device="cuda")
    n_local = 0
    for r in range(world):
        shard = ep.EpDecodeLayer(r, world, seed)
        ep.layer_decode_ep(wr, shard, xd, ws, parts[r])
        torch.cuda.synchronize()
        wk = ws.work()
        n_local += wk.n_pairs
        assert wk.n_cold == tokens * 10 - wk.n_pairs and ws.status() == 0
    assert n_local == tokens * 10  # every pair is computed by exactly one rank
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    ep.sum_ranks(parts, y)
    torch.cuda.synchronize()
    got, ref = y.cpu().numpy(), y_full.cpu().numpy()
    assert max(rel_l2(got[t], ref[t]) for t in range(tokens)) <= 1e-6
    logits = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)[:, :512]
    ids, w = O.topk(logits)
    want = oracle_layer(IQ3_S, IQ3_S, 512, seed, x, ids, w)
    assert max(rel_l2(got[t], want[t]) for t in range(tokens)) <= TOL


def test_decode_shards_from_a_placement_plan():
    """Decode over shards that follow a placement plan instead of contiguous ranges (experts spread over four
    ranks by a routing average, fngine_b200/placement.py): each rank's slot map comes from the plan, the ranks
    are played one after another on a single GPU, and the rank-order sum equals the single-GPU layer."""
    torch = _torch()
    from types import SimpleNamespace

    from fngine_b200 import ep, moe, placement
    tokens, seed, world = 16, 5003, 4
    wr = torch.from_numpy(synth.router_weights(304, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    xd = torch.from_numpy(synth.activations(78, tokens)).cuda()
    full = moe.synth_layer(IQ3_S, IQ3_S, 512, 512, seed)
    ws = moe.DecodeWorkspace(full)
    y_full = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, full, xd, ws, y_full)
    torch.cuda.synchronize()
    # a routing average with a few hot experts, as decode traffic has; no copies at decode (a copy would be
    # streamed by two ranks in the same step)
    avg = placement.RoutingEma(1).update(np.bincount(np.asarray(ws.work().topk_expert).reshape(-1)[:tokens * 10],
                                                      minlength=512).astype(np.uint32)[None, :])[0] + 0.01
    plan = placement.plan_placement(avg, world, 128)
    assert all(len(c) == 1 for c in plan.copies) and plan.imbalance(avg) <= placement.Placement.contiguous(world).imbalance(avg)
    parts = torch.empty(world, tokens, H, dtype=torch.float32, device="cuda")
    n_local = 0
    for r in range(world):
        shard = SimpleNamespace(layer=moe.synth_layer_of(IQ3_S, IQ3_S, 512, plan.rank_experts[r], seed),
                                slot_of=torch.from_numpy(plan.slot_map(r)).cuda())
        ep.layer_decode_ep(wr, shard, xd, ws, parts[r])
        torch.cuda.synchronize()
        n_local += ws.work().n_pairs
        assert ws.status() == 0
    assert n_local == tokens * 10
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    ep.sum_ranks(parts, y)
    torch.cuda.synchronize()
    got, ref = y.cpu().numpy(), y_full.cpu().numpy()
    assert max(rel_l2(got[t], ref[t]) for t in range(tokens)) <= 1e-6


def test_peer_exchange_layer_with_one_rank_equals_the_plain_layer():
    """fb_moe_layer_decode_ep_p2p with a world of one rank: the rank is its own peer, so the publish /
    wait / partial-row / rank-order-sum machinery runs on one GPU (nobody else is waited for) and must
    reproduce fb_moe_layer_decode bit for bit, step after step, on both buffer parities."""
    torch = _torch()
    import ctypes as C

    from fngine_b200 import ep, lib as fblib, moe
    tokens, seed = 16, 5000
    wr = torch.from_numpy(synth.router_weights(303, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    full = moe.synth_layer(IQ3_S, IQ3_S, 512, 512, seed)
    ws = moe.DecodeWorkspace(full)
    slot_of = torch.arange(512, dtype=torch.int32, device="cuda")
    lib = fblib.load()
    bufs = [torch.zeros(lib.fb_ep_exchange_bytes(k), dtype=torch.uint8, device="cuda") for k in (0, 1)]
    xchg = ep.PeerExchange.__new__(ep.PeerExchange)
    xchg.rank, xchg.world, xchg.step, xchg.local = 0, 1, 0, bufs
    xchg.peers = fblib.EpPeers()
    xchg.peers.rank, xchg.peers.n_ranks = 0, 1
    xchg.peers.x_all[0], xchg.peers.y_parts[0] = (b.data_ptr() for b in bufs)
    shard = C.Structure.__new__(C.Structure) if False else type("S", (), {})()
    shard.layer, shard.slot_of = full, slot_of
    y_ref = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    for step in range(3):
        xd = torch.from_numpy(synth.activations(80 + step, tokens)).cuda()
        moe.moe_layer_decode(wr, full, xd, ws, y_ref)
        torch.cuda.synchronize()
        ep.layer_decode_ep_p2p(wr, shard, xd, ws, xchg, y)
        torch.cuda.synchronize()
        assert ws.status() == 0
        assert torch.equal(y, y_ref)


def test_peer_wait_that_nobody_answers_runs_out_and_is_reported():
    """A bounded device-side wait actually running out (the reference has the same test for its CPU
    exchange, tests/kernels/moe/test_moe_exchange.cpp:286-307): a two-rank peer-exchange step on ONE GPU
    whose second rank does not exist. Both "ranks'" buffers are local, zeroed, and nobody publishes
    rank 1's rows, so every reader of those lines gives up after the (shortened) poll limit: the call
    returns, the status word says FB_STATUS_PIPELINE_TIMEOUT, nothing faults or hangs, and the library
    keeps working - a plain layer on a fresh workspace right afterwards is bit-exact."""
    torch = _torch()
    from fngine_b200 import ep, lib as fblib, moe
    tokens, seed = 16, 5000
    lib = fblib.load()
    wr = torch.from_numpy(synth.router_weights(303, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    full = moe.synth_layer(IQ3_S, IQ3_S, 512, 512, seed)
    ws = moe.DecodeWorkspace(full)
    x = torch.from_numpy(synth.activations(80, tokens)).cuda()
    y_ref = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, full, x, ws, y_ref)
    torch.cuda.synchronize()
    assert ws.status() == 0

    bufs = [[torch.zeros(lib.fb_ep_exchange_bytes(k), dtype=torch.uint8, device="cuda") for k in (0, 1)] for _ in range(2)]
    xchg = ep.PeerExchange.__new__(ep.PeerExchange)
    xchg.rank, xchg.world, xchg.step = 0, 2, 0
    xchg.peers = fblib.EpPeers()
    xchg.peers.rank, xchg.peers.n_ranks = 0, 2
    for d in range(2):
        xchg.peers.x_all[d], xchg.peers.y_parts[d] = (b.data_ptr() for b in bufs[d])
    shard = type("S", (), {})()
    shard.layer = full  # rank 0 of 2 would hold experts 0..255; every slot is resident here, which is harmless
    shard.slot_of = torch.arange(512, dtype=torch.int32, device="cuda")
    ws2 = moe.DecodeWorkspace(full)
    y = torch.empty(tokens // 2, H, dtype=torch.float32, device="cuda")
    lib.fb_ep_set_wait_limit(2000)  # a fraction of a millisecond per awaited line
    try:
        ep.layer_decode_ep_p2p(wr, shard, x[: tokens // 2].contiguous(), ws2, xchg, y)
        torch.cuda.synchronize()
    finally:
        lib.fb_ep_set_wait_limit(0)
    assert ws2.status() == fblib.STATUS_PIPELINE_TIMEOUT
    # the context is intact and the kernels still give the same bits
    ws3 = moe.DecodeWorkspace(full)
    y2 = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, full, x, ws3, y2)
    torch.cuda.synchronize()
    assert ws3.status() == 0 and torch.equal(y2, y_ref)


@pytest.mark.parametrize("fg,fd,inter", [(IQ3_S, IQ3_S, 512), (IQ4_NL, IQ4_NL, 512), (IQ3_S, IQ4_NL, 640)])
def test_workspace_without_a_layout_gives_the_same_bits(fg, fd, inter):
    """The reference makes its decode workspace from a base address alone (make_moe_decode_workspace,
    src/kernels/moe/moe.h:117) and its selection does not see the expert layout. A workspace made that way
    (NULL layout) must drive select -> gate/up -> down -> combine to the same bits as one made for the
    layout; the selection then writes the tokens' Q8_K and Q8_0 rows both."""
    torch = _torch()
    from fngine_b200 import moe
    tokens = 7
    layer = moe.synth_layer(fg, fd, inter, 512, 909)
    wr = torch.from_numpy(synth.router_weights(41, rows=513).view(np.int16)).cuda().view(torch.bfloat16)
    x = torch.from_numpy(synth.to_bf16_bits(synth.activations(42, tokens)).view(np.int16)).cuda().view(torch.bfloat16)
    outs = []
    for ws in (moe.DecodeWorkspace(layer), moe.DecodeWorkspace(None)):
        y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
        moe.router_logits(wr, x, ws.logits)
        moe.moe_select_publish(ws.logits, x, None, 0, None, None, tokens, ws)
        moe.moe_hot_gate_up(layer, tokens, ws)
        moe.moe_hot_down(layer, tokens, ws)
        moe.moe_combine(ws, None, None, 0, None, None, None, y, tokens)
        torch.cuda.synchronize()
        assert ws.status() == 0
        outs.append(y)
    assert torch.equal(outs[0], outs[1])
    both = moe.DecodeWorkspace(None)
    moe.router_logits(wr, x, both.logits)
    moe.moe_select_publish(both.logits, x, None, 0, None, None, tokens, both)
    torch.cuda.synchronize()
    xf = synth.bf16_bits_to_f32(synth.to_bf16_bits(synth.activations(42, tokens)))
    for act in (O.ACT_Q8_K, O.ACT_Q8_0):
        rows = both.xq(tokens, act)
        for t in range(tokens):
            codes, scales = planar_from_blocks(act, O.quantize_act(act, xf[t]), H)
            assert np.array_equal(rows[t, :H].view(np.int8), codes)
            assert np.array_equal(rows[t, H:H + 4 * len(scales)].copy().view(np.float32), scales)


@pytest.mark.skipif(not O.pool_available(), reason="the reference's cpu::ExpertPool is not built on this host")
def test_decode_layer_against_the_reference_expert_pool():
    """The GPU decode layer at the reference's native shape (IQ3_S gate/up, IQ4_NL down, intermediate 640,
    bf16 tokens) against the reference's production CPU tier, cpu::ExpertPool, run through its own host
    exchange on the same tokens, experts and routing weights."""
    torch = _torch()
    from fngine_b200 import moe
    tokens, inter, seed = 9, 640, 2027
    layer = moe.synth_layer(IQ3_S, IQ4_NL, inter, 512, seed)
    ws = moe.DecodeWorkspace(layer)
    wr = torch.from_numpy(synth.router_weights(515, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    xb = synth.to_bf16_bits(synth.activations(516, tokens))
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    y = torch.empty(tokens, H, dtype=torch.float32, device="cuda")
    moe.moe_layer_decode(wr, layer, x, ws, y)
    torch.cuda.synchronize()
    assert ws.status() == 0
    logits = ws.logits.cpu().numpy()[:tokens * 513].reshape(tokens, 513)[:, :512]
    ids, w = O.topk(logits)
    used = sorted(set(ids.reshape(-1).tolist()))
    stride = synth.blob_bytes(IQ3_S, IQ4_NL, inter)
    blobs = np.concatenate([synth.expert_blob(IQ3_S, IQ4_NL, inter, seed, e) for e in used])
    local = np.vectorize({e: i for i, e in enumerate(used)}.get)(ids).astype(np.int32)
    want = O.pool_decode_step(IQ3_S, IQ4_NL, blobs, stride, xb, local, w)
    got = y.cpu().numpy()
    err = max(rel_l2(got[t], want[t]) for t in range(tokens))
    print("decode layer vs cpu::ExpertPool (inter 640, IQ3_S + IQ4_NL): max rel L2 %.2e" % err)
    assert err <= TOL, err
