"""Expert-parallel host logic on CPU ranks (gloo, world size 2): ownership maps, dispatch, combine
ordering, and what happens when a rank does not show up. The expert math on each rank is the CPU
oracle, so only the exchange logic of fngine_b200/ep.py is under test here."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fngine_b200 import ep, synth
from oracle import oracle as O

IQ3_S, H, INTER, T, SEED = 21, 2560, 512, 4, 321


def test_ownership_maps():
    for world in (1, 2, 4, 8):
        owners = [ep.owner_of(e, world) for e in range(512)]
        assert owners == sorted(owners) and owners.count(0) == 512 // world
        seen = np.zeros(512, dtype=int)
        for r in range(world):
            m = ep.local_slot_map(r, world)
            mine = np.nonzero(m >= 0)[0]
            assert list(m[mine]) == list(range(512 // world))
            assert all(ep.owner_of(int(e), world) == r for e in mine)
            seen[mine] += 1
        assert (seen == 1).all()
        assert [ep.token_range(r, world, 16) for r in range(world)][-1][1] == 16
    with pytest.raises(ValueError):
        ep.token_range(0, 3, 16)


def _routing():
    x = synth.activations(11, T)
    logits = (synth.normal(12, T * 512) * 2).astype(np.float32).reshape(T, 512)
    ids, w = O.topk(logits)
    return x, ids, w


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, ids, w = _routing()
    lo, hi = ep.token_range(rank, world, T)
    x_all = ep.dispatch(torch.from_numpy(x[lo:hi].copy()), world)
    assert np.array_equal(x_all.numpy(), x)  # every rank sees all tokens, in owner order
    slot = ep.local_slot_map(rank, world)
    part = np.zeros((T, H), dtype=np.float32)
    for t in range(T):
        for e in sorted(ids[t].tolist()):  # ascending expert id == ascending local slot
            if slot[e] < 0:
                continue
            k = list(ids[t]).index(e)
            _, ye = O.expert_ffn(IQ3_S, IQ3_S, H, INTER, synth.expert_blob(IQ3_S, IQ3_S, INTER, SEED, e), x_all[t].numpy(),
                                 lib=O.ref())
            part[t] += w[t, k] * ye[0]
    parts = ep.combine_exchange(torch.from_numpy(part), world)
    assert tuple(parts.shape) == (world, T // world, H)
    y = ep.combine_sum(parts)
    np.save(os.path.join(out_dir, "y%d.npy" % rank), y.numpy())
    dist.destroy_process_group()


def test_two_rank_layer_equals_single_rank(tmp_path):
    mp.spawn(_rank_main, args=(2, 29611, str(tmp_path)), nprocs=2, join=True)
    x, ids, w = _routing()
    used = sorted(set(ids.reshape(-1).tolist()))
    blobs = np.concatenate([synth.expert_blob(IQ3_S, IQ3_S, INTER, SEED, e) for e in used])
    ids2 = np.vectorize({e: i for i, e in enumerate(used)}.get)(ids).astype(np.int32)
    want = O.moe_layer(IQ3_S, IQ3_S, H, INTER, blobs, synth.blob_bytes(IQ3_S, IQ3_S, INTER), x, ids2, w, threads=4,
                       lib=O.ref())
    got = np.concatenate([np.load(os.path.join(str(tmp_path), "y%d.npy" % r)) for r in range(2)])
    err = max(np.linalg.norm(got[t] - want[t]) / np.linalg.norm(want[t]) for t in range(T))
    assert err <= 1e-5, err


def _absent_rank_main(rank, world, port, out_dir):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    if rank == 1:  # this rank leaves between steps without joining the next dispatch
        dist.destroy_process_group()
        return
    try:
        ep.dispatch(torch.zeros(2, H), world)
        outcome = "returned"
    except Exception as e:  # the collective ends with an error instead of waiting forever
        outcome = "error:" + type(e).__name__
    open(os.path.join(out_dir, "outcome.txt"), "w").write(outcome)


def test_missing_rank_ends_the_collective_with_an_error(tmp_path):
    mp.spawn(_absent_rank_main, args=(2, 29612, str(tmp_path)), nprocs=2, join=True)
    assert open(os.path.join(str(tmp_path), "outcome.txt")).read().startswith("error:")


# ---------------------------------------------------------------------------------- prefill (all-to-all-v)
from fngine_b200 import ep_prefill  # noqa: E402

TP = 6  # tokens of the prefill exchange test (3 per rank)


def test_prefill_dispatch_plan():
    rng = np.random.default_rng(5)
    for world in (1, 2, 4, 8):
        ids = np.stack([rng.choice(512, size=10, replace=False) for _ in range(17)]).astype(np.int32)
        send_tok, counts, row_of = ep_prefill.plan_dispatch(torch.from_numpy(ids), world)
        per = 512 // world
        want = [(d, t) for d in range(world) for t in range(17) if (ids[t] // per == d).any()]
        got, pos = [], 0
        for d in range(world):
            for _ in range(counts[d]):
                got.append((d, int(send_tok[pos])))
                pos += 1
        assert got == want  # once per (rank, token), ordered by rank then token
        for i, (d, t) in enumerate(want):
            assert int(row_of[t, d]) == i
        assert int((row_of >= 0).sum()) == len(want)


def _prefill_routing():
    x = synth.to_bf16_bits(synth.activations(21, TP))
    logits = (synth.normal(22, TP * 512) * 2).astype(np.float32).reshape(TP, 512)
    ids, w = O.topk(logits)
    return x, ids, w


def _expert_row(e, x_bits):
    _, y = O.expert_ffn_bf16(IQ3_S, IQ3_S, H, INTER, synth.expert_blob(IQ3_S, IQ3_S, INTER, SEED, e), x_bits)
    return y[0]


def _prefill_rank_main(rank, world, port, out_dir, mode):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, ids, w = _prefill_routing()
    lo, hi = ep.token_range(rank, world, TP)

    plan = _skewed_plan(world) if mode == "placed" else None

    def local_rows(x_rows, e_rows, w_rows, elo, ehi):  # what route_ep + grouped kernels + combine compute
        out = np.zeros((x_rows.shape[0], H), dtype=np.float32)
        for r in range(x_rows.shape[0]):
            if plan is not None:  # fb_moe_route_placed: the share table decides, rows numbered as they arrive
                keep = lambda e: plan.keeps(rank, e, r)  # noqa: E731
            else:
                keep = lambda e: elo <= e < ehi  # noqa: E731
            pairs = sorted((int(e), float(wt)) for e, wt in zip(e_rows[r].tolist(), w_rows[r].tolist()) if keep(int(e)))
            assert pairs or mode != "sparse", "a row was sent to a rank that holds none of its experts"
            for e, wt in pairs:  # ascending expert id
                out[r] += np.float32(wt) * _expert_row(e, x_rows[r].numpy().view(np.uint16))
        return torch.from_numpy(out)

    def scatter_sum(y_back, row_of):
        y = np.zeros((row_of.shape[0], H), dtype=np.float32)
        for t in range(row_of.shape[0]):
            for d in range(row_of.shape[1]):  # rank order
                if row_of[t, d] >= 0:
                    y[t] += y_back[int(row_of[t, d])].numpy()
        return torch.from_numpy(y)

    args = (torch.from_numpy(x[lo:hi].view(np.int16).copy()), torch.from_numpy(ids[lo:hi].copy()),
            torch.from_numpy(w[lo:hi].copy()), rank, world, local_rows)
    if mode != "sparse":
        y, stats = ep_prefill.ep_layer_dense(*args, ep.combine_sum, chunks=3 if mode == "dense3" else 1)
        assert stats["rows_received"] == TP
    else:
        y, stats = ep_prefill.ep_layer_generic(*args, scatter_sum)
        assert stats["rows_sent"] <= (hi - lo) * world
    np.save(os.path.join(out_dir, "yp%d.npy" % rank), y.numpy())
    dist.destroy_process_group()


def _skewed_plan(world):
    """A placement with copies: the load is the routing histogram of the test's tokens with three experts
    made hot, planned with four spare slots per rank."""
    from fngine_b200 import placement
    _, ids, _ = _prefill_routing()
    load = np.bincount(ids.reshape(-1), minlength=512).astype(np.float64)
    hot = np.argsort(-load)[:3]
    load[hot] *= 40
    plan = placement.plan_placement(load, world, 512 // world + 4)
    assert any(len(c) > 1 for c in plan.copies)
    return plan


@pytest.mark.parametrize("mode,port", [("sparse", 29613), ("dense", 29614), ("dense3", 29615), ("placed", 29616)])
def test_two_rank_prefill_exchange_equals_single_rank(tmp_path, mode, port):
    mp.spawn(_prefill_rank_main, args=(2, port, str(tmp_path), mode), nprocs=2, join=True)
    x, ids, w = _prefill_routing()
    want = np.zeros((TP, H), dtype=np.float32)
    for t in range(TP):
        for e, wt in sorted(zip(ids[t].tolist(), w[t].tolist())):
            want[t] += np.float32(wt) * _expert_row(int(e), x[t])
    got = np.concatenate([np.load(os.path.join(str(tmp_path), "yp%d.npy" % r)) for r in range(2)])
    err = max(np.linalg.norm(got[t] - want[t]) / np.linalg.norm(want[t]) for t in range(TP))
    assert err <= 1e-5, err
