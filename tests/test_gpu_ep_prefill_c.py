"""fb_ep_prefill_layer, the expert-parallel prefill layer behind one C call. On one GPU: with one rank the call
is the single-GPU layer, bit for bit. With two or more GPUs in the box: two ranks as child processes over the
collective library (in-switch reduction off), each comparing the C call with the Python mirror of the same
exchange, and their gathered result with the single-GPU layer."""
import os

import numpy as np
import pytest

from fngine_b200 import synth

pytestmark = pytest.mark.gpu
IQ3_S, H = 21, 2560


def _inputs(torch, T, seed):
    xd = torch.from_numpy(synth.to_bf16_bits(synth.activations(seed, T)).view(np.int16)).cuda().view(torch.bfloat16)
    lg = (synth.normal(seed + 1, T * 513) * 1.5).astype(np.float32).reshape(T, 513)
    lg[:, :512] += synth.zipf_router_bias(seed + 2)[None, :]
    return xd, torch.from_numpy(lg).cuda()


def test_one_rank_is_the_single_gpu_layer():
    import torch
    from fngine_b200 import ep_prefill, prefill
    T, inter, seed = 160, 512, 81
    xd, logits = _inputs(torch, T, 921)
    shard = ep_prefill.EpPrefillShard(0, 1, seed, IQ3_S, inter)
    ws = prefill.PrefillWorkspace(T, inter)
    want = torch.empty(T, H, dtype=torch.float32, device="cuda")
    prefill.moe_layer_prefill(logits, shard.layer, xd, ws, want)
    torch.cuda.synchronize()
    for combine in ("all_to_all", "reduce_scatter"):
        scratch = ep_prefill.EpPrefillScratch(T, 1, combine)
        got = torch.full((T, H), float("nan"), dtype=torch.float32, device="cuda")
        ep_prefill.ep_prefill_layer_c(logits, xd, shard, ws, scratch, got)
        torch.cuda.synchronize()
        assert ws.status() == 0 and torch.equal(got, want)


def test_rows_beyond_the_workspace_are_refused():
    import torch
    from fngine_b200 import ep_prefill, lib, prefill
    T, inter = 64, 512
    xd, logits = _inputs(torch, T, 931)
    shard = ep_prefill.EpPrefillShard(0, 2, 82, IQ3_S, inter)
    ws = prefill.PrefillWorkspace(T, inter)  # two ranks need 2 T rows
    scratch = ep_prefill.EpPrefillScratch(T, 2)
    y = torch.empty(T, H, dtype=torch.float32, device="cuda")
    with pytest.raises(lib.FbError):
        ep_prefill.ep_prefill_layer_c(logits, xd, shard, ws, scratch, y, comm=0)


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from fngine_b200 import ep_prefill, placement, prefill
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        T, inter, seed = 192, 512, 83
        tl = T // world
        xd, logits = _inputs(torch, T, 941)
        x_local, lg_local = xd[rank * tl:(rank + 1) * tl].contiguous(), logits[rank * tl:(rank + 1) * tl].contiguous()
        ws = prefill.PrefillWorkspace(T, inter)
        comm = ep_prefill.comm_pointer()
        e_all, _ = ep_prefill.topk(logits)
        load = np.bincount(e_all.cpu().numpy().reshape(-1), minlength=512)
        plan = placement.plan_placement(load, world, 512 // world + 4, tolerance=-1.0)
        result = {}
        for name, pl in (("contiguous", None), ("placed", plan)):
            shard = ep_prefill.EpPrefillShard(rank, world, seed, IQ3_S, inter, placement=pl)
            for combine in ("all_to_all", "reduce_scatter"):
                mirror, _ = ep_prefill.ep_prefill_layer(lg_local, x_local, shard, ws, combine=combine)
                torch.cuda.synchronize()
                scratch = ep_prefill.EpPrefillScratch(tl, world, combine)
                got = torch.full((tl, H), float("nan"), dtype=torch.float32, device="cuda")
                ep_prefill.ep_prefill_layer_c(lg_local, x_local, shard, ws, scratch, got, comm)
                torch.cuda.synchronize()
                assert ws.status() == 0
                if combine == "all_to_all":
                    assert torch.equal(got, mirror), (name, combine)
                else:
                    assert float((got - mirror).norm() / mirror.norm()) <= 1e-6, (name, combine)
                result[name + "/" + combine] = got.cpu().numpy()
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **result)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_the_collective_library(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from fngine_b200 import ep_prefill, prefill
    world, T, inter, seed = 2, 192, 512, 83
    mp.spawn(_rank_main, args=(world, 29641, str(tmp_path)), nprocs=world, join=True)
    xd, logits = _inputs(torch, T, 941)
    single = ep_prefill.EpPrefillShard(0, 1, seed, IQ3_S, inter)
    ws = prefill.PrefillWorkspace(T, inter)
    want = torch.empty(T, H, dtype=torch.float32, device="cuda")
    prefill.moe_layer_prefill(logits, single.layer, xd, ws, want)
    torch.cuda.synchronize()
    want = want.cpu().numpy()
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    for key in parts[0].files:
        got = np.concatenate([p[key] for p in parts])
        err = max(float(np.linalg.norm(got[t] - want[t]) / np.linalg.norm(want[t])) for t in range(T))
        print("two ranks, %s: max rel L2 against the single-GPU layer %.2e" % (key, err))
        assert err <= 1e-5, (key, err)
