"""Expert-parallel decode over the GPUs of one node (one process per GPU, torch.distributed).

The reference engine is single-GPU; its only notion of "experts that live elsewhere" is the cold
CPU tier (src/kernels/moe/moe.h:119-121 of the reference). Here "elsewhere" is another rank:

  * the 512 experts of a layer are sharded contiguously, expert e lives on rank e // (512/R);
  * the step's tokens are data-parallel: rank r owns tokens [r*T/R, (r+1)*T/R);
  * dispatch  = all-to-all of token activations (every owner sends its rows to the ranks that hold
                experts for them; at decode widths each token needs experts on most ranks, so the
                rows go to every rank and each rank routes all T tokens itself, router replicated);
  * compute   = fb_moe_layer_decode_ep: the decode kernels over the rank's own experts only;
  * combine   = all-to-all of the partial y rows back to the owning rank, which adds the R partial
                rows of each token in rank order (deterministic).

Two exchanges are implemented on GPUs. ep_layer_step runs the collectives through NCCL
(all_to_all_single for dispatch and combine, fb_ep_sum_ranks for the owner's rank-order sum).
layer_decode_ep_p2p (PeerExchange + fb_moe_layer_decode_ep_p2p) does the same exchange inside the
layer's own kernels: ranks store flag-in-data lines into each other's CUDA-IPC-mapped buffers over
NVLink and poll their own memory, so a step makes no collective call; both give the same bits.

The split / ordering logic in this file is backend-agnostic and is exercised on CPU ranks (gloo) by
tests/test_ep_gloo.py.
"""
import json
import os
import time

import numpy as np

EXPERTS = 512
HIDDEN = 2560


def experts_per_rank(world):
    if EXPERTS % world:
        raise ValueError("world size must divide 512")
    return EXPERTS // world


def owner_of(expert, world):
    return expert // experts_per_rank(world)


def local_slot_map(rank, world):
    """int32[512]: local slot of each expert on `rank`, -1 for experts of other ranks."""
    per = experts_per_rank(world)
    m = np.full(EXPERTS, -1, dtype=np.int32)
    m[rank * per:(rank + 1) * per] = np.arange(per, dtype=np.int32)
    return m


def token_range(rank, world, tokens):
    if tokens % world:
        raise ValueError("the step's token count must be a multiple of the world size")
    per = tokens // world
    return rank * per, (rank + 1) * per


def dispatch(x_local, world, group=None):
    """x_local [T/R][H] (this rank's tokens) -> [T][H], all tokens in owner-rank order."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return x_local
    send = x_local.repeat(world, 1).contiguous()  # the same rows go to every rank
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def combine_exchange(y_partial, world, group=None):
    """y_partial [T][H] (this rank's experts, all tokens) -> [R][T/R][H]: for this rank's own tokens,
    the partial rows computed by every rank, indexed by source rank."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return y_partial.unsqueeze(0)
    recv = torch.empty_like(y_partial)
    dist.all_to_all_single(recv, y_partial.contiguous(), group=group)
    return recv.view(world, y_partial.shape[0] // world, y_partial.shape[1])


def combine_sum(parts):
    """[R][rows][H] -> [rows][H], added in rank order (what fb_ep_sum_ranks does on the device)."""
    y = parts[0].clone()
    for r in range(1, parts.shape[0]):
        y += parts[r]
    return y


# --------------------------------------------------------------------------------------------- GPU side
class EpDecodeLayer:
    """One layer's shard on this rank: local experts, replicated router, slot map."""

    def __init__(self, rank, world, seed, fmt=21, inter=512):
        import torch
        from . import moe, synth
        from . import lib as L
        self.rank, self.world = rank, world
        per = experts_per_rank(world)
        lib = L.load()
        stride = lib.fb_moe_blob_bytes(fmt, fmt, inter)
        buf = torch.empty(per * stride, dtype=torch.uint8, device="cuda")
        table = torch.from_numpy(synth.d_table(fmt).view(np.int16)).cuda()
        gu_bytes = 2 * inter * lib.fb_moe_row_bytes(fmt, HIDDEN)
        nb_gu = gu_bytes // synth.BLOCK_BYTES[fmt]
        nb_dn = (stride - gu_bytes) // synth.BLOCK_BYTES[fmt]
        stream = torch.cuda.current_stream().cuda_stream
        for s in range(per):  # same bytes the single-GPU layer holds for global expert e
            e = rank * per + s
            base = buf.data_ptr() + s * stride
            L.check(lib.fb_synth_fill_blocks(fmt, base, nb_gu, e * nb_gu, seed, table.data_ptr(), stream))
            L.check(lib.fb_synth_fill_blocks(fmt, base + gu_bytes, nb_dn, e * nb_dn, seed ^ 0xD0, table.data_ptr(), stream))
        self.layer = moe.ExpertLayer(buf, fmt, fmt, inter)
        self.slot_of = torch.from_numpy(local_slot_map(rank, world)).cuda()


def layer_decode_ep(router, ep_layer, x_all, ws, y_partial):
    import ctypes as C
    import torch
    from . import lib as L
    from .moe import _dtype_code, _ptr, _stream
    L.check(L.load().fb_moe_layer_decode_ep(_ptr(router), C.byref(ep_layer.layer.layout), _ptr(ep_layer.slot_of),
                                            _ptr(x_all), _dtype_code(x_all), x_all.shape[0], C.byref(ws.ws),
                                            _ptr(ws.logits), _ptr(y_partial), _stream()), "moe_layer_decode_ep")


def sum_ranks(parts, y):
    from . import lib as L
    from .moe import _ptr, _stream
    L.check(L.load().fb_ep_sum_ranks(_ptr(parts), parts.shape[0], parts.shape[1], _ptr(y), _stream()), "ep_sum_ranks")


class PeerExchange:
    """The two exchange buffers of fb_moe_layer_decode_ep_p2p on this rank, mapped into every peer
    process with CUDA IPC (the 128 handle bytes travel through the process group once, at set-up)."""

    def __init__(self, rank, world, group=None):
        import ctypes as C
        import torch.distributed as dist
        from . import lib as L
        lib = L.load()
        self.rank, self.world, self.step = rank, world, 0
        own = [C.c_void_p() for _ in range(2)]
        handles = (C.c_uint8 * 128)()
        L.check(lib.fb_ep_exchange_create(C.byref(own[0]), C.byref(own[1]), handles), "ep_exchange_create")
        gathered = [None] * world
        dist.all_gather_object(gathered, bytes(handles), group=group)
        self.peers = L.EpPeers()
        self.peers.rank, self.peers.n_ranks = rank, world
        self._opened = []
        for d in range(world):
            if d == rank:
                ptrs = own
            else:
                ptrs = [C.c_void_p() for _ in range(2)]
                hb = (C.c_uint8 * 128).from_buffer_copy(gathered[d])
                L.check(lib.fb_ep_exchange_open(hb, C.byref(ptrs[0]), C.byref(ptrs[1])), "ep_exchange_open")
                self._opened.append(ptrs)
            self.peers.x_all[d], self.peers.y_parts[d] = (p.value for p in ptrs)
        self._own = own
        dist.barrier(group=group)

    def close(self):
        from . import lib as L
        lib = L.load()
        for ptrs in self._opened:
            lib.fb_ep_exchange_close(ptrs[0], ptrs[1], 0)
        self._opened = []
        if self._own:
            lib.fb_ep_exchange_close(self._own[0], self._own[1], 1)
            self._own = None


def layer_decode_ep_p2p(router, ep_layer, x_local, ws, xchg, y_local):
    """One expert-parallel decode layer with the exchange inside the kernels (peer stores + flags)."""
    import ctypes as C
    from . import lib as L
    from .moe import _ptr, _stream
    xchg.step += 1
    tokens = x_local.shape[0] * xchg.world
    L.check(L.load().fb_moe_layer_decode_ep_p2p(_ptr(router), C.byref(ep_layer.layer.layout), _ptr(ep_layer.slot_of),
                                                _ptr(x_local), tokens, C.byref(xchg.peers), xchg.step, C.byref(ws.ws),
                                                _ptr(ws.logits), _ptr(y_local), _stream()), "moe_layer_decode_ep_p2p")
    return y_local


def ep_layer_step(router, ep_layer, x_local, ws, bufs):
    """dispatch -> local experts -> combine for one layer; returns y of this rank's tokens."""
    world = ep_layer.world
    x_all = dispatch(x_local, world)
    layer_decode_ep(router, ep_layer, x_all, ws, bufs["y_partial"])
    parts = combine_exchange(bufs["y_partial"], world)
    sum_ranks(parts.contiguous(), bufs["y_local"])
    return bufs["y_local"]


def bench_main(args, rank, world, local_rank):
    """bench.py for N > 1: strong scaling of the same 16-token decode step over expert-parallel ranks.
    The timed step exchanges through peer memory inside the kernels (fb_moe_layer_decode_ep_p2p); the
    same step with NCCL all-to-alls is timed beside it and the two results are compared bit for bit."""
    import torch
    import torch.distributed as dist
    from . import moe, synth
    from bench import BLOB, ROUTER_BYTES, ClockSampler, peaks, workload_config  # bench.py is the caller

    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B, Lr = args.batch, args.layers
    lo, hi = token_range(rank, world, B)
    layers, routers, xs_host, xs = [], [], [], []
    for l in range(Lr):
        layers.append(EpDecodeLayer(rank, world, 5000 + l))
        wr = synth.router_weights(9000 + l)
        routers.append(torch.from_numpy(wr.view(np.int16)).cuda().view(torch.bfloat16))
        xh = torch.from_numpy(synth.activations(7000 + l, B)[lo:hi].copy()).pin_memory()
        xs_host.append(xh)
        xs.append(xh.cuda())
    ws = moe.DecodeWorkspace(layers[0].layer)
    bufs = {"y_partial": torch.empty(B, HIDDEN, dtype=torch.float32, device="cuda"),
            "y_local": torch.empty(hi - lo, HIDDEN, dtype=torch.float32, device="cuda")}
    xchg = PeerExchange(rank, world)
    y_p2p = torch.empty(hi - lo, HIDDEN, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    def step_nccl():
        for l in range(Lr):
            ep_layer_step(routers[l], layers[l], xs[l], ws, bufs)

    def step():
        for l in range(Lr):
            layer_decode_ep_p2p(routers[l], layers[l], xs[l], ws, xchg, y_p2p)

    # the two exchanges give the same bits (same partial rows, same rank-order sum)
    same = True
    for l in range(Lr):
        y_a = ep_layer_step(routers[l], layers[l], xs[l], ws, bufs).clone()
        layer_decode_ep_p2p(routers[l], layers[l], xs[l], ws, xchg, y_p2p)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(y_a, y_p2p))
    flag = torch.tensor([1.0 if same else 0.0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    same = bool(flag.item() == 1.0)

    # local distinct experts per layer (for the byte count) and a parity check of layer 0 on rank 0
    distinct = []
    for l in range(Lr):
        ep_layer_step(routers[l], layers[l], xs[l], ws, bufs)
        torch.cuda.synchronize()
        distinct.append(ws.work().n_items)
        if l == 0:
            layer_decode_ep_p2p(routers[l], layers[l], xs[l], ws, xchg, y_p2p)
            torch.cuda.synchronize()
            y0 = y_p2p.clone()
    local_bytes = torch.tensor([float(sum(d * BLOB + ROUTER_BYTES for d in distinct))], device="cuda")
    dist.all_reduce(local_bytes)
    step_bytes = float(local_bytes.item())

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # the NCCL all-to-all step beside it
    for _ in range(3):
        step_nccl()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0.record()
    for _ in range(args.steps):
        step_nccl()
    n1.record()
    torch.cuda.synchronize()
    dist.barrier()
    tn = torch.tensor([n0.elapsed_time(n1)], device="cuda")
    dist.all_reduce(tn, op=dist.ReduceOp.MAX)
    nccl_ms = float(tn.item())

    # end to end: pinned host rows of the own tokens in, own y rows out, every layer
    yh = torch.empty(hi - lo, HIDDEN, dtype=torch.float32).pin_memory()
    xd = torch.empty(hi - lo, HIDDEN, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    dist.barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        for l in range(Lr):
            xd.copy_(xs_host[l], non_blocking=True)
            y = layer_decode_ep_p2p(routers[l], layers[l], xd, ws, xchg, y_p2p)
            yh.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    f1.record()
    torch.cuda.synchronize()
    t2 = torch.tensor([f0.elapsed_time(f1)], device="cuda")
    dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item())

    clocks = sampler.stop() if rank == 0 else None
    status = ws.status()

    # parity of the measured workload: layer 0 of this rank's tokens against the CPU oracle
    parity = None
    if rank == 0:
        from oracle import oracle as O
        x_full = synth.activations(7000, B)
        wr_bits = synth.router_weights(9000)
        logits = x_full.astype(np.float32) @ synth.bf16_bits_to_f32(wr_bits).T
        ids, w = O.topk(np.ascontiguousarray(logits[:, :EXPERTS]))
        ids, w, xo = ids[lo:hi], w[lo:hi], x_full[lo:hi]
        used = sorted(set(ids.reshape(-1).tolist()))
        blobs = np.concatenate([synth.expert_blob(21, 21, 512, 5000, e) for e in used])
        ids2 = np.vectorize({e: i for i, e in enumerate(used)}.get)(ids).astype(np.int32)
        want = O.moe_layer(21, 21, HIDDEN, 512, blobs, BLOB, xo, ids2, w, threads=os.cpu_count() or 1, lib=O.ref())
        got = y0.cpu().numpy()
        parity = float(max(np.linalg.norm(got[i] - want[i]) / np.linalg.norm(want[i]) for i in range(hi - lo)))
    dist.barrier()
    # the 48-layer prefill stack, expert-parallel (the decode layers are released first)
    pre = None
    if args.sections == "all" or "prefill" in args.sections.split(","):
        from . import ep_prefill
        del layers
        torch.cuda.empty_cache()
        pre = ep_prefill.bench_section(rank, world, n_layers=args.prefill_layers)
    if rank == 0:
        peak, peak_src = peaks()
        value = step_bytes * args.steps / (ms * 1e-3) / 1e9
        ach = value / world  # per GPU, whole layer step (kernels are timed one by one only at N = 1)
        cfg = workload_config(args, Lr)
        cfg["parallelism"] = ("ep%d: %d experts per GPU, tokens data-parallel (%d per GPU), dispatch + combine by peer "
                              "stores over NVLink inside the kernels (no collective call in the step)" % (
                                  world, EXPERTS // world, B // world))
        line = {"metric": "iq3s_expert_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": cfg, "tokens_per_s": B * Lr * args.steps / (ms * 1e-3), "us_per_layer": ms / args.steps / Lr * 1e3,
                "distinct_local_experts_rank0": distinct,
                "nccl_all_to_all_step": {"us_per_layer": nccl_ms / args.steps / Lr * 1e3,
                                         "value": step_bytes * args.steps / (nccl_ms * 1e-3) / 1e9,
                                         "bitwise_equal_to_peer_exchange": same},
                "roofline": {"bound": "hbm", "kernel": "whole expert-parallel layer step, per GPU (incl. the exchange)", "achieved": ach, "peak": peak,
                             "unit": "GB/s", "frac": ach / peak, "peak_source": peak_src, "traffic": None},
                "e2e": {"value": step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                        "h2d_bytes_per_step": (hi - lo) * HIDDEN * 4 * Lr * world,
                        "d2h_bytes_per_step": (hi - lo) * HIDDEN * 4 * Lr * world, "ms_per_step": e2e_ms / args.steps},
                "gpu_launches": args.steps * Lr * 4 * world, "parity_vs_cpu_max_rel_l2": parity,
                "device_status": status, "clocks": clocks, "prefill_stack": pre,
                "cpu_baseline": None}
        print(json.dumps(line))
    xchg.close()
    dist.destroy_process_group()
