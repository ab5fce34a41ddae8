"""Expert-parallel prefill over the GPUs of one node (one process per GPU, torch.distributed).

The reference engine is single-GPU. Here the 512 experts of a layer are sharded contiguously
(expert e lives on rank e // (512/R)) and the tokens are data-parallel (rank r owns tokens
[r*T/R, (r+1)*T/R) and a replica of the router). One layer:

  1. the owner takes the top-10 of its tokens (fb_moe_topk, the rule of fb_moe_route);
  2. plan: a token's row goes ONCE to every rank that holds at least one of its experts, rows
     ordered by (destination rank, token);
  3. counts all-to-all, then dispatch all-to-all-v of the bf16 rows and of their (expert, weight)
     lists;
  4. every rank runs route_ep -> grouped gate/up -> grouped down -> combine over the rows it
     received, restricted to its own experts: one fp32 partial row per received row, summed in
     ascending expert order;
  5. combine all-to-all-v returns the partial rows (the reverse splits, so they land in the order
     they were sent) and the owner adds a token's partial rows in rank order (fb_ep_scatter_sum).

That is the SPARSE exchange (ep_layer_generic): it moves the fewest bytes but needs the counts on the
host before buffers can be sized. The DENSE exchange (ep_layer_dense, what bench.py times) trades
bytes for zero host synchronisation: all-gather of the rows and lists, every rank computes a partial
row for EVERY token over its own experts (zero when it holds none of them), one fixed-size
all-to-all returns them and the owner adds the R partial rows of a token in rank order
(fb_ep_sum_ranks). At 8 ranks a token's ten experts touch 5.9 ranks on average, so dense moves about
a third more bytes than sparse; at 2 ranks both move the same.

Experts are sharded contiguously, so "rank order of per-rank ascending-expert sums" is the
single-GPU ascending-expert sum with different parentheses: equal within fp32 rounding, not
bitwise. The planning and exchange code below is device-agnostic and is exercised on CPU ranks
(gloo) by tests/test_ep_gloo.py; the collectives run over NCCL (NVLink / NVSwitch) on GPUs.
"""
import numpy as np
import torch

EXPERTS = 512
HIDDEN = 2560
TOPK = 10


def experts_per_rank(world):
    if EXPERTS % world:
        raise ValueError("world size must divide 512")
    return EXPERTS // world


def plan_dispatch(topk_expert, world):
    """topk_expert int32 [T_local][10] -> (send_tok int64 [n], send_counts list[R], row_of int32 [T_local][R]).

    send_tok lists the local tokens whose rows are sent, ordered by (destination rank, token); a
    token appears once per destination rank however many of its experts live there. row_of[t][d]
    is the position of token t's row in the send order for rank d (= the position of the partial
    row rank d returns), -1 when rank d holds none of the token's experts."""
    per = experts_per_rank(world)
    T = topk_expert.shape[0]
    dest = torch.div(topk_expert.long(), per, rounding_mode="floor")
    mask = torch.zeros(T, world, dtype=torch.bool, device=topk_expert.device)
    mask.scatter_(1, dest, True)
    idx = mask.t().nonzero()  # rows (d, t), ordered by d then t
    send_tok = idx[:, 1].contiguous()
    send_counts = mask.sum(0).tolist()
    row_of = torch.full((T, world), -1, dtype=torch.int32, device=topk_expert.device)
    row_of[idx[:, 1], idx[:, 0]] = torch.arange(idx.shape[0], dtype=torch.int32, device=topk_expert.device)
    return send_tok, send_counts, row_of


def exchange_counts(send_counts, world, device, group=None):
    """send_counts[d] rows go to rank d -> recv_counts[s] rows arrive from rank s."""
    import torch.distributed as dist
    if world == 1:
        return list(send_counts)
    s = torch.tensor(send_counts, dtype=torch.int64, device=device)
    r = torch.empty_like(s)
    dist.all_to_all_single(r, s, group=group)
    return r.tolist()


def exchange_rows(send, send_counts, recv_counts, world, group=None):
    """All-to-all-v of rows: send [sum(send_counts)][...] grouped by destination rank ->
    [sum(recv_counts)][...] grouped by source rank."""
    import torch.distributed as dist
    if world == 1:
        return send
    # rows travel as bytes: one code path for bf16 / int32 / fp32 rows on every backend
    rows_out = int(sum(recv_counts))
    send_b = send.contiguous().view(torch.uint8).reshape(send.shape[0], -1)
    recv_b = torch.empty(rows_out, send_b.shape[1], dtype=torch.uint8, device=send.device)
    dist.all_to_all_single(recv_b, send_b, list(recv_counts), list(send_counts), group=group)
    return recv_b.view(send.dtype).reshape((rows_out,) + tuple(send.shape[1:]))


def pack_lists(topk_expert, topk_weight):
    """(int32 [T][10], float32 [T][10]) -> int32 [T][20], one row per token for the dispatch."""
    return torch.cat([topk_expert.view(torch.int32), topk_weight.view(torch.int32)], dim=1)


def unpack_lists(lists):
    return lists[:, :TOPK].contiguous(), lists[:, TOPK:].contiguous().view(torch.float32)


def ep_layer_generic(x_local, topk_expert, topk_weight, rank, world, local_rows_fn, scatter_sum_fn, group=None):
    """One expert-parallel layer with the compute and the owner-side sum passed in:
    local_rows_fn(x_rows, topk_e_rows, topk_w_rows, lo, hi) -> fp32 partial rows over experts [lo, hi);
    scatter_sum_fn(returned_rows, row_of) -> y of this rank's tokens. The GPU path and the CPU test
    share everything else. Returns (y_local, stats)."""
    per = experts_per_rank(world)
    send_tok, send_counts, row_of = plan_dispatch(topk_expert, world)
    recv_counts = exchange_counts(send_counts, world, x_local.device, group)
    x_send = x_local.index_select(0, send_tok)
    l_send = pack_lists(topk_expert, topk_weight).index_select(0, send_tok)
    x_recv = exchange_rows(x_send, send_counts, recv_counts, world, group)
    l_recv = exchange_rows(l_send, send_counts, recv_counts, world, group)
    e_rows, w_rows = unpack_lists(l_recv)
    y_part = local_rows_fn(x_recv, e_rows, w_rows, rank * per, (rank + 1) * per)
    y_back = exchange_rows(y_part, recv_counts, send_counts, world, group)
    y = scatter_sum_fn(y_back, row_of)
    stats = {"rows_sent": int(sum(send_counts)), "rows_received": int(sum(recv_counts)),
             "dispatch_bytes": int(sum(send_counts)) * (x_local.shape[1] * x_local.element_size() + 8 * TOPK),
             "combine_bytes": int(sum(recv_counts)) * x_local.shape[1] * 4}
    return y, stats


def ep_layer_dense(x_local, topk_expert, topk_weight, rank, world, local_rows_fn, sum_ranks_fn, group=None, chunks=1,
                   combine="all_to_all"):
    """Dense exchange: all-gather rows and lists, partial rows for all tokens, fixed-size all-to-all,
    rank-order sum. local_rows_fn as in ep_layer_generic; sum_ranks_fn([R][rows][H]) -> [rows][H].
    combine = "reduce_scatter": the all-to-all and the owner's sum are one reduce-scatter of the library
    (a rank's partial rows are already grouped by owner): a rank then receives one summed row per token
    instead of R partial rows, and the switch may add them on the way; the order of the additions is the
    library's (fixed for a topology, not rank order), so results agree with the all-to-all form to fp32
    rounding, not bit for bit.
    With chunks > 1 the rank's tokens are cut into that many pieces and pipelined: the all-to-all of
    piece c runs (on the collective library's stream) while piece c+1 is gathered and computed. That
    only pays when the grouped GEMMs are bound by the tokens: they are bound by the dequantization of
    the weight tiles, which every piece repeats (measured at 2 GPUs, 4 layers: 7.8 ms with two pieces
    against 6.0 ms with one), so the default is one piece."""
    import torch.distributed as dist
    per = experts_per_rank(world)
    tl = x_local.shape[0]
    lists = pack_lists(topk_expert, topk_weight)
    stats = {"rows_received": tl * world,
             "dispatch_bytes": tl * (world - 1) * (x_local.shape[1] * x_local.element_size() + 8 * TOPK),
             "combine_bytes": tl * (world - 1) * x_local.shape[1] * 4}
    if world == 1:
        e_rows, w_rows = unpack_lists(lists)
        return sum_ranks_fn(local_rows_fn(x_local, e_rows, w_rows, 0, per).unsqueeze(0)), stats
    chunks = max(1, min(chunks, tl))
    bounds = [tl * c // chunks for c in range(chunks + 1)]

    def gather(c):
        lo, hi = bounds[c], bounds[c + 1]
        xb = x_local[lo:hi].contiguous().view(torch.uint8).reshape(hi - lo, -1)
        x_all_b = torch.empty((hi - lo) * world, xb.shape[1], dtype=torch.uint8, device=x_local.device)
        l_all = torch.empty((hi - lo) * world, lists.shape[1], dtype=lists.dtype, device=lists.device)
        w1 = dist.all_gather_into_tensor(x_all_b, xb, group=group, async_op=True)
        w2 = dist.all_gather_into_tensor(l_all, lists[lo:hi].contiguous(), group=group, async_op=True)
        return x_all_b, l_all, (w1, w2)

    pending = gather(0)
    returns = []
    for c in range(chunks):
        x_all_b, l_all, works = pending
        for w in works:
            w.wait()
        if c + 1 < chunks:
            pending = gather(c + 1)
        n = bounds[c + 1] - bounds[c]
        x_all = x_all_b.view(x_local.dtype).reshape(n * world, x_local.shape[1])
        e_rows, w_rows = unpack_lists(l_all)
        y_part = local_rows_fn(x_all, e_rows, w_rows, rank * per, (rank + 1) * per)  # [n * R][H] fp32
        if combine == "reduce_scatter":
            recv = torch.empty(n, y_part.shape[1], dtype=y_part.dtype, device=y_part.device)
            work = dist.reduce_scatter_tensor(recv, y_part.contiguous(), group=group, async_op=True)
        else:
            recv = torch.empty_like(y_part)
            work = dist.all_to_all_single(recv, y_part.contiguous(), group=group, async_op=True)
        returns.append((recv, work, n, y_part))
    outs = []
    for recv, work, n, _keep in returns:
        work.wait()
        outs.append(recv if combine == "reduce_scatter" else sum_ranks_fn(recv.view(world, n, recv.shape[1])))
    return (outs[0] if chunks == 1 else torch.cat(outs)), stats


# --------------------------------------------------------------------------------------------- GPU side
class EpPrefillShard:
    """One layer's experts on this rank, with the [512] table of blob addresses by global expert id
    (0 for experts of other ranks) the grouped kernels index. With a placement (placement.Placement) the
    rank holds the experts the plan gives it, copies of hot experts included, and `share` is its table
    for fb_moe_route_placed; without one the shards are contiguous."""

    def __init__(self, rank, world, seed, fmt=21, inter=512, placement=None):
        from . import ep, moe
        self.rank, self.world = rank, world
        table = np.zeros(EXPERTS, dtype=np.int64)
        if placement is None:
            shard = ep.EpDecodeLayer(rank, world, seed, fmt, inter)  # the same bytes the single-GPU layer holds
            self.layer = shard.layer
            per = experts_per_rank(world)
            stride = self.layer.layout.blob_stride
            table[rank * per:(rank + 1) * per] = self.layer.slots.data_ptr() + stride * np.arange(per, dtype=np.int64)
            self.share = None
        else:
            held = placement.rank_experts[rank]
            self.layer = moe.synth_layer_of(fmt, fmt, inter, held, seed)
            stride = self.layer.layout.blob_stride
            table[np.asarray(held, dtype=np.int64)] = self.layer.slots.data_ptr() + stride * np.arange(len(held), dtype=np.int64)
            self.share = torch.from_numpy(placement.share_table(rank)).cuda()
        self.blob_table = torch.from_numpy(table).cuda()


def topk(logits, tokens=None):
    import ctypes as C
    from . import lib as L
    from .moe import _ptr, _stream
    tokens = tokens or logits.shape[0]
    e = torch.empty(tokens, TOPK, dtype=torch.int32, device=logits.device)
    w = torch.empty(tokens, TOPK, dtype=torch.float32, device=logits.device)
    L.check(L.load().fb_moe_topk(_ptr(logits), logits.shape[-1], tokens, _ptr(e), _ptr(w), _stream()), "moe_topk")
    return e, w


def local_rows(shard, ws, x_rows, e_rows, w_rows, lo, hi):
    """fp32 [rows][2560]: every received row's sum over this rank's experts."""
    import ctypes as C
    from . import lib as L
    from . import prefill
    from .moe import _ptr, _stream
    rows = x_rows.shape[0]
    y = torch.empty(rows, HIDDEN, dtype=torch.float32, device=x_rows.device)
    if rows == 0:
        return y
    if getattr(shard, "share", None) is not None:  # placed shards: the share table decides, not [lo, hi)
        L.check(L.load().fb_moe_route_placed(_ptr(e_rows), _ptr(w_rows), _ptr(shard.share), rows, C.byref(ws.ws),
                                             _stream()), "moe_route_placed")
    else:
        L.check(L.load().fb_moe_route_ep(_ptr(e_rows), _ptr(w_rows), lo, hi, rows, C.byref(ws.ws), _stream()),
                "moe_route_ep")
    prefill.moe_grouped_gate_up(shard.layer, shard.blob_table, x_rows, rows, ws)
    prefill.moe_grouped_down(shard.layer, shard.blob_table, rows, ws)
    prefill.moe_prefill_combine(ws, None, None, 0, None, None, None, y, rows)
    return y


def scatter_sum(y_back, row_of):
    from . import lib as L
    from .moe import _ptr, _stream
    tokens, world = row_of.shape
    y = torch.empty(tokens, HIDDEN, dtype=torch.float32, device=row_of.device)
    if y_back.shape[0] == 0:
        return y.zero_()
    L.check(L.load().fb_ep_scatter_sum(_ptr(y_back), _ptr(row_of), world, tokens, _ptr(y), _stream()), "ep_scatter_sum")
    return y


def sum_ranks(parts):
    from . import ep
    y = torch.empty(parts.shape[1], parts.shape[2], dtype=torch.float32, device=parts.device)
    ep.sum_ranks(parts.contiguous(), y)
    return y


def ep_prefill_layer(logits_local, x_local, shard, ws, group=None, mode="dense", chunks=1, combine="all_to_all"):
    """One expert-parallel prefill layer on GPUs; returns (y of this rank's tokens, stats). Shards built
    from a placement need the dense exchange (their copies split pairs by row number, which must mean the
    same row on every rank)."""
    if getattr(shard, "share", None) is not None and mode != "dense":
        raise ValueError("placed shards run with the dense exchange only")
    e, w = topk(logits_local)
    compute = lambda xr, er, wr, lo, hi: local_rows(shard, ws, xr, er, wr, lo, hi)  # noqa: E731
    if mode == "dense":
        return ep_layer_dense(x_local, e, w, shard.rank, shard.world, compute, sum_ranks, group, chunks, combine)
    return ep_layer_generic(x_local, e, w, shard.rank, shard.world, compute, scatter_sum, group)


# --------------------------------------------------------------------------------------------- one C call
COMBINE_CODES = {"all_to_all": 0, "reduce_scatter": 1}


def comm_pointer(group=None, device=None):
    """The ncclComm_t of a torch.distributed NCCL process group as an integer, for fb_ep_prefill_layer. The group
    creates its communicator at its first collective, so one small all-reduce runs first; the caller must not have
    collectives of the same group in flight on other streams while the C entry point uses the communicator."""
    import torch.distributed as dist
    device = device or torch.device("cuda", torch.cuda.current_device())
    dist.all_reduce(torch.zeros(1, device=device), group=group)
    torch.cuda.synchronize()
    backend = (group or dist.group.WORLD)._get_backend(device)
    return int(backend._comm_ptr())


class EpPrefillScratch:
    """Caller-owned device memory of fb_ep_prefill_layer for `tokens_local` tokens per rank."""

    def __init__(self, tokens_local, world, combine="reduce_scatter", device="cuda"):
        from . import lib as L
        self.combine = COMBINE_CODES[combine]
        n = L.load().fb_ep_prefill_scratch_bytes(tokens_local, world, self.combine)
        if n == 0:
            raise L.FbError("unsupported expert-parallel prefill shape")
        self.buf = torch.empty(n + 256, dtype=torch.uint8, device=device)
        self.base = (self.buf.data_ptr() + 255) & ~255
        self.tokens_local, self.world = tokens_local, world


def ep_prefill_layer_c(logits_local, x_local, shard, ws, scratch, y_local, comm=0):
    """Mirror of fb_ep_prefill_layer: the whole dense-exchange layer (top-10, all-gather, this rank's experts,
    combine) enqueued by one C call on the current stream; `comm` = comm_pointer() (0 with one rank)."""
    import ctypes as C
    from . import lib as L
    from .moe import _ptr, _stream
    assert x_local.dtype == torch.bfloat16 and y_local.dtype == torch.float32
    assert x_local.shape[0] == scratch.tokens_local and shard.world == scratch.world
    per = experts_per_rank(shard.world)
    L.check(L.load().fb_ep_prefill_layer(C.byref(shard.layer.layout), _ptr(shard.blob_table), _ptr(shard.share),
                                         shard.rank * per, (shard.rank + 1) * per, _ptr(logits_local),
                                         logits_local.shape[-1], _ptr(x_local), x_local.shape[0], shard.world,
                                         scratch.combine, C.byref(ws.ws), scratch.base, _ptr(y_local), comm, _stream()),
            "ep_prefill_layer")
    return y_local
