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


# --------------------------------------------------------------------------------------------- GPU side
class EpPrefillShard:
    """One layer's experts on this rank, with the [512] table of blob addresses by global expert id
    (0 for experts of other ranks) the grouped kernels index."""

    def __init__(self, rank, world, seed, fmt=21, inter=512):
        from . import ep
        self.rank, self.world = rank, world
        shard = ep.EpDecodeLayer(rank, world, seed, fmt, inter)  # the same bytes the single-GPU layer holds
        self.layer = shard.layer
        per = experts_per_rank(world)
        stride = self.layer.layout.blob_stride
        table = np.zeros(EXPERTS, dtype=np.int64)
        table[rank * per:(rank + 1) * per] = self.layer.slots.data_ptr() + stride * np.arange(per, dtype=np.int64)
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
    L.check(L.load().fb_moe_route_ep(_ptr(e_rows), _ptr(w_rows), lo, hi, rows, C.byref(ws.ws), _stream()), "moe_route_ep")
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


def ep_prefill_layer(logits_local, x_local, shard, ws, group=None):
    """One expert-parallel prefill layer on GPUs; returns (y of this rank's tokens, stats)."""
    e, w = topk(logits_local)
    return ep_layer_generic(
        x_local, e, w, shard.rank, shard.world,
        lambda xr, er, wr, lo, hi: local_rows(shard, ws, xr, er, wr, lo, hi),
        scatter_sum, group)
