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
        from . import moe
        self.rank, self.world = rank, world
        per = experts_per_rank(world)
        # the same bytes the single-GPU layer holds for global experts rank * per .. rank * per + per - 1
        self.layer = moe.synth_layer(fmt, fmt, inter, per, seed, first_expert=rank * per)
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
