"""The C-ABI library builds, loads, and exports every symbol the header declares (no compute)."""
import ctypes
import os
import re

from fngine_b200 import lib as fblib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            txt = open(os.path.join(ROOT, "include", fn)).read()
            txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
            names |= set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", txt))
    return names


def test_header_and_binding_agree():
    assert declared_symbols() == set(fblib.exported_names())


def test_library_exports_every_declared_symbol(fb_built):
    lib = ctypes.CDLL(fb_built)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_format_tables(fb_built):
    lib = fblib.load()
    assert lib.fb_abi_version() == 1 and lib.fb_compiled_sm() == 100
    # src/kernels/moe/moe_format.cpp:5-15 of the reference
    assert lib.fb_moe_row_bytes(21, 2560) == 1100 and lib.fb_moe_row_bytes(21, 512) == 220
    assert lib.fb_moe_row_bytes(20, 2560) == 1440 and lib.fb_moe_row_bytes(20, 640) == 360
    assert lib.fb_moe_row_bytes(21, 640) == 0 and lib.fb_moe_row_bytes(99, 2560) == 0
    assert lib.fb_moe_blob_bytes(21, 21, 512) == 1689600
    assert lib.fb_moe_blob_bytes(20, 20, 512) == 2211840
    assert lib.fb_moe_blob_bytes(21, 20, 640) == 2329600
    assert lib.fb_act_row_bytes(0, 2560) == 2920 and lib.fb_act_row_bytes(1, 2560) == 2720
    assert lib.fb_moe_act_format(21) == 0 and lib.fb_moe_act_format(20) == 1


def test_layout_and_argument_errors(fb_built):
    lib = fblib.load()
    lay = fblib.ExpertLayout()
    assert lib.fb_moe_expert_layout_make(0x1000, 1689600, 21, 21, 512, ctypes.byref(lay)) == 0
    assert (lay.gate_offset, lay.up_offset, lay.down_offset) == (0, 563200, 1126400)
    # IQ3_S down needs inter % 256 == 0; stride must hold a blob and be 16-aligned
    assert lib.fb_moe_expert_layout_make(0x1000, 4000000, 21, 21, 640, ctypes.byref(lay)) == 1
    assert lib.fb_moe_expert_layout_make(0x1000, 1000, 21, 21, 512, ctypes.byref(lay)) == 1
    assert b"blob_stride" in lib.fb_last_error_string()
    assert lib.fb_moe_decode_workspace_bytes(512) % 256 == 0
    # a CPU exchange is refused (no CPU tier) before anything is launched
    ws = fblib.DecodeWorkspace()
    for f in ("work", "xq", "h", "hq", "partial", "item_done", "sched", "status"):
        setattr(ws, f, 0x1000)
    st = lib.fb_moe_select_publish(0x1000, 513, 0x1000, 0, None, 0, None, 0x1000, 4, ctypes.byref(ws), None, None)
    assert st == 1 and b"exchange" in lib.fb_last_error_string()
    st = lib.fb_moe_select_publish(0x1000, 513, 0x1000, 0, None, 0, None, None, 17, ctypes.byref(ws), None, None)
    assert st == 1


def test_decode_width_projection_argument_checks(fb_built):
    """fb_linear_fp8_decode refuses bad shapes, epilogues and workspaces before anything is launched
    (where the reference throws std::invalid_argument, src/kernels/linear/linear_fp8.cpp:83-95)."""
    lib = fblib.load()
    need = lib.fb_linear_fp8_decode_workspace_bytes(2560, 640)
    # pieces [48][k] + two 256-byte words + tickets + 512 partial tiles of 128 x 16 fp32
    assert need == 48 * 640 + 256 + 256 + 256 + 512 * 128 * 16 * 4
    assert lib.fb_linear_fp8_decode_workspace_bytes(0, 640) == 0
    p = 0x10000
    epi = fblib.LinearEpilogue(fblib.EPI_STORE_F32, 0, p, None, None)
    e = ctypes.byref(epi)
    assert lib.fb_linear_fp8_decode(p, 0, p, p, 0, 256, 256, e, p, need, None) == 1
    assert lib.fb_linear_fp8_decode(p, 17, p, p, 0, 256, 256, e, p, need, None) == 1
    assert b"1..16" in lib.fb_last_error_string()
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 192, e, p, need, None) == 1     # k % 128
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 250, 256, e, p, need, None) == 1     # n % 8
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, e, p + 8, need, None) == 1  # workspace alignment
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, e, p, 1000, None) == 1
    assert b"workspace" in lib.fb_last_error_string()
    sw = fblib.LinearEpilogue(fblib.EPI_SWIGLU, 0, p, None, None)
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 264, 256, ctypes.byref(sw), p, need, None) == 1  # SwiGlu n % 16
    sh = fblib.LinearEpilogue(fblib.EPI_SHARED_SCALE, 513, p, None, None)
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, ctypes.byref(sh), p, need, None) == 1  # no gate logit
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, None, p, need, None) == 1


def test_peer_exchange_layer_refuses_rank_counts_that_do_not_divide_its_grid(fb_built):
    """fb_moe_layer_decode_ep_p2p hands the 128 blocks of its route kernel out to the ranks in equal
    shares, so only 1, 2, 4 and 8 ranks are accepted; 3 ranks with 3 tokens passes every other check
    and must be refused before anything is launched."""
    lib = fblib.load()
    lay = fblib.ExpertLayout()
    assert lib.fb_moe_expert_layout_make(0x1000, 1689600, 21, 21, 512, ctypes.byref(lay)) == 0
    ws = fblib.DecodeWorkspace()
    for f in ("work", "xq", "h", "hq", "partial", "item_done", "sched", "status"):
        setattr(ws, f, 0x1000)
    ws.gate_up_format, ws.down_format, ws.inter = 21, 21, 512
    for ranks, tokens in ((3, 3), (5, 5), (6, 12), (7, 14)):
        peers = fblib.EpPeers()
        peers.rank, peers.n_ranks = 0, ranks
        for d in range(ranks):
            peers.x_all[d], peers.y_parts[d] = 0x2000, 0x3000
        st = lib.fb_moe_layer_decode_ep_p2p(0x1000, ctypes.byref(lay), 0x1000, 0x1000, tokens, ctypes.byref(peers), 1,
                                            ctypes.byref(ws), 0x1000, 0x1000, None)
        assert st == 1 and b"1, 2, 4 or 8" in lib.fb_last_error_string(), ranks


def test_static_status_needs_a_prior_static_call(fb_built):
    """fb_moe_layer_decode_static_status reads the status word of the static array; before the static
    entry point has run on the device there is nothing to read and the call says so."""
    lib = fblib.load()
    out = ctypes.c_uint32(7)
    assert lib.fb_moe_layer_decode_static_status(None, None) == 1
    st = lib.fb_moe_layer_decode_static_status(ctypes.byref(out), None)
    assert st != 0 and out.value == 7


def test_ep_prefill_layer_scratch_and_argument_checks(fb_built):
    """fb_ep_prefill_layer refuses bad shapes before anything runs; the scratch grows with ranks and with the
    all-to-all combine's receive buffer."""
    import ctypes as C
    from fngine_b200 import lib as L
    lib = L.load()
    f = lib.fb_ep_prefill_scratch_bytes
    assert f(0, 2, 0) == 0 and f(64, 0, 0) == 0 and f(64, 9, 0) == 0
    rows = 64 * 2
    payload = rows * 2560 * 2 + rows * 2560 * 4 + 2 * rows * 40 + 2 * 64 * 40
    assert payload <= f(64, 2, 1) <= payload + 8 * 256
    assert f(64, 2, 0) - f(64, 2, 1) == rows * 2560 * 4
    assert f(64, 1, 0) == f(64, 1, 1)  # one rank: nothing to receive
    layout, ws = L.ExpertLayout(), L.PrefillWorkspace()
    assert lib.fb_ep_prefill_layer(None, None, None, 0, 256, None, 512, None, 64, 2, 0, None, None, None, None, None) != 0
    one = C.c_void_p(256)
    ws.capacity = 64
    args = lambda **kw: [C.byref(layout), one, kw.get("share"), kw.get("lo", 0), kw.get("hi", 256), one, 512, one,
                         kw.get("tokens", 64), kw.get("ranks", 2), kw.get("combine", 0), C.byref(ws), kw.get("scratch", one),
                         one, kw.get("comm"), None]
    assert lib.fb_ep_prefill_layer(*args(ranks=9)) != 0
    assert lib.fb_ep_prefill_layer(*args(combine=2)) != 0
    assert lib.fb_ep_prefill_layer(*args(scratch=C.c_void_p(264))) != 0
    assert lib.fb_ep_prefill_layer(*args()) != 0  # 128 rows in a workspace of 64
    assert b"capacity" in lib.fb_last_error_string()
    ws.capacity = 128
    assert lib.fb_ep_prefill_layer(*args(lo=300, hi=200)) != 0
    assert lib.fb_ep_prefill_layer(*args()) != 0  # two ranks, no communicator
    assert b"communicator" in lib.fb_last_error_string()
