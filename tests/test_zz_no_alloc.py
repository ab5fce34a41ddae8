"""The allocation-free decode entry point (fb_moe_layer_decode_static).

Some users of the library cannot allocate device memory at the point where a layer runs (their
memory plan is frozen, or they are a plug-in that only receives tensor pointers). For them the
layer's scratch lives in a static device array inside the library. This test calls that entry
point through the C ABI twice in a row and checks both results, bit for bit, against the regular
entry point that takes a caller workspace. It is collected last on purpose: a run that stops at
the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest

from fngine_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_layer_matches_workspace_layer():
    import torch
    from fngine_b200 import lib as fblib
    from fngine_b200 import moe
    assert torch.cuda.is_available()
    layer = moe.synth_layer(21, 21, 512, 512, 31337)
    wr = torch.from_numpy(synth.router_weights(808, rows=512).view(np.int16)).cuda().view(torch.bfloat16)
    ws = moe.DecodeWorkspace(layer)
    for call, tokens in enumerate((5, 16)):  # two calls in a row share the static array
        x = torch.from_numpy(synth.activations(900 + call, tokens)).cuda()
        want = torch.empty(tokens, 2560, dtype=torch.float32, device="cuda")
        moe.moe_layer_decode(wr, layer, x, ws, want)
        got = torch.full((tokens, 2560), float("nan"), dtype=torch.float32, device="cuda")
        moe.moe_layer_decode_static(wr, layer, x, got)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
        # the hidden scratch's status word is readable: no bounded wait ran out, the work list was usable
        assert moe.moe_layer_decode_static_status() == 0
    # requests beyond the static array's size are refused, nothing is launched
    lib = fblib.load()
    st = lib.fb_moe_layer_decode_static(wr.data_ptr(), ctypes.byref(layer.layout), x.data_ptr(), 0, 17,
                                        got.data_ptr(), None)
    assert st == 1 and b"tokens must be 1..16" in lib.fb_last_error_string()
