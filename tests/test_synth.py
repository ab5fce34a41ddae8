import numpy as np

from fngine_b200 import synth


def test_splitmix_matches_sequential_generator():
    # tests/common/test_util.h:58-67 of the reference: state += golden; mix.
    state = 42
    want = []
    for _ in range(5):
        state = (state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        want.append(z ^ (z >> 31))
    assert [int(v) for v in synth.splitmix_words(42, 0, 5)] == want
    assert [int(v) for v in synth.splitmix_words(42, 2, 3)] == want[2:]


def test_blocks_are_position_addressed():
    a = synth.fill_blocks(21, 10, 0, 9)
    b = synth.fill_blocks(21, 4, 6, 9)
    assert np.array_equal(a[6 * 110:], b)
    assert synth.blob_bytes(21, 21, 512) == 1689600 == len(synth.expert_blob(21, 21, 512, 1, 0))
    assert synth.blob_bytes(20, 20, 512) == 2211840


def test_scale_distribution():
    t = synth.d_table(21).view(np.float16).astype(np.float64)
    assert abs(t.mean() - 0.02 * np.sqrt(2 / np.pi)) < 5e-4
    x = synth.activations(3, 4)
    assert abs(x.std() - 1) < 0.02
