"""Activation test patterns shared by the CPU and GPU quantizer tests.

The categories are the ones the reference's quantizer test exercises
(tests/cpu/test_q8_quant.cpp:17-36): plain normals, many magnitude ties with the negative
maximum first, all-zero rows, a single non-zero per stretch, very small and very large scales,
values exactly on .5 rounding boundaries, and sign-alternating uniforms.
"""
import numpy as np

from fngine_b200 import synth

N_PATTERNS = 8


def make_input(k, pattern, seed):
    n = synth.normal(seed, k)
    u = synth.uniform(seed ^ 0x5151, 0, k)
    i = np.arange(k)
    if pattern == 0:
        x = n
    elif pattern == 1:
        x = np.floor(u * 9 - 4) * 0.25
        x[0], x[1] = -1.0, 1.0
    elif pattern == 2:
        x = np.zeros(k)
    elif pattern == 3:
        x = np.where(i % 97 == 5, n, 0.0)
    elif pattern == 4:
        x = n * 1e-30
    elif pattern == 5:
        x = n * 3e4
    elif pattern == 6:
        x = (np.floor(u * 509 - 254) + 0.5) / 254.0 * 127.0
    else:
        x = (u * 2 - 1) * np.where(i % 32 == 0, -1.0, 0.5)
    return x.astype(np.float32)


def all_inputs(k=2560, trials=24, seed=1234):
    return np.stack([make_input(k, t % N_PATTERNS, seed + 17 * t) for t in range(trials)])
