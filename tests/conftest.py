import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped (not failed) when no CUDA device is visible and they were not
    explicitly selected with -m gpu."""
    import torch
    if torch.cuda.is_available():
        return
    selected = config.getoption("-m") or ""
    if "gpu" in selected and "not gpu" not in selected:
        return  # asked for explicitly: let them fail loudly
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    return O


def make_weights(N, K, seed, std=0.02):
    """fp32 weights ~N(0, std) from one PCG64 generator per tensor."""
    return (np.random.Generator(np.random.PCG64(seed)).standard_normal((N, K)) * std).astype(np.float32)


def make_acts(M, K, seed, dtype):
    """activations ~N(0,1) rounded to the activation dtype; returns (torch tensor on CPU, fp32 values)."""
    import torch
    x = np.random.Generator(np.random.PCG64(seed)).standard_normal((M, K)).astype(np.float32)
    t = torch.from_numpy(x).to(dtype)
    return t, t.to(torch.float32).numpy()


def fuzz_blocks(qt, nblocks, seed):
    """Random bytes for `nblocks` blocks with every fp16 field forced finite (Inf/NaN scales
    are outside the bit-exact gate: the reference canonicalises NaN)."""
    from oracle import oracle as O
    bb = O.block_bytes(qt)
    rng = np.random.Generator(np.random.PCG64(seed))
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    half_fields = {O.Q4_0: [0], O.Q4_1: [0, 2], O.Q8_0: [0], O.Q4_K: [0, 2], O.NF4: [0]}[qt]
    for off in half_fields:
        hi = raw[:, off + 1]
        bad = (hi & 0x7C) == 0x7C           # exponent all ones
        raw[bad, off + 1] = hi[bad] & 0xBF  # clear one exponent bit
    return raw.reshape(-1)
