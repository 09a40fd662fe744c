"""Test configuration: the `gpu` marker (tests that need a B200), import paths, shared helpers."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import dm_oracle
    return dm_oracle


def load_golden(name):
    """One golden case as a dict of torch tensors (bf16 tensors rebuilt from their bit patterns)."""
    import numpy as np
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        if k in ("q", "k", "v", "do", "O"):
            out[k] = torch.from_numpy(a.copy()).view(torch.bfloat16)
        elif k.endswith("_codes"):
            out[k] = torch.from_numpy(a.copy())
        elif a.dtype.kind in "US":
            out[k] = str(a)
        else:
            out[k] = torch.from_numpy(a.copy())
    B, N, H, Hk, D, causal, seed = (int(x) for x in out["shape"])
    out["dims"] = dict(B=B, N=N, H=H, Hk=Hk, D=D, causal=bool(causal), seed=seed)
    return out


GOLDEN_CASES = ("c1_matched", "c1_stale", "gqa_noncausal_stale", "hd256_matched",
                "c1_matched_ds32", "c1_stale_ds32", "c1_matched_nonorm", "hd256_matched_ds32")
