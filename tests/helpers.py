"""Shared helpers of the GPU parity tests: run the CUDA path through the public API / op layer, run the oracle on the
same inputs (on the kernel's own K mean, as the reference's tests do: tests/test_sm100.py:79-96), record distances."""
import json
import os

import torch


def run_api(q, k, v, do, causal, mode, numerics="sm100-mx"):
    """Forward + backward through dm_attn_func and autograd -> dict O, dQ, dK, dV."""
    import delta_matching_b200 as dm
    from delta_matching_b200 import ops
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    o = dm.dm_attn_func(*leaves, causal=causal, mode=mode, numerics=numerics)
    o.backward(do)
    torch.cuda.synchronize()
    ops.check_status(q.device)
    return {"O": o.detach(), "dQ": leaves[0].grad, "dK": leaves[1].grad, "dV": leaves[2].grad}


def run_ops(q, k, v, do, causal, mode, identity=False, numerics="sm100-mx", two_pass=True):
    """The same pipeline through the op layer, keeping the intermediates (codes, scales, K mean, LSE, delta).
    two_pass=False takes the backward without a workspace (the dQ kernel that recomputes)."""
    import os
    from delta_matching_b200 import ops
    ds32, norm = ops.NUMERICS[numerics]
    qh, kh, vh, doh = (t.transpose(1, 2) for t in (q, k, v, do))
    q8, qs, k8, ks, v8, vs, km = ops.quant_qkv(qh, kh, vh)
    o, lse = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
    if mode == "matched":
        do8, dos, _ = ops.quant_do(doh, None)
        delta = ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal, norm)
    else:
        do8, dos, delta = ops.quant_do(doh, o.permute(0, 2, 1, 3))
    old = os.environ.get("DM_BWD_WORKSPACE_MB")
    if not two_pass:
        os.environ["DM_BWD_WORKSPACE_MB"] = "0"
    try:
        res = ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, identity=identity, ds32=ds32)
    finally:
        if not two_pass:
            if old is None:
                del os.environ["DM_BWD_WORKSPACE_MB"]
            else:
                os.environ["DM_BWD_WORKSPACE_MB"] = old
    torch.cuda.synchronize()
    ops.check_status(q.device)
    out = {"O": o, "LSE": lse, "delta": delta, "dQ": res[0], "dK": res[1], "dV": res[2], "kmean": km,
           "q8": q8, "qs": qs, "k8": k8, "ks": ks, "v8": v8, "vs": vs, "do8": do8, "dos": dos}
    if identity:
        out["rowsum_dS"], out["sum_abs_PdP"] = res[3], res[4]
    return out


def record(test, case, name, value):
    """DM_TEST_RECORD=<file>: append measured distances as JSON lines (the reference's tests/test_sm100.py:64-70)."""
    f = os.environ.get("DM_TEST_RECORD")
    if f:
        with open(f, "a") as fh:
            fh.write(json.dumps({"test": test, "case": case, "out": name, "value": value}) + "\n")
