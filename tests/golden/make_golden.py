"""Generate the golden vectors of tests/golden/ by running the reference's own emulation.

Run where a checkout of the reference (jet-ai-projects/delta-matching) is available and pass its path (or set
DM_REFERENCE_ROOT):

    python tests/golden/make_golden.py /path/to/delta-matching [case ...]      (no case names: all of them)

It loads delta_matching/reference.py by file path (that file has no imports besides torch), runs `dm_reference` with the
Blackwell presets on small seeded inputs, and writes one compressed .npz per case with the inputs (bf16 bit patterns),
the reference's producer codes and scales, and its outputs.  The reference cannot travel to the GPU machine; these files
can.  Cases: the CPU-runnable headline configuration (B=1, N=256, H=Hk=2, D=128, causal) in both delta modes, a
non-causal GQA stale case, and a head_dim-256 case; then the other numerics arms the kernels implement (dS scaled per
32 x 32 block at both head dims, matched delta without the division by sum P).
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = {
    # name: (B, N, H, Hk, D, causal, mode, seed, preset)
    "c1_matched": (1, 256, 2, 2, 128, True, "matched", 0, "sm100-mx"),
    "c1_stale": (1, 256, 2, 2, 128, True, "stale", 0, "sm100-mx"),
    "gqa_noncausal_stale": (1, 128, 2, 1, 128, False, "stale", 1, "sm100-mx"),
    "hd256_matched": (1, 128, 1, 1, 256, True, "matched", 2, "sm100-mx-d256"),
    "c1_matched_ds32": (1, 256, 2, 2, 128, True, "matched", 0, "sm100-mx-ds32"),
    "c1_stale_ds32": (1, 256, 2, 2, 128, True, "stale", 0, "sm100-mx-ds32"),
    "c1_matched_nonorm": (1, 256, 2, 2, 128, True, "matched", 0, "sm100-mx-nonorm"),
    "hd256_matched_ds32": (1, 128, 1, 1, 256, True, "matched", 2, "sm100-mx-d256-ds32"),
}


def load_reference(root):
    path = os.path.join(root, "delta_matching", "reference.py")
    spec = importlib.util.spec_from_file_location("dm_reference_golden", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits16(t):
    return t.contiguous().view(torch.int16).numpy()


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DM_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: make_golden.py /path/to/delta-matching [case ...]   (or set DM_REFERENCE_ROOT)")
    only = set(sys.argv[2:])
    if only - set(CASES):
        sys.exit(f"unknown case(s): {sorted(only - set(CASES))}")
    R = load_reference(root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name, (B, N, H, Hk, D, causal, mode, seed, preset) in CASES.items():
        if only and name not in only:
            continue
        g = torch.Generator(device="cpu").manual_seed(seed)
        q, k, v, do = [torch.randn(B, N, h, D, generator=g).to(torch.bfloat16) for h in (H, Hk, Hk, H)]
        r = R.dm_reference(q, k, v, do, causal, mode, preset, aux=True)
        out = {"shape": np.array([B, N, H, Hk, D, int(causal), seed]), "mode": np.array(mode), "preset": np.array(preset),
               "q": bits16(q), "k": bits16(k), "v": bits16(v), "do": bits16(do),
               "O": bits16(r["O"].contiguous()), "LSE": r["LSE"].numpy(), "delta": r["delta"].numpy(),
               "dQ": r["dQ"].contiguous().numpy(), "dK": r["dK"].contiguous().numpy(),
               "rowsum_dS": r["rowsum_dS"].numpy(), "sum_absPdP": r["sum_absPdP"].numpy()}
        if mode == "matched":          # dV does not depend on the delta mode
            out["dV"] = r["dV"].contiguous().numpy()
        # the producers, through the reference's own quantiser pieces (reference.py:96-107, 328-338, 408-416)
        f32 = torch.float32
        kh = k.to(f32).transpose(1, 2)
        km = R.kmean_sm90(kh)
        out["kmean"] = km.squeeze(-2).numpy()
        for nm, x in (("q", q.to(f32).transpose(1, 2) * (D ** -0.5)), ("k", kh - km), ("v", v.to(f32).transpose(1, 2)),
                      ("do", do.to(f32).transpose(1, 2))):
            xb = x.reshape(B, x.shape[1], N // 32, 32 * D)
            s = R.pow2_scale(xb.abs().amax(-1, keepdim=True))
            codes = R.e4m3_round(xb / s).reshape(B, x.shape[1], N, D)
            assert torch.equal((codes.reshape(xb.shape) * s).reshape(x.shape), R.fake_blockrows_pow2(x, 32))
            out[nm + "_codes"] = codes.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
            out[nm + "_scales"] = s.squeeze(-1).numpy()
        ex = R.attention_fp32(q, k, v, do, causal)
        out["err_vs_fp32"] = np.array([float(((r[n].double() - ex[n].double()).norm() / ex[n].double().norm()))
                                       for n in ("O", "dQ", "dK", "dV")])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {n: round(float(e), 4) for n, e in zip(("O", "dQ", "dK", "dV"), out["err_vs_fp32"])})


if __name__ == "__main__":
    main()
