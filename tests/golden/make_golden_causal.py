"""Golden fixtures of the causal (vision-language) call site, produced by running the UNMODIFIED reference on CPU.

    python tests/golden/make_golden_causal.py --ref /path/to/Pyramid-Sparse-Attention

Runs the reference's own ``estimate_block_importance`` (its pure-PyTorch branch, ``use_triton=False``: no GPU here) and
``transfer_attn_to_mask`` from qwen2.5-vl-example/src/attention/PSA_casual on the seeded inputs of cases.py, stores the
outputs in causal_reference_outputs.npz and prints the deviation of the CPU restatement (oracle/psa_oracle.py).
``torch.sort`` is forced to ``stable=True`` for the mask builder (equal scores - the zeros above the diagonal - then
come in ascending column order, which is the rule the kernels implement); nothing else is touched.
"""
import argparse
import contextlib
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import numpy as np
import torch

import cases as C
from oracle import psa_oracle as O


@contextlib.contextmanager
def stable_sort_shim():
    orig = torch.sort

    def stable_sort(x, *a, **k):
        k["stable"] = True
        return orig(x, *a, **k)

    torch.sort = stable_sort
    try:
        yield
    finally:
        torch.sort = orig


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of ziplab/Pyramid-Sparse-Attention")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "qwen2.5-vl-example", "src", "attention"))
    from PSA_casual.PyramidAdaptiveBlockSparseAttn import estimate_block_importance, transfer_attn_to_mask

    out = {}
    for name, L, D, H, block, stride, chunk, causal in C.ANTIDIAG_CASES:
        q, k, _ = C.qkv(500, 1, H, L, D, torch.float32)
        ref = estimate_block_importance(q, k, block_size=block, stride=stride, norm=1.0, softmax=True, chunk_size=chunk,
                                        select_mode="inverse", use_triton=False, causal=causal, kdb=1)
        mine = O.antidiag_block_scores(q, k, block, stride, causal, chunk)
        print(f"{name}: |oracle - reference| = {float((mine - ref.double()).abs().max()):.3e}  (max {float(ref.max()):.3f})")
        out[name] = ref.float().numpy()

    bad = 0
    for name, n, H, dt, mode, causal, text in C.CAUSAL_MASK_CASES:
        attn = C.causal_scores(900 + n, H, n, C.DT[dt], causal)
        ratios = C.RATIOS_CAUSAL if mode == "topk" else C.RATIOS_ENERGY
        with stable_sort_shim():
            ref = transfer_attn_to_mask(attn, ratios, text, mode, block_size=128, causal=causal)
        mine = O.causal_level_mask(attn, ratios, text, mode, 128, causal)
        diff = int((mine != ref).sum())
        bad += diff
        if diff:
            print(f"{name}: {diff} of {ref.numel()} mask entries differ")
        out[name] = ref.to(torch.int8).numpy()
    print(f"causal level masks: {len(C.CAUSAL_MASK_CASES)} cases, {bad} differing entries in total")
    np.savez_compressed(os.path.join(HERE, "causal_reference_outputs.npz"), **out)


if __name__ == "__main__":
    main()
