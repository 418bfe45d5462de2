"""Generate the golden fixtures by running the UNMODIFIED reference on CPU.

Usage (only works where the reference checkout is present; the fixtures it writes are committed):

    python tests/golden/make_golden.py [--ref /path/to/Pyramid-Sparse-Attention]

The reference is pure Python + Triton.  Its kernels are executed with the Triton interpreter
(TRITON_INTERPRET=1) and three shims that touch no arithmetic: ``is_hip`` (asks a GPU driver),
``torch.cuda.device`` (context manager entered around launches) and ``python -O`` (drops an
``assert tensor.is_cuda`` in the legacy backward).  bf16 is not exercised through the kernels
(the interpreter's bf16 path yields NaN); the pure-torch mask builder is exercised in bf16 too.

Tie order: ``torch.sort(descending=True)`` on CPU is an unstable sort whose order among EQUAL scores
is an artefact of the host library (it is neither ascending nor descending index).  Cases named
``*_distinct`` hold rows of distinct scores and run the reference untouched.  Cases named ``*_ties``
and the end-to-end cases run the reference with ``torch.sort`` forced to ``stable=True`` (ties in
ascending index order - the order a stable device radix sort yields); nothing else is changed.

For every case the script stores the reference's outputs and, as a self-check, prints the
deviation of the CPU restatement (oracle/psa_oracle.py) from them.
"""
import argparse
import contextlib
import os
import sys

if __debug__ and __name__ == "__main__":
    os.execv(sys.executable, [sys.executable, "-O"] + sys.argv)

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
sys.path.insert(0, HERE)

import numpy as np
import torch

import cases as C
from oracle import psa_oracle as O


def load_reference(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    torch.cuda.device = lambda *a, **k: contextlib.nullcontext()
    import psa_triton  # noqa: F401
    from psa_triton.kernels import attn_pooling_kernel, psa_kernel, psa_kernel_legacy
    for m in (psa_kernel, psa_kernel_legacy, attn_pooling_kernel):
        m.is_hip = lambda: False
    return psa_triton


@contextlib.contextmanager
def stable_sort_shim():
    """Force stable=True on torch.sort so that equal scores come out in ascending index order."""
    orig = torch.sort

    def stable_sort(x, *a, **k):
        k["stable"] = True
        return orig(x, *a, **k)

    torch.sort = stable_sort
    try:
        yield
    finally:
        torch.sort = orig


def maxdiff(a, b):
    return float((a.double() - b.double()).abs().max())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("PSA_REFERENCE_DIR"), required=os.environ.get("PSA_REFERENCE_DIR") is None,
                    help="checkout of ziplab/Pyramid-Sparse-Attention (or set PSA_REFERENCE_DIR)")
    args = ap.parse_args()
    load_reference(args.ref)
    import psa_triton.attention as RA
    from psa_triton.kernels.attn_pooling_kernel import attn_with_pooling_optimized
    from psa_triton.kernels.calc_ksim_kernel import calc_k_similarity_pytorch, calc_k_similarity_triton
    from psa_triton.kernels.psa_kernel import pooling as ref_pooling, pad_to_multiple as ref_pad
    from psa_triton.kernels.psa_kernel import sparse_attention_factory as new_factory
    from psa_triton.kernels.psa_kernel_legacy import sparse_attention_factory as legacy_factory
    from psa_triton.utils.transfer_attn_to_mask import (calc_density, calc_density_newtype,
                                                          transfer_attn_to_mask)

    out = {}

    # ---- pyramid (a1) -------------------------------------------------------------
    for dt in ("fp32", "bf16", "fp16"):
        x = C.randn(11, (1, 2, 333, 64), C.DT[dt])
        xp = ref_pad(x, 64)
        r2 = ref_pooling(xp, 2); r4 = ref_pooling(r2, 2); r8 = ref_pooling(r4, 2)
        mine = O.pyramid_kv(x, 64)
        for l, r in ((2, r2), (4, r4), (8, r8)):
            assert torch.equal(mine[l], r), f"pyramid {dt} level {l}"
            out[f"pyramid_{dt}_l{l}"] = r.float().numpy()
    print("pyramid: oracle bit-equal to reference (fp32/bf16/fp16)")

    # ---- block scores (a2+a3) -------------------------------------------------------
    for name, S, D, H, bm, bn, dt in C.SCORE_CASES:
        q, k, v = C.qkv(100, 1, H, S, D, C.DT[dt])
        iq, ik = C.sample_idx(7, 1, H, bm, bm // 4), C.sample_idx(8, 1, H, bn, bn // 4)
        sq, sk = O.gather_samples(q, bm, iq), O.gather_samples(k, bn, ik)
        # the reference's own sampler, driven with our indices, must pick the same rows
        _, po = attn_with_pooling_optimized(sq, sk, v, False, 1.0 / (D ** 0.5), bm // 4, bn // 4)
        Mq, Nk = -(-S // bm), -(-S // bn)
        po = po[:, :, :Mq, :Nk].contiguous()
        mine = O.block_scores(q, k, iq, ik, bm, bn)
        print(f"scores {name}: oracle vs ref max|d| = {maxdiff(mine, po):.3e}  (row max {float(po.max()):.3e})")
        out[f"scores_{name}"] = po.float().numpy()

    # reference sampler equivalence (attention.py:116-137) under a fixed torch seed
    x = C.randn(5, (1, 2, 300, 64))
    torch.manual_seed(1234)
    ref_s = RA._random_sample_tokens(RA._pad_to_multiple(x, 64), 64, 16)
    torch.manual_seed(1234)
    idx = O.draw_sample_indices(1, 2, 64, 16)
    mine_s = O.gather_samples(x, 64, idx)[:, :, :ref_s.shape[2]]
    assert torch.equal(ref_s, mine_s)
    print("sampler: oracle bit-equal to reference")

    # ---- level assignment (a4/a5) + density (a10) ---------------------------------------
    nbad = 0
    for name, Mq, Nk, bn, tn, mode, rn, dt, text, ties in C.ASSIGN_CASES:
        po = C.scores_like(sum(map(ord, name)), 1, 2, Mq, Nk, C.DT[dt], ties=ties)
        ratios = getattr(C, rn)
        with (stable_sort_shim() if ties else contextlib.nullcontext()):
            ref = transfer_attn_to_mask(po, ratios, text_length=text, mode=mode, blocksize=bn, compute_tile=tn)
        mine = O.assign_levels(po, ratios, mode, bn, tn, text_length=text)
        if not torch.equal(ref, mine):
            nbad += 1
            print("MISMATCH", name, int((ref != mine).sum()))
        out[f"assign_{name}"] = ref.numpy().astype(np.int32)
        if mode.endswith("newtype") and len(ratios) == 5:
            d_ref = calc_density_newtype(ref)
            d_mine = O.density_newtype(ref)
            assert abs(d_ref[0] - d_mine[0]) < 1e-6
            out[f"density_{name}"] = np.array([d_ref[0]] + d_ref[1], dtype=np.float64)
        elif not mode.endswith("newtype"):
            d_ref = calc_density(ref)
            d_mine = O.density_old(ref)
            assert abs(d_ref[0] - d_mine[0]) < 1e-6
            out[f"density_{name}"] = np.array([d_ref[0]] + d_ref[1], dtype=np.float64)
    print(f"assign: {len(C.ASSIGN_CASES)} cases, {nbad} mismatching the oracle")
    assert nbad == 0

    # ---- new-mask forward (a6) --------------------------------------------------------
    for name, S, D, H, bm, bn, tn, mode, rn in C.FWD_CASES:
        q, k, v = C.qkv(200, 1, H, S, D)
        Mq, Nk = -(-S // bm), -(-S // bn)
        po = C.scores_like(300, 1, H, Mq, Nk, torch.float32)
        mask = transfer_attn_to_mask(po, getattr(C, rn), text_length=0, mode=mode + "_newtype", blocksize=bn,
                                     compute_tile=tn)
        ref = new_factory(bm, tn, bn)(q, k, v, mask, None)
        mine = O.psa_forward_newmask(q, k, v, mask, bm, bn, tn, quirk=True)
        clean = O.psa_forward_newmask(q, k, v, mask, bm, bn, tn, quirk=False)
        print(f"fwd {name}: oracle(quirk) vs ref {maxdiff(mine, ref):.3e}; oracle(clean) vs ref {maxdiff(clean, ref):.3e}")
        out[f"{name}_out"] = C.sub(ref.numpy())
        out[f"{name}_mask"] = mask.numpy()

    # ---- legacy forward + backward (a7/a8) -----------------------------------------------
    for name, S, D, H, B, causal, diag1 in C.LEGACY_CASES:
        q, k, v = C.qkv(400, B, H, S, D)
        do = C.randn(404, (B, H, S, D))
        mask = C.legacy_mask(405, B, H, S, causal, diag1)
        fn = legacy_factory(128, 32, 128, causal=causal)
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = fn(qr, kr, vr, mask, None)
        o.backward(do)
        mo, mlse = O.legacy_forward(q, k, v, mask, causal)
        dq, dk, dv = O.legacy_backward(q, k, v, mask, mo, mlse, do, causal)
        print(f"legacy {name}: fwd {maxdiff(mo, o.detach()):.3e} dq {maxdiff(dq, qr.grad):.3e} "
              f"dk {maxdiff(dk, kr.grad):.3e} dv {maxdiff(dv, vr.grad):.3e}")
        out[f"{name}_out"] = C.sub(o.detach().numpy())
        out[f"{name}_dq"] = C.sub(qr.grad.numpy()); out[f"{name}_dk"] = C.sub(kr.grad.numpy()); out[f"{name}_dv"] = C.sub(vr.grad.numpy())

    # ---- K similarity (a9) -----------------------------------------------------------
    class T:  # thresholds of the Wan2.1_1.3b preset (configs/attention_config.yaml)
        sim_2x_threshold, sim_4x_threshold, sim_8x_threshold = 0.7, 0.65, 0.6
    for name, S, D, H, bn in C.KSIM_CASES:
        k = C.randn(500, (1, H, S, D), smooth=12)
        k = k * torch.linspace(0.05, 3.0, S).view(1, 1, S, 1) ** 2 + C.randn(501, (1, H, 1, D)) * torch.linspace(2.0, 0.0, S).view(1, 1, S, 1)
        kp = RA._pad_to_multiple(k, bn)
        ref_t = calc_k_similarity_triton(kp, bn, T)
        ref_p = calc_k_similarity_pytorch(kp, bn, T)
        mine = O.k_similarity(k, bn, 0.7, 0.65, 0.6)
        print(f"ksim {name}: oracle==triton {bool(torch.equal(mine, ref_t))} "
              f"triton==pytorch-fallback {bool(torch.equal(ref_t.to(ref_p.dtype), ref_p))} hist {torch.bincount(ref_t.flatten()).tolist()}")
        out[name] = ref_t.numpy().astype(np.int32)

    # ---- whole plug-and-play call (attention.py:261-310) ---------------------------------
    for name, S, D, H, kw, seed in C.E2E_CASES:
        kw = dict(kw)
        if "mask_ratios" in kw:
            kw["mask_ratios"] = getattr(C, kw["mask_ratios"])
        q, k, v = C.qkv(600, 1, H, S, D)
        cfg = RA.PSAConfig(**kw)
        torch.manual_seed(seed)
        with stable_sort_shim():
            ref = RA.PSAAttention(cfg)(q, k, v)
        torch.manual_seed(seed)
        mine, mmask, _ = O.psa_attention(q, k, v, block_m=cfg.block_m, block_n=cfg.block_n, tile_n=cfg.tile_n,
                                         mask_ratios=cfg.mask_ratios, mask_mode=cfg.mask_mode, attn_impl=cfg.attn_impl)
        print(f"e2e {name}: oracle vs ref {maxdiff(mine, ref):.3e}")
        out[f"{name}_out"] = C.sub(ref.numpy())
        # the reference's module returns no mask: this is the ORACLE's mask for the same inputs and sample offsets (the
        # oracle's assignment is pinned bit for bit against transfer_attn_to_mask by the assign_* fixtures above)
        out[f"{name}_mask"] = mmask.numpy()

    # ---- Gilbert curve order (src/psa_triton/utils/gilbert3d.py via GilbertRearranger) ----------------
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_gilbert3d", os.path.join(args.ref, "src/psa_triton/utils/gilbert3d.py"))
    g3 = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(g3)
    from psa_b200.rearrange import gilbert_order
    for (w, h, d) in C.GILBERT_SHAPES:
        ref = np.array([x + w * (y + h * z) for x, y, z in g3.gilbert3d(w, h, d)], dtype=np.int64)
        assert np.array_equal(ref, gilbert_order(w, h, d)), (w, h, d)
        if ref.size <= 512:
            out[f"gilbert_{w}x{h}x{d}"] = ref.astype(np.int32)
        out[f"gilbert_sum_{w}x{h}x{d}"] = np.array([C.order_checksum(ref)], dtype=np.int64)
    print("gilbert: own curve equals the reference's on", len(C.GILBERT_SHAPES), "grids")

    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, f"{os.path.getsize(path) / 1e6:.2f} MB, {len(out)} arrays")


if __name__ == "__main__":
    main()
