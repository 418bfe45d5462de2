#!/usr/bin/env python
"""PSA attention-layer benchmark on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A "step" is one Pyramid-Sparse-Attention layer call (pyramid K/V builder -> block scores -> level assignment ->
multi-level sparse forward) on a Wan2.1-14B-shaped attention layer (B=1, 40 heads x 128, S=75600 video tokens on a
21x45x80 latent grid, bf16, ~90% block sparsity; other shapes via --workload).  Inputs are seeded synthetic
structured fields (psa_b200/synthetic.py).

N GPUs: heads are sharded across ranks (strong scaling, total work fixed).  Activations start sequence-sharded
([S/N, H, D] per rank, as a sequence-parallel DiT holds them) and are reshuffled to head-sharded with one NCCL
all-to-all before the layer and one after it; both are inside the timed region.

Prints ONE JSON line (rank 0).  `value` = dense-equivalent TFLOP/s of the whole job (4*B*H*S^2*D / step time) with
inputs resident in HBM; `e2e` = the same through the public module call with pinned HOST q/k/v in and O back out.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
sys.path.insert(0, ROOT)

import torch

RATIOS_90 = {1: (0.0, 0.05), 2: (0.05, 0.1), 4: (0.1, 0.15), 8: (0.15, 0.25), 0: (0.25, 1.0)}
DEFAULT_RATIOS = {1: (0.0, 0.1), 2: (0.1, 0.15), 4: (0.15, 0.15), 8: (0.15, 0.35), 0: (0.35, 1.0)}
BLOCK_M, BLOCK_N, TILE_N = 128, 64, 32
CPU_SAMPLE_TOKENS = 32768


# kernels of this library launched by one call of each entry point the benchmark uses (memsets and torch's own
# kernels are not counted)
KERNELS_PER_CALL = {
    "psa_pyramid_kv_images": 1, "psa_pyramid_kv": 1, "psa_block_scores": 4, "psa_block_scores_samples": 2,
    # bf16 forward: the fixed-reference kernel and, right behind it, the exact kernel that returns at once unless the first
    # one raised its guard word
    "psa_assign_levels": 1, "psa_fwd_images": 2, "psa_fwd": 2, "psa_fwd_images_scatter": 2, "psa_push_heads": 1,
    "psa_push_samples": 1, "psa_pull_heads": 1, "psa_density": 1, "psa_legacy_fwd_images": 2, "psa_legacy_bwd_tc": 3,
    "psa_legacy_bwd_tcgen05": 5, "psa_ksim": 1, "psa_ksim_perm": 1, "psa_legacy_fwd_images_perm": 2, "psa_gather_rows": 1,
    "psa_pyramid_kv_images_perm": 1, "psa_block_scores_perm": 4, "psa_antidiag_scores_impl": 2, "psa_assign_levels_causal": 1,
}


class LaunchCounter:
    """Counts this library's kernel launches by wrapping the C-ABI entry points (calls x kernels per call)."""

    def __init__(self, lib):
        self.lib, self.count, self.on, self.orig = lib, 0, False, {}
        for name, per_call in KERNELS_PER_CALL.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue
            self.orig[name] = fn
            setattr(lib, name, self._wrap(fn, per_call))

    def _wrap(self, fn, per_call):
        def call(*a):
            if self.on:
                self.count += per_call
            return fn(*a)
        return call


# DRAM read+write bytes of one forward launch per (head x token), from ncu captures of psa_fwd_tc_kernel at the named
# shape with a reduced head count (profiles/); the figure is about the unique bytes of Q, O and the K/V images, so it
# scales with heads x tokens.
FWD_TRAFFIC_PER_HEAD_TOKEN = {
    "wan2.1-1.3b-attn-layer": (1539.0, "profiles/psa_fwd_tc_kernel__wan2.1-1.3b-shape_6heads.md"),
    "wan2.1-14b-attn-layer": (2837.0, "profiles/psa_fwd_tc_kernel__wan2.1-14b-shape_5heads_dram.md"),
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []
        self.t_begin = self.t_end = None

    def mark_begin(self):
        self.t_begin = time.monotonic()

    def mark_end(self):
        self.t_end = time.monotonic()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        # the sampler is started before the warm-up steps (nvidia-smi takes a while to come up); only the samples taken
        # inside the marked (timed) window count, widened by one sampling period when the window was very short
        lo = (self.t_begin or 0.0) - 0.06
        hi = (self.t_end or float("inf")) + 0.06
        inside = [(ts, ln) for ts, ln in self.lines if lo <= ts <= hi]
        window = "timed region"
        if not inside:
            # a timed region of a few tens of milliseconds can fall between two samples: take the ones right around it
            inside = [(ts, ln) for ts, ln in self.lines if lo - 0.5 <= ts <= hi + 0.5]
            window = "within 0.5 s of the timed region"
        sm, mx, reasons = [], [], set()
        for ts, ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def load_synthetic():
    """The input generator, loaded by file so that the CPU arms never import the package (whose __init__ opens the CUDA
    library)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "psa_synthetic_inputs", os.path.join(ROOT, "pyramid-sparse-attention_b200", "psa_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def use_all_host_threads() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm uses every core it is given."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def oracle_sample_time(workload, ratios, steps, warmup):
    """Time the CPU restatement of the same layer on a bounded sample (head 0, first CPU_SAMPLE_TOKENS tokens).
    Returns (dense-equivalent TFLOP/s, seconds per call, description)."""
    from oracle import psa_oracle as O
    synthetic = load_synthetic()
    use_all_host_threads()
    S = min(synthetic.seq_len(workload), CPU_SAMPLE_TOKENS)
    D = workload["head_dim"]
    q, k, v = synthetic.make_qkv(workload, 1000, torch.float32, "cpu", head_range=(0, 1), token_range=(0, S))
    times = []
    for i in range(warmup + steps):
        torch.manual_seed(2000)
        t0 = time.perf_counter()
        O.psa_attention(q, k, v, block_m=BLOCK_M, block_n=BLOCK_N, tile_n=TILE_N, mask_ratios=ratios, mask_mode="topk")
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    f_dense = 4.0 * S * S * D
    return f_dense / sec / 1e12, sec, f"head 0 of {workload['heads']}, first {S} tokens, fp32 inputs, fp64 softmax"


def oracle_legacy_sample_time(workload, steps, warmup, tokens=4096):
    """CPU restatement of the causal legacy forward + backward on a bounded sample: (batch 0, head 0), first `tokens`
    tokens.  Returns (dense-equivalent TFLOP/s of forward+backward, seconds per call, description)."""
    from oracle import psa_oracle as O
    synthetic = load_synthetic()
    use_all_host_threads()
    S, D = min(synthetic.seq_len(workload), tokens), workload["head_dim"]
    q, k, v = synthetic.make_qkv(workload, 1000, torch.float32, "cpu", head_range=(0, 1), token_range=(0, S))
    do = torch.randn(q.shape, generator=torch.Generator().manual_seed(5))
    mask = legacy_level_mask(77, 1, 1, S)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        o, lse = O.legacy_forward(q, k, v, mask, causal=True)
        O.legacy_backward(q, k, v, mask, o, lse, do, causal=True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return 3.5 * 2.0 * S * S * D / sec / 1e12, sec, f"batch 0, head 0, first {S} tokens, fp32 inputs, fp64 math"


def legacy_level_mask(seed, B, H, S):
    """Random causal old-format mask [B, H, S/128, S/128] in {0,1,2,4,8} (p = 0.2/0.3/0.2/0.15/0.15), column 0 at level 1
    so that no row is empty.  Mean token density ~0.46 of the causal triangle."""
    import numpy as np
    n = -(-S // 128)
    rng = np.random.default_rng(seed)
    m = rng.choice(np.array([0, 1, 2, 4, 8], dtype=np.int32), size=(B, H, n, n), p=[0.2, 0.3, 0.2, 0.15, 0.15])
    m[..., 0] = 1
    m = m * np.tril(np.ones((n, n), dtype=np.int32))
    return torch.from_numpy(m.astype(np.int32))


def run_causal_training(args, workload, synthetic):
    """--workload causal-legacy-fwd-bwd: one training step of the legacy (old-format mask) kernels, causal forward +
    backward on B=2 x 16 heads x 32768 tokens x 128, bf16, random level mask (token density ~0.46 of the causal triangle),
    dO ~ N(0,1).  The (batch, head) pairs are independent: N GPUs take 32/N of them each, no collective."""
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    B, H, D, S = workload["batch"], workload["heads"], workload["head_dim"], synthetic.seq_len(workload)
    if args.heads:
        H = args.heads
    f_dense = 3.5 * 4.0 * B * H * float(S) * S * D / 2            # forward 1 + backward 2.5, causal half
    cfg_json = {"workload": workload["name"], "B": B, "heads": H, "head_dim": D, "seq_len": S, "grid": list(workload["grid"]),
                "causal": True, "mask": "random levels {0,1,2,4,8} p=(.2,.3,.2,.15,.15), column 0 at level 1",
                "block": 128, "parallelism": f"(batch, head) pairs/{world}", "l2": "inputs (q,k,v,dO) larger than L2"}
    if args.impl == "reference":
        if rank != 0:
            return
        tf, sec, sample = oracle_legacy_sample_time(workload, args.steps, args.warmup)
        print(json.dumps({
            "impl": "reference", "metric": "psa_attn_dense_equiv_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg_json,
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    import psa_b200
    from psa_b200 import ops, _lib
    launches = LaunchCounter(_lib.lib)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        assert (B * H) % world == 0, "(batch, head) pairs must divide by the number of GPUs"
    per = B * H // world
    mine = range(rank * per, (rank + 1) * per)
    dtype = torch.bfloat16
    wl = dict(workload); wl["heads"] = H
    parts = {0: [], 1: [], 2: []}
    for idx in mine:
        b, h = idx // H, idx % H
        for i, x in enumerate(synthetic.make_qkv(wl, 1000 + 7919 * b, dtype, dev, head_range=(h, h + 1))):
            parts[i].append(x)
    q, k, v = (torch.cat(parts[i], dim=1).contiguous() for i in range(3))                  # [1, per, S, D]
    do = torch.randn(q.shape, device=dev, dtype=dtype, generator=torch.Generator(device=dev).manual_seed(5 + rank))
    mask_all = legacy_level_mask(77, B, H, S).view(1, B * H, -(-S // 128), -(-S // 128))
    mask = mask_all[:, rank * per:(rank + 1) * per].contiguous().to(dev)
    n = mask.shape[-1]
    dens = float(torch.where(mask > 0, 1.0 / mask.clamp(min=1).float(), torch.zeros((), device=dev)).sum() / (per * n * (n + 1) / 2))
    scale = D ** -0.5
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step(rec=None):
        a, b, c = ev(), ev(), ev()
        a.record()
        o, lse, pooled = ops.legacy_forward(q, k, v, mask, True, scale, need_lse=True)
        b.record()
        grads = ops.legacy_backward(q, k, v, mask, o, lse, do, True, scale, pooled)
        c.record()
        if rec is not None:
            rec.append((a, b, c))
        return o, grads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        o, grads = step()
    barrier()
    status = int(ops.status_word(dev).item())
    rec = []
    barrier()
    sampler.mark_begin()
    e0, e1 = ev(), ev()
    torch.cuda.profiler.start()
    e0.record()
    launches.on = True
    for _ in range(args.steps):
        step(rec)
    launches.on = False
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    fwd_ms = sum(a.elapsed_time(b) for a, b, _ in rec) / len(rec)
    bwd_ms = sum(b.elapsed_time(c) for _, b, c in rec) / len(rec)

    e2e = None
    if not args.no_e2e:
        host = [x.cpu().pin_memory() for x in (q, k, v, do)]
        staged = [torch.empty_like(x) for x in (q, k, v, do)]
        back = [torch.empty(q.shape, dtype=dtype).pin_memory() for _ in range(3)]

        def e2e_step():
            for d_, h_ in zip(staged, host):
                d_.copy_(h_, non_blocking=True)
            qq, kk, vv, dd = staged
            o_, lse_, pooled_ = ops.legacy_forward(qq, kk, vv, mask, True, scale, need_lse=True)
            g_ = ops.legacy_backward(qq, kk, vv, mask, o_, lse_, dd, True, scale, pooled_)
            for h_, d_ in zip(back, g_):
                h_.copy_(d_, non_blocking=True)
        for _ in range(2):
            e2e_step()
        barrier()
        a0, a1 = ev(), ev()
        a0.record()
        for _ in range(args.steps):
            e2e_step()
        a1.record()
        barrier()
        te = torch.tensor([a0.elapsed_time(a1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e2e = float(te.item()) / args.steps
        nb = q.numel() * 2
        e2e = {"value": f_dense / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": 4 * nb * world, "d2h_bytes_per_step": 3 * nb * world}
    if world > 1 and rank != 0:
        dist.destroy_process_group()
        return
    peaks = load_peaks()
    peak_tf = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]
    f_surv_fwd = 4.0 * per * float(S) * S * D / 2 * dens            # surviving forward work of this rank
    bwd_tf = 2.5 * f_surv_fwd / (bwd_ms * 1e-3) / 1e12
    line = {
        "metric": "psa_attn_dense_equiv_tflops", "value": f_dense / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg_json,
        "stage_ms": {"forward": fwd_ms, "backward": bwd_ms}, "density": dens, "kernel_status": status,
        "gpu_launches": launches.count,
        "surviving_tflops_forward": f_surv_fwd / (fwd_ms * 1e-3) / 1e12,
        # the backward (dQ kernel + dK/dV kernel + small ones): 2.5x the surviving forward work; what the kernels execute on
        # top of that (both kernels recompute S and dP; level groups of the dK/dV kernel carry unselected key blocks) is
        # not counted
        "roofline": {"bound": "tensor", "kernel": "bwd_dq_tc_kernel + bwd_dkdv_tc_kernel", "achieved": bwd_tf, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": bwd_tf / peak_tf, "traffic": None,
                     "peak_source": f"{peaks['source']} (sustained bf16: kernels timed inside a long step)"},
        "clocks": clocks, "e2e": e2e}
    if not args.no_cpu_baseline and world == 1:
        tf, sec, sample = oracle_legacy_sample_time(workload, 1, 0)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": sample, "seconds": sec}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_preset_layer(args, workload, synthetic):
    """--workload wan2.1-1.3b-default-preset: one call of the plug-and-play module (PyramidSparseAttention) configured by
    the pipeline's default preset of attention_config.yaml - old mask format, block 128, cumulative-mass thresholds,
    similarity cap, Gilbert token order - on the Wan2.1-1.3B attention shape (single GPU).  Reports the layer with the
    reordering folded into the kernels and, beside it, with the reference's four reordering copies."""
    import psa_b200
    from psa_b200 import ops, _lib
    from psa_b200.presets import WanAttentionConfigLoader
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    assert int(os.environ.get("WORLD_SIZE", "1")) == 1, "this workload runs on one GPU"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    launches = LaunchCounter(_lib.lib)
    H, D, S = workload["heads"], workload["head_dim"], synthetic.seq_len(workload)
    info = WanAttentionConfigLoader().get_attention_config(workload["model"], None, list(workload["video_shape"]))
    params = dict(info["params"]); params["warmup_steps"] = 0; params["verbose"] = False
    cfg = AttentionConfig(**params)
    module = PyramidSparseAttention(cfg, inference_num=50, layer_num=30, model_type=workload["model"])
    q, k, v = synthetic.make_qkv(workload, 1000, torch.bfloat16, dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    with torch.no_grad():
        assert module._rows_in_place_old_format(q, k)
        sampler = ClockSampler(0)
        sampler.start()
        for _ in range(args.warmup):
            module(q, k, v, 0)
        torch.cuda.synchronize()
        sampler.mark_begin()
        launches.on = True
        ms = timed(lambda: module(q, k, v, 0), args.steps, 0)
        launches.on = False
        sampler.mark_end()
        clocks = sampler.stop()
        dens = float(module.logger.records[-1]["density"].mean().item())
        module.logger.records.clear()
        folded = PyramidSparseAttention._rows_in_place_old_format
        PyramidSparseAttention._rows_in_place_old_format = lambda self, q_, k_: False      # the copy route, for comparison
        ms_copies = timed(lambda: module(q, k, v, 0), args.steps, args.warmup)
        PyramidSparseAttention._rows_in_place_old_format = folded
    ops.check_status(dev)
    f_dense = 4.0 * H * float(S) * S * D
    print(json.dumps({
        "metric": "psa_attn_dense_equiv_tflops", "value": f_dense / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload["name"], "B": 1, "heads": H, "head_dim": D, "seq_len": S, "grid": list(workload["grid"]),
                   "preset": info["name"], "attn_impl": cfg.attn_impl, "block": [cfg.block_m, cfg.block_n, cfg.tile_n],
                   "mask_mode": cfg.mask_mode, "use_sim_mask": cfg.use_sim_mask, "rearrange": cfg.rearrange_method,
                   "l2": "inputs (q,k,v) larger than L2"},
        "ms_per_layer": ms, "ms_per_layer_with_reordering_copies": ms_copies, "density": dens, "gpu_launches": launches.count,
        "clocks": clocks}))


def run_causal_prefill(args, workload, synthetic):
    """--workload qwen2.5-vl-causal-layer: the causal (vision-language prefill) call site on one GPU - antidiagonal
    block-importance estimate, causal level mask, similarity cap, legacy causal forward - through the module that mirrors
    PyramidAdaptiveBlockSparseAttnTrain, with the stages timed one by one as well."""
    import psa_b200
    from psa_b200 import ops, _lib
    from psa_b200.causal import AttentionConfig, PyramidAdaptiveBlockSparseAttnTrain, transfer_attn_to_mask, x_block_imp_estimate
    assert int(os.environ.get("WORLD_SIZE", "1")) == 1, "this workload runs on one GPU"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    launches = LaunchCounter(_lib.lib)
    H = args.heads or workload["heads"]
    D, S = workload["head_dim"], synthetic.seq_len(workload)
    wl = dict(workload); wl["heads"] = H
    q, k, v = synthetic.make_qkv(wl, 1000, torch.bfloat16, dev)
    cfg = AttentionConfig(text_length=0)
    module = PyramidAdaptiveBlockSparseAttnTrain(cfg, layer_idx=0)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, steps):
        a, b = ev(), ev()
        a.record()
        for _ in range(steps):
            r = fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps, r

    with torch.no_grad():
        for _ in range(args.warmup):
            module(q, k, v)
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        sampler.mark_begin()
        torch.cuda.profiler.start()
        launches.on = True
        ms, _ = timed(lambda: module(q, k, v), args.steps)
        launches.on = False
        torch.cuda.profiler.stop()
        sampler.mark_end()
        clocks = sampler.stop()
        est_kw = dict(block_size=cfg.query_block, stride=cfg.xattn_stride, chunk_size=cfg.xattn_chunk_size, causal=True)
        ms_est, est = timed(lambda: x_block_imp_estimate(q, k, **est_kw), args.steps)
        ms_mask, mask = timed(lambda: transfer_attn_to_mask(est, cfg.mask_ratios, 0, cfg.mask_mode, block_size=cfg.query_block,
                                                            causal=True), args.steps)
    ops.check_status(dev)
    n = S // cfg.xattn_stride
    f_est = 2.0 * H * n * n * cfg.xattn_stride * D * 0.5 * (1.0 + 128.0 / n)      # lower triangle of 128x128 tiles
    f_dense = 4.0 * H * float(S) * S * D * 0.5
    peaks = load_peaks()
    print(json.dumps({
        "metric": "psa_attn_dense_equiv_tflops", "value": f_dense / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload["name"] + (f"-{H}heads" if args.heads else ""), "B": 1, "heads": H, "head_dim": D,
                   "seq_len": S, "block": 128, "stride": cfg.xattn_stride, "chunk": cfg.xattn_chunk_size, "mask_mode": cfg.mask_mode,
                   "causal": True, "dense_equiv": "causal triangle: 2*H*S^2*D", "l2": "inputs (q,k,v) larger than L2"},
        "ms_per_layer": ms, "stage_ms": {"estimate": ms_est, "level_mask": ms_mask},
        "estimate_gemm_tflops": f_est / (ms_est * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "kernel": "antidiag_logits_tc_kernel + antidiag_combine_kernel (the estimate stage)",
                     "achieved": f_est / (ms_est * 1e-3) / 1e12, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": f_est / (ms_est * 1e-3) / 1e12 / peaks["bf16_tflops"], "traffic": None,
                     "peak_source": peaks["source"] + " (burst bf16: a sub-millisecond stage)"},
        "gpu_launches": launches.count, "clocks": clocks}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wan2.1-14b-attn-layer")
    ap.add_argument("--sparsity", default="90", choices=["90", "85"])
    ap.add_argument("--chunks", type=int, default=5, help="head chunks per rank for exchange/compute overlap (N>1)")
    ap.add_argument("--pull-blocks", type=int, default=48,
                    help="grid cap of the full-row push that runs under the score kernels")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "p2p-push", "p2p-pull", "nccl"],
                    help="N>1: our kernels over peer memory - sampled rows pushed first, full rows under the scores (p2p), all "
                         "rows pushed before the layer (p2p-push) or pulled by the head owners (p2p-pull), "
                         "output rows stored into the token owners' buffers - or NCCL all-to-all (nccl)")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (smaller captures for profilers)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    synthetic = load_synthetic()
    workload = dict(synthetic.WORKLOADS[args.workload])
    if workload["name"] == "causal-legacy-fwd-bwd":
        return run_causal_training(args, workload, synthetic)
    if workload["name"] == "wan2.1-1.3b-default-preset":
        return run_preset_layer(args, workload, synthetic)
    if workload["name"] == "qwen2.5-vl-causal-layer":
        return run_causal_prefill(args, workload, synthetic)
    if args.heads:
        workload["heads"] = args.heads
        workload["name"] += f"-{args.heads}heads"
    ratios = RATIOS_90 if args.sparsity == "90" else DEFAULT_RATIOS
    H, D, S = workload["heads"], workload["head_dim"], synthetic.seq_len(workload)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    f_dense = 4.0 * H * float(S) * S * D
    cfg_json = {"workload": workload["name"], "B": 1, "heads": H, "head_dim": D, "seq_len": S, "grid": list(workload["grid"]),
                "text_tokens": workload["text"], "block_m": BLOCK_M, "block_n": BLOCK_N, "tile_n": TILE_N,
                "mask_mode": "topk", "mask_ratios": {str(k): list(v) for k, v in ratios.items()},
                "parallelism": f"heads/{max(world, 1)}" + ("+all_to_all" if world > 1 else ""),
                "l2": "inputs (q,k,v) larger than L2"}

    # ------------------------------------------------------------------ reference arm: the CPU restatement
    if args.impl == "reference":
        if rank != 0:
            return
        tf, sec, sample = oracle_sample_time(workload, ratios, args.steps, args.warmup)
        print(json.dumps({
            "impl": "reference", "metric": "psa_attn_dense_equiv_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg_json,
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ------------------------------------------------------------------ our arm
    import torch.distributed as dist
    import psa_b200
    from psa_b200 import ops, _lib
    launches = LaunchCounter(_lib.lib)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        assert S % world == 0, "tokens must divide by the number of GPUs"
    from psa_b200.parallel import GridShard, HeadShard, PeerExchange
    # heads that do not divide over the ranks (12 heads on 8 GPUs): head groups x query-block ranges, NCCL reshuffle
    grid = GridShard(world, rank, H, S, D, BLOCK_M) if (world > 1 and H % world != 0) else None
    if grid is not None:
        args.exchange = "nccl"
    hp = grid.heads_per_rank if grid is not None else H // world
    h0 = grid.head_range()[0] if grid is not None else rank * hp
    q_rows = grid.query_range() if grid is not None else (0, S)
    dtype = torch.bfloat16
    cfg = psa_b200.PSAConfig(block_m=BLOCK_M, block_n=BLOCK_N, tile_n=TILE_N, mask_ratios=ratios, mask_mode="topk")

    if world == 1:
        q, k, v = synthetic.make_qkv(workload, 1000, dtype, dev)
        seq_shard = None
    else:
        # what a sequence-parallel DiT holds: this rank's tokens, all heads -> [3, S/N, H, D]
        sl = S // world
        qs, ks, vs = synthetic.make_qkv(workload, 1000, dtype, dev, token_range=(rank * sl, (rank + 1) * sl))
        seq_shard = torch.stack([qs[0], ks[0], vs[0]]).permute(0, 2, 1, 3).contiguous()       # [3, S/N, H, D]
        del qs, ks, vs
        q = k = v = None

    fence_buf = None

    def fence():
        """Cross-rank ordering point on the current stream (a one-word all-reduce: unlike dist.barrier() it does not make
        the host wait for the device)."""
        nonlocal fence_buf
        if fence_buf is None:
            fence_buf = torch.zeros(1, device=dev)
        dist.all_reduce(fence_buf)

    def draw_indices_all():
        torch.manual_seed(2000)                      # same draw on every rank
        return (ops.draw_sample_indices(1, H, BLOCK_M, BLOCK_M // 4, dev), ops.draw_sample_indices(1, H, BLOCK_N, BLOCK_N // 4, dev))

    def draw_indices():
        torch.manual_seed(2000)                      # same draw on every rank, sliced by head
        iq = ops.draw_sample_indices(1, H, BLOCK_M, BLOCK_M // 4, dev)[:, h0:h0 + hp]
        ik = ops.draw_sample_indices(1, H, BLOCK_N, BLOCK_N // 4, dev)[:, h0:h0 + hp]
        return iq.contiguous(), ik.contiguous()

    shard = HeadShard(world, rank, H, S, D) if grid is None else None
    peer = None
    if world > 1 and args.exchange != "nccl":
        peer = PeerExchange(H, S, D, dtype, dev)
        if args.exchange == "p2p":
            peer.enable_sample_push(BLOCK_M, BLOCK_N)
        peer.q.copy_(seq_shard[0]); peer.k.copy_(seq_shard[1]); peer.v.copy_(seq_shard[2])
        torch.cuda.synchronize()
        dist.barrier()

    ev = lambda: torch.cuda.Event(enable_timing=True)
    stage_names = ["a2a_in", "sample", "pyramid", "scores", "assign", "forward", "a2a_out"]

    comm_stream = torch.cuda.Stream(device=dev, priority=-1) if world > 1 else None
    chunk_list = shard.chunks(args.chunks) if (world > 1 and grid is None) else [(0, hp)]

    def timed(name, fn, rec, stream=None):
        """Run fn; when rec is a list, bracket it with CUDA events on the stream its kernels are launched on."""
        if rec is None:
            return fn()
        st = stream if stream is not None else torch.cuda.current_stream(dev)
        a, b = ev(), ev()
        a.record(st)
        r = fn()
        b.record(st)
        rec.append((name, a, b))
        return r

    def layer_on(qq, kk, vv, iq, ik, rec):
        build = ops.pyramid_kv_images if ops.images_supported(kk, BLOCK_M, BLOCK_N, TILE_N) else ops.pyramid_kv
        pyr = timed("pyramid", lambda: build(kk, vv, BLOCK_N), rec)
        po = timed("scores", lambda: ops.block_scores(qq, kk, iq, ik, BLOCK_M, BLOCK_N), rec)
        mask = timed("assign", lambda: ops.assign_levels(po, ratios, "topk_newtype", BLOCK_N, TILE_N), rec)
        out = timed("forward", lambda: ops.psa_forward(qq, kk, vv, mask, BLOCK_M, BLOCK_N, TILE_N, pyramid=pyr), rec)
        return out, mask

    def layer_step(rec=None):
        """One PSA layer.  N = 1: inputs are already [1, H, S, D].  N > 1: the rank's heads are processed in chunks; the
        all-to-all of chunk c+1 (and the return of chunk c-1) runs on a second stream under the kernels of chunk c."""
        if peer is not None:
            return layer_step_p2p(rec, torch.cuda.current_stream(dev))
        iq, ik = timed("sample", draw_indices, rec)
        if world == 1:
            out, mask = layer_on(q, k, v, iq, ik, rec)
            return out, mask, out
        if grid is not None:
            qp, kk, vv = timed("a2a_in", lambda: grid.to_grid(seq_shard), rec)
            out, mask = layer_on(qp.unsqueeze(0), kk.unsqueeze(0), vv.unsqueeze(0), iq, ik, rec)
            out_final = timed("a2a_out", lambda: grid.to_seq(out[0]), rec)
            return out_final, mask, out
        cur = torch.cuda.current_stream(dev)
        out_final = torch.empty((H, S // world, D), dtype=dtype, device=dev)
        comm_stream.wait_stream(cur)
        arrived = []

        def fetch(ci):
            with torch.cuda.stream(comm_stream):
                x = timed("a2a_in", lambda: shard.to_head_sharded_chunk(seq_shard, *chunk_list[ci]), rec, comm_stream)
                e = ev(); e.record(comm_stream)
                arrived.append((x, e))
        fetch(0)
        mask = out = None
        for ci, (first, count) in enumerate(chunk_list):
            if ci + 1 < len(chunk_list):
                fetch(ci + 1)                                  # prefetch the next chunk's heads under this chunk's kernels
            x, e_in = arrived[ci]
            cur.wait_event(e_in)
            out, mask = layer_on(x[0].unsqueeze(0), x[1].unsqueeze(0), x[2].unsqueeze(0),
                                 iq[:, first:first + count].contiguous(), ik[:, first:first + count].contiguous(), rec)
            x.record_stream(cur)
            e_done = ev(); e_done.record(cur)
            with torch.cuda.stream(comm_stream):              # send this chunk's output back
                comm_stream.wait_event(e_done)
                o = out[0]
                timed("a2a_out", lambda: shard.to_seq_sharded_chunk(o, first, out_final), rec, comm_stream)
                o.record_stream(comm_stream)
        cur.wait_stream(comm_stream)
        return out_final, mask, out

    pull_buf = None
    step_no = 0
    draw_stream = torch.cuda.Stream(device=dev) if world > 1 else None
    pending_draw = None

    def launch_draw():
        with torch.cuda.stream(draw_stream):
            idx = draw_indices_all()
            e = ev(); e.record(draw_stream)
        return idx, e

    def prefetched_draw(cur):
        nonlocal pending_draw
        if pending_draw is None:
            pending_draw = launch_draw()
        idx, e = pending_draw
        cur.wait_event(e)
        for t_ in idx:
            t_.record_stream(cur)
        pending_draw = launch_draw()
        return idx

    def layer_step_p2p(rec, cur, v_ready=None):
        """N > 1 without a collective: q/k/v rows travel by our own copy kernel over peer memory (pushed by the token owners,
        or pulled by the head owners), the forward stores its output rows into the token owners' buffers, and the only
        cross-rank synchronisation is one barrier per step."""
        nonlocal pull_buf, step_no
        step_no += 1
        par = step_no & 1
        if args.exchange == "p2p":
            # Sender-driven and pipelined: (1) the sampled rows (a quarter of q and k) go first; (2) one barrier; (3) the
            # block scores and the level assignment run from them while, on a second stream, every rank stores its full
            # rows into the owners' receive buffers (alternating between steps) and a second barrier follows; (4) images
            # and forward wait for that.
            # the sample offsets do not depend on the data: the draw of the NEXT step runs on a side stream under this step
            # (same generator consumption, one draw per step), this step waits only for the one made during the previous step
            iq_all, ik_all = timed("sample", lambda: prefetched_draw(cur), rec)
            timed("a2a_in", lambda: peer.push_samples(par, iq_all, ik_all), rec)
            fence()
            comm_stream.wait_stream(cur)
            with torch.cuda.stream(comm_stream):
                if v_ready is not None:
                    comm_stream.wait_event(v_ready)          # end-to-end run: v is still on its way from the host
                x = timed("a2a_in", lambda: peer.push(par, max_blocks=args.pull_blocks), rec, comm_stream)
                fence()
                e_side = ev(); e_side.record(comm_stream)
            po = timed("scores", lambda: peer.scores_from_samples(par), rec)
            mask = timed("assign", lambda: ops.assign_levels(po, ratios, "topk_newtype", BLOCK_N, TILE_N), rec)
            cur.wait_event(e_side)
            qq, kk, vv = x[0].unsqueeze(0), x[1].unsqueeze(0), x[2].unsqueeze(0)
        else:
            iq, ik = timed("sample", draw_indices, rec)            # data-independent: before the exchange
            if v_ready is not None:
                cur.wait_event(v_ready)
            if args.exchange == "p2p-push":
                x = timed("a2a_in", lambda: peer.push(par), rec)
                fence()
            else:
                fence()                                            # inputs of all ranks are in their exchange buffers
                if pull_buf is None:
                    pull_buf = torch.empty((3, hp, S, D), dtype=dtype, device=dev)
                x = timed("a2a_in", lambda: peer.pull(out=pull_buf), rec)
            qq, kk, vv = x[0].unsqueeze(0), x[1].unsqueeze(0), x[2].unsqueeze(0)
            po = timed("scores", lambda: ops.block_scores(qq, kk, iq, ik, BLOCK_M, BLOCK_N), rec)
            mask = timed("assign", lambda: ops.assign_levels(po, ratios, "topk_newtype", BLOCK_N, TILE_N), rec)
        pyr = timed("pyramid", lambda: ops.pyramid_kv_images(kk, vv, BLOCK_N), rec)
        status = timed("forward", lambda: peer.forward_scatter(qq, pyr, mask, BLOCK_M, BLOCK_N, TILE_N), rec)
        holder = torch.empty(0, device=dev)
        holder._psa_status = status
        return peer.o, mask, holder

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        out_final, mask, out = layer_step()
    barrier()
    status = int(out._psa_status.item())
    dens = float(ops.density(mask, True).mean().item())

    records = []
    barrier()
    sampler.mark_begin()
    e0, e1 = ev(), ev()
    torch.cuda.profiler.start()          # lets `ncu --profile-from-start off` see the timed region only
    e0.record()
    launches.on = True
    for _ in range(args.steps):
        out_final, mask, out = layer_step(records)
    launches.on = False
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    stage_ms = {n: 0.0 for n in stage_names}        # per step, summed over the chunks of this rank; overlapped stages add up to more than the step
    for name, a, b in records:
        stage_ms[name] += a.elapsed_time(b) / args.steps

    # ------------------------------------------------------------------ N > 1: one head of this rank against one GPU
    parity = None
    if world > 1:
        # outside the timed region: the rank recomputes its first head from the same seeded inputs on its own GPU with the
        # single-GPU calls, and compares with what the sharded step left for its tokens (same kernels, same sample
        # offsets: the rows must be bit-identical)
        launches.on = False
        q1, k1, v1 = synthetic.make_qkv(workload, 1000, dtype, dev, head_range=(h0, h0 + 1))
        iq_all, ik_all = draw_indices_all()
        o1, _ = layer_on(q1, k1, v1, iq_all[:, h0:h0 + 1].contiguous(), ik_all[:, h0:h0 + 1].contiguous(), None)
        sl = S // world
        mine = o1[0, 0, rank * sl:(rank + 1) * sl]
        got = peer.o[:, h0] if peer is not None else out_final[h0]
        diff = (got.float() - mine.float()).abs()
        worst = torch.tensor([float(diff.max()), float((diff != 0).sum())], device=dev, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        parity = {"what": "first head of every rank: sharded step vs single-GPU calls on the same inputs, this rank's tokens",
                  "max_abs_diff": float(worst[0].item()), "rows_differing_max_over_ranks": int(worst[1].item()),
                  "bit_identical": bool(worst[0].item() == 0.0)}
        del q1, k1, v1, o1

    # ------------------------------------------------------------------ end to end: host buffers in, O back out
    e2e = None
    if not args.no_e2e:
        if world == 1:
            hq, hk, hv = (x.cpu().pin_memory() for x in (q, k, v))
        else:
            hx = seq_shard.cpu().pin_memory()
        module = psa_b200.PSAAttention(cfg)
        h_out = None
        copy_stream = torch.cuda.Stream(device=dev) if world > 1 else None

        def e2e_step():
            nonlocal h_out
            cur = torch.cuda.current_stream(dev)
            if peer is not None:
                # q and k first (the sampled rows leave as soon as they are here); v follows on a side stream under the
                # sample push and the scores.  No host-side wait anywhere: the ranks are ordered by stream-ordered fences.
                peer.q.copy_(hx[0], non_blocking=True); peer.k.copy_(hx[1], non_blocking=True)
                copy_stream.wait_stream(cur)
                with torch.cuda.stream(copy_stream):
                    peer.v.copy_(hx[2], non_blocking=True)
                    v_here = ev(); v_here.record(copy_stream)
                layer_step_p2p(None, cur, v_ready=v_here)
                fence()                           # every rank's forward has stored its rows: this rank's o is complete
                if h_out is None:
                    h_out = torch.empty(peer.o.shape, dtype=peer.o.dtype).pin_memory()
                h_out.copy_(peer.o, non_blocking=True)
                return
            if world == 1:
                # the library's host-buffer call: head chunks, copies in and out overlapped with the compute
                iq, ik = draw_indices()
                h_out = psa_b200.psa_attention_host(hq, hk, hv, cfg, out=h_out, device=dev, idx_q=iq, idx_k=ik)
                return
            iq, ik = draw_indices()
            xd = hx.to(dev, non_blocking=True)
            if grid is not None:
                qp, kk, vv = grid.to_grid(xd)
                o = grid.to_seq(module(qp.unsqueeze(0), kk.unsqueeze(0), vv.unsqueeze(0), idx_q=iq, idx_k=ik)[0])
            else:
                x = shard.to_head_sharded(xd)
                o = shard.to_seq_sharded(module(x[0].unsqueeze(0), x[1].unsqueeze(0), x[2].unsqueeze(0), idx_q=iq, idx_k=ik)[0])
            if h_out is None:
                h_out = torch.empty(o.shape, dtype=o.dtype).pin_memory()
            h_out.copy_(o, non_blocking=True)
        for _ in range(2):
            e2e_step()
        barrier()
        a0, a1 = ev(), ev()
        a0.record()
        for _ in range(args.steps):
            e2e_step()
        a1.record()
        barrier()
        te = torch.tensor([a0.elapsed_time(a1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e2e = float(te.item()) / args.steps
        esz = 2
        per_rank_in = 3 * (S // world) * H * D * esz
        per_rank_out = (S // world) * H * D * esz
        e2e = {"value": f_dense / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": per_rank_in * world, "d2h_bytes_per_step": per_rank_out * world,
               # what the host link of one rank sustained if the whole step were copies (a lower bound on its speed)
               "per_rank_host_link_gbs_lower_bound": (per_rank_in + per_rank_out) / (ms_e2e * 1e-3) / 1e9}

    if peer is not None:
        barrier()
        peer.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    # dominant kernel: the tcgen05 forward.  Algorithmic FLOPs per launch = 4*hp*S^2*D*density (surviving blocks).
    f_surv_launch = 4.0 * hp * float(q_rows[1] - q_rows[0]) * S * D * dens
    fwd_tflops = f_surv_launch / (stage_ms["forward"] * 1e-3) / 1e12
    peak_tf = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]
    n_elem = hp * S * D
    per_ht = FWD_TRAFFIC_PER_HEAD_TOKEN.get(synthetic.WORKLOADS[args.workload]["name"])
    traffic = per_ht[0] * hp * S if per_ht else None
    traffic_source = (f"{per_ht[1]}: ncu dram bytes of one launch at this shape with fewer heads, scaled by heads"
                      if per_ht else "no capture at this shape")
    line = {
        "metric": "psa_attn_dense_equiv_tflops", "value": f_dense / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg_json,
        "ms_per_layer": ms_step, "stage_ms": stage_ms, "density": dens, "sparsity": 1.0 - dens,
        "surviving_tflops_forward": fwd_tflops, "kernel_status": status,
        # this library's kernels launched by this rank inside the timed region, counted at the C-ABI boundary
        "gpu_launches": launches.count,
        "exchange": (args.exchange if world > 1 else None),
        "roofline": {"bound": "tensor", "kernel": "psa_fwd_tc_kernel", "achieved": fwd_tflops, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": fwd_tflops / peak_tf,
                     "traffic": traffic, "traffic_unit": "bytes per launch", "traffic_source": traffic_source,
                     "peak_source": f"{peaks['source']} (sustained bf16: kernel timed inside a long step)",
                     # tile-image pyramid: read K,V once (2 N e), write levels 1,2,4,8 of both (3.75 N e)
                     "pyramid_gbs": 5.75 * n_elem * 2 / (stage_ms["pyramid"] * 1e-3) / 1e9,
                     "pyramid_frac_of_hbm": 5.75 * n_elem * 2 / (stage_ms["pyramid"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     # the same on the algorithmic bytes of a pyramid (levels 2/4/8 only: 3.75 N e); the level-1 image
                     # is this library's own extra write
                     "pyramid_frac_algorithmic": 3.75 * n_elem * 2 / (stage_ms["pyramid"] * 1e-3) / 1e9 / peaks["hbm_gbs"]},
        "clocks": clocks, "e2e": e2e,
    }
    if parity is not None:
        line["parity_check"] = parity
    if grid is not None:
        line["config"]["parallelism"] = f"{grid.groups} head groups x {grid.parts} query-block ranges + all_to_all"
    if not args.no_cpu_baseline and world == 1:
        tf, sec, sample = oracle_sample_time(workload, ratios, 1, 1)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": sample, "seconds": sec}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
