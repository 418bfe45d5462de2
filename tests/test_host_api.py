"""CPU: host-side logic that needs no GPU - Gilbert order, presets, installer wiring, interval arithmetic."""
import numpy as np
import pytest
import torch

import cases as C
from oracle import psa_oracle as O


@pytest.mark.parametrize("shape", C.GILBERT_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gilbert_order_matches_reference_curve(golden, shape):
    from psa_b200.rearrange import gilbert_order
    w, h, d = shape
    order = gilbert_order(w, h, d)
    assert sorted(order.tolist()) == list(range(w * h * d))
    assert C.order_checksum(order) == int(golden[f"gilbert_sum_{w}x{h}x{d}"][0])
    key = f"gilbert_{w}x{h}x{d}"
    if key in golden.files:
        assert np.array_equal(order, golden[key])


def test_gilbert_rearranger_round_trip_with_text():
    from psa_b200.rearrange import GilbertRearranger
    r = GilbertRearranger(6, 4, 3, text_length=5)
    x = torch.arange(2 * (5 + 72) * 3, dtype=torch.float32).view(1, 2, 77, 3)
    q, k, v = r.rearrange(x, x + 1, x + 2)
    assert torch.equal(q[..., -5:, :], x[..., :5, :])                 # text moved to the end
    assert torch.equal(r.reversed_rearrange(q), x)
    assert torch.equal(r.reversed_rearrange(v), x + 2)
    # the row table the kernels read: gathering through it is rearrange_single, scattering through it is the inverse
    rows = r.source_rows("cpu").long()
    assert torch.equal(x.index_select(-2, rows), q)
    back = torch.empty_like(q)
    back[..., rows, :] = q
    assert torch.equal(back, x)
    r0 = GilbertRearranger(6, 4, 3, text_length=0)
    y = x[..., :72, :]
    assert torch.equal(r0.reversed_rearrange(r0.rearrange_single(y)), y)


def test_preset_loader_values_and_errors():
    from psa_b200.presets import WanAttentionConfigLoader
    L = WanAttentionConfigLoader()
    assert set(L.list_presets("Wan2.1_1.3b")) == {"baseline", "psa_balanced", "psa_topk"}
    info = L.get_attention_config("Wan2.1_1.3b", "psa_topk", [832, 480, 81])
    p = info["params"]
    assert (p["width"], p["height"], p["depth"]) == (52, 30, 21)
    assert (p["block_m"], p["block_n"], p["tile_n"]) == (128, 32, 32)
    assert p["mask_ratios"] == C.RATIOS_90 and p["mask_mode"] == "topk" and p["warmup_steps"] == 15
    d = L.get_attention_config("Wan2.1_1.3b", None, [832, 480, 81])["params"]       # default preset
    assert d["attn_impl"] == "old_mask_type" and d["use_sim_mask"] and d["sim_2x_threshold"] == 0.7
    c = L.get_attention_config("CogVideo_5b", "psa_balanced", [720, 480, 49])["params"]
    assert c["text_length"] == 226 and not c["use_rearrange"] and (c["width"], c["height"], c["depth"]) == (45, 30, 13)
    assert L.get_attention_config("Wan2.1_14b", "baseline", [1280, 720, 81])["type"] == "dense"
    for bad in (lambda: L.get_attention_config("Wan2.1_1.3b_4steps", None, [1, 1, 1]),
                lambda: L.get_attention_config("Wan2.1_14b", "nope", [1, 1, 1]),
                lambda: L.get_attention_config("Wan2.1_14b", None, [1, 1])):
        with pytest.raises(ValueError):
            bad()


class _Attn:
    def __init__(self):
        self.processor = None
        self.inner_attention = None

    def set_processor(self, p):
        self.processor = p


class _Block:
    def __init__(self):
        self.attn1 = _Attn()


class _Transformer:
    def __init__(self, n):
        self.blocks = [_Block() for _ in range(n)]


class _Pipe:
    def __init__(self, n, two=False):
        self.transformer = _Transformer(n)
        self.transformer_2 = _Transformer(n) if two else None


def test_installer_shares_one_module_and_dense_preset_is_a_no_op():
    from psa_b200.presets import set_adaptive_sparse_attention, reset_wan_attention_to_dense
    pipe = _Pipe(4, two=True)
    mod = set_adaptive_sparse_attention(pipe, "Wan2.2_A14B", inference_num=40, video_shape=[832, 480, 81])
    assert mod is not None and mod.layer_num == 4 and mod.inference_num == 40
    mods = {id(b.attn1.inner_attention) for t in (pipe.transformer, pipe.transformer_2) for b in t.blocks}
    assert mods == {id(mod)}
    assert [b.attn1.processor.layer_idx for b in pipe.transformer.blocks] == [0, 1, 2, 3]
    assert mod.config.block_n == 32 and mod.config.mask_mode == "thresholdbound" and mod.gilbert_rearranger is not None
    reset_wan_attention_to_dense(pipe)
    assert all(b.attn1.inner_attention is None for b in pipe.transformer.blocks)
    pipe2 = _Pipe(2)
    assert set_adaptive_sparse_attention(pipe2, "Wan2.1_14b", video_shape=[832, 480, 81], attention_preset="baseline") is None
    assert pipe2.transformer.blocks[0].attn1.processor is None
    with pytest.raises(ValueError):
        set_adaptive_sparse_attention(pipe2, "NotAModel", video_shape=[1, 1, 1])


def test_warmup_schedule_follows_the_reference_counter_rule():
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    cfg = AttentionConfig(use_rearrange=False, use_sim_mask=False, warmup_steps=2, enable_logging=False)
    wan = PyramidSparseAttention(cfg, inference_num=5, layer_num=3, model_type="wan")
    cog = PyramidSparseAttention(cfg, inference_num=5, layer_num=3, model_type="cogvideo")
    times_wan, times_cog = [], []
    for _ in range(40):
        times_wan.append(wan.get_current_time()); wan.sparsity_counter += 1
        times_cog.append(cog.get_current_time()); cog.sparsity_counter += 1
    assert times_wan[:13] == [0] * 6 + [1] * 6 + [2]          # two CFG passes per step: 2 * layer_num calls per step
    assert times_cog[:7] == [0] * 3 + [1] * 3 + [2]
    assert times_cog[15] == 0                                 # wraps after inference_num steps
    with pytest.raises(ValueError):
        AttentionConfig()                                      # default new_mask_type + use_sim_mask=True is rejected
    with pytest.raises(NotImplementedError):
        PyramidSparseAttention(AttentionConfig(use_sim_mask=False, rearrange_method="STA"))


def test_topk_intervals_host_arithmetic_equals_oracle():
    from psa_b200.ops import topk_intervals
    for nk in (1, 9, 37, 64, 139, 278, 512, 1182, 2363):
        for bn in (32, 64, 128):
            for ratios in (C.DEFAULT_RATIOS, C.RATIOS_90, C.RATIOS_DENSE, C.RATIOS_THR):
                for newtype in (True, False):
                    mine = [(l, s, e) for l, s, e in topk_intervals(nk, ratios, bn, 32, newtype) if newtype or s < e]
                    assert mine == O.topk_intervals(nk, ratios, bn, 32, newtype)


def test_sparsity_log_writes_jsonl(tmp_path):
    """The per-call records (densities as tensors, None for warm-up calls) become one JSON line each."""
    import json
    from psa_b200.pyramid_sparse_attention import SparsityLog
    log = SparsityLog()
    log.log_sparsity(layer_idx=0, density=None, sequence_length=640, batch_size=1, num_heads=2, is_warmup=True)
    log.log_sparsity(layer_idx=1, density=torch.tensor([[0.25, 0.75]]), sequence_length=640, batch_size=1, num_heads=2,
                     is_warmup=False)
    path = tmp_path / "logs" / "sparsity.jsonl"
    assert log.write_jsonl(str(path)) == 2
    lines = [json.loads(x) for x in path.read_text().splitlines()]
    assert lines[0]["is_warmup"] and lines[0]["per_head_density"] == [] and lines[0]["density"] == 1.0
    assert lines[1]["per_head_density"] == [0.25, 0.75] and lines[1]["density"] == 0.5 and lines[1]["sparsity"] == 0.5
    assert lines[1]["global_step"] == 1 and lines[1]["layer_idx"] == 1
