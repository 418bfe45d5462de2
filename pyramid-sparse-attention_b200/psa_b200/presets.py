"""attention_config.yaml presets and their installation into diffusers-style pipelines.

WanAttentionConfigLoader reads the same YAML schema and returns the same dictionaries as the reference loader
(modify_diffusers.py:39-178); set_adaptive_sparse_attention / reset_wan_attention_to_dense have the reference's
signatures (:551-678).  diffusers is not imported: the installer only needs objects that look like a pipeline
(``pipe.transformer.blocks[i].attn1`` with ``set_processor``), so it also works on stand-ins in tests.
"""
from __future__ import annotations

import math
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import yaml

from .pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention

SUPPORTED_MODELS = {
    "CogVideo": ["CogVideo_5b", "CogVideo_2b"],
    "Wan": ["Wan2.1_14b", "Wan2.1_1.3b", "Wan2.1_1.3b_4steps", "Wan2.2_A14B", "Wan2.2_5B"],
}
DEFAULT_CONFIG_PATH = Path(__file__).resolve().parent.parent / "configs" / "attention_config.yaml"


class WanAttentionConfigLoader:
    def __init__(self, config_path: Optional[str] = None):
        path = Path(config_path) if config_path is not None else DEFAULT_CONFIG_PATH
        if not path.exists():
            raise FileNotFoundError(f"Config file not found: {path}")
        with open(path, "r", encoding="utf-8") as f:
            self._config = yaml.safe_load(f) or {}

    def _model(self, model_name: str) -> Dict[str, Any]:
        cfg = self._config.get(model_name)
        if cfg is None:
            raise ValueError(f"Model '{model_name}' not found in config. Available models: {list(self._config.keys())}")
        return cfg

    def list_presets(self, model_name: str) -> List[str]:
        return list(self._model(model_name).get("attention_configs", {}).keys())

    def get_attention_config(self, model_name: str, preset_name: Optional[str],
                             video_shape: Union[List[int], Tuple[int, int, int]]) -> Dict[str, Any]:
        model_cfg = self._model(model_name)
        presets = model_cfg.get("attention_configs", {})
        if not presets:
            raise ValueError(f"No attention presets defined for model '{model_name}'.")
        if preset_name is None:
            preset_name = model_cfg.get("default_attention")
        if preset_name is None:
            raise ValueError(f"Preset name must be provided for model '{model_name}'. Available presets: {list(presets.keys())}")
        if preset_name not in presets:
            raise ValueError(f"Preset '{preset_name}' not found for model '{model_name}'. "
                             f"Available presets: {list(presets.keys())}")
        pc = presets[preset_name]
        ptype = pc.get("type", "psa").lower()
        if video_shape is None or len(video_shape) != 3:
            raise ValueError("video_shape must be a sequence of [width, height, depth].")
        vs = [int(x) for x in video_shape]
        if "video_scale" not in model_cfg:
            raise ValueError("Missing 'video_scale' configuration for model.")
        sc = model_cfg["video_scale"]
        dims = {"width": math.ceil(vs[0] / sc["width_divisor"]), "height": math.ceil(vs[1] / sc["height_divisor"]),
                "depth": math.ceil(vs[2] / sc["depth_divisor"])}
        info: Dict[str, Any] = {"name": preset_name, "type": ptype, "description": pc.get("description"), "video_dims": dims,
                                "original_video_shape": {"width": vs[0], "height": vs[1], "depth": vs[2]}}
        if ptype == "dense":
            return info
        if ptype != "psa":
            raise ValueError(f"Unsupported preset type '{ptype}' for model '{model_name}'.")
        blk = pc.get("block_size", {})
        tile = pc.get("tile_size")
        params: Dict[str, Any] = {
            **dims,
            "text_length": pc.get("text_length", model_cfg.get("text_length", 0)),
            "use_rearrange": pc.get("use_rearrange", True),
            "use_sim_mask": pc.get("use_sim_mask", True),
            "block_m": blk.get("m", 128), "block_n": blk.get("n", 128), "tile_n": blk.get("tile_n", 32),
            "mask_ratios": {int(k): tuple(v) for k, v in pc.get("mask_ratios", {}).items()},
            "mask_mode": pc.get("mask_mode", "thresholdbound"),
            "attn_impl": pc.get("attn_impl", "new_mask_type"),
            "warmup_steps": pc.get("warmup_steps", 0),
            "tile_size": tuple(tile) if tile is not None else None,
            "rearrange_method": pc.get("rearrange_method", "Gilbert"),
            "verbose": pc.get("verbose", False),
            "enable_logging": pc.get("enable_logging", True),
            "log_dir": pc.get("log_dir", "./psa_logs/"),
        }
        for key in ("sim_2x_threshold", "sim_4x_threshold", "sim_8x_threshold"):
            if key in pc:
                params[key] = pc[key]
        st = pc.get("sim_thresholds", {})
        if st:
            params.setdefault("sim_2x_threshold", st.get("x2"))
            params.setdefault("sim_4x_threshold", st.get("x4"))
            params.setdefault("sim_8x_threshold", st.get("x8"))
        info["params"] = params
        return info


class SparseAttnProcessor:
    """Attention processor for Wan / CogVideoX style blocks: projections, q/k norms and rotary embedding as the stock
    processor does, then ``attn.inner_attention(q, k, v, layer_idx)`` on [B, H, S, D] tensors, then the output
    projection (modify_diffusers.py:192-381).  ``text_first`` prepends encoder tokens (CogVideoX joint attention)."""

    def __init__(self, layer_idx: int, text_first: bool = False):
        self.layer_idx = layer_idx
        self.text_first = text_first

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, attention_mask=None, rotary_emb=None, **kw):
        text_len = 0
        if self.text_first and encoder_hidden_states is not None:
            text_len = encoder_hidden_states.shape[1]
            hidden_states = torch.cat([encoder_hidden_states, hidden_states], dim=1)
        q, k, v = attn.to_q(hidden_states), attn.to_k(hidden_states), attn.to_v(hidden_states)
        if getattr(attn, "norm_q", None) is not None:
            q = attn.norm_q(q)
        if getattr(attn, "norm_k", None) is not None:
            k = attn.norm_k(k)
        B, S, _ = q.shape
        H = attn.heads
        q, k, v = (x.view(B, S, H, -1).transpose(1, 2) for x in (q, k, v))
        if rotary_emb is not None:
            q, k = rotary_emb(q, k) if callable(rotary_emb) else (q, k)
        out = attn.inner_attention(q, k, v, self.layer_idx)
        out = out.transpose(1, 2).reshape(B, S, -1).to(hidden_states.dtype)
        out = attn.to_out[0](out)
        if len(attn.to_out) > 1:
            out = attn.to_out[1](out)
        if text_len:
            return out[:, text_len:], out[:, :text_len]
        return out


def _install(transformer, module: PyramidSparseAttention, text_first: bool) -> int:
    blocks = getattr(transformer, "blocks", None) or getattr(transformer, "transformer_blocks")
    for idx, block in enumerate(blocks):
        block.attn1.inner_attention = module
        block.attn1.set_processor(SparseAttnProcessor(idx, text_first=text_first))
    return len(blocks)


def set_adaptive_sparse_attention(pipe, model_name: str, inference_num: int = 50, video_shape=None,
                                  attention_type: str = "PSA", attention_preset: Optional[str] = None, verbose: bool = False,
                                  config_path: Optional[str] = None):
    """Resolve the preset for (model, video shape) and route every self-attention of the pipeline's transformer(s)
    through ONE shared PyramidSparseAttention instance.  Dense presets leave the pipeline untouched."""
    known = [m for ms in SUPPORTED_MODELS.values() for m in ms]
    if model_name not in known:
        raise ValueError(f"Unsupported model '{model_name}'. Supported: {known}")
    info = WanAttentionConfigLoader(config_path).get_attention_config(model_name, attention_preset, video_shape)
    if info["type"] == "dense":
        return None
    params = dict(info["params"])
    if not verbose:
        params["verbose"] = False
    cfg = AttentionConfig(**params)
    transformers = [t for t in (getattr(pipe, "transformer", None), getattr(pipe, "transformer_2", None)) if t is not None]
    first_blocks = getattr(transformers[0], "blocks", None) or getattr(transformers[0], "transformer_blocks")
    is_cog = model_name in SUPPORTED_MODELS["CogVideo"]
    model_type = "cogvideo" if is_cog else model_name.lower()
    module = PyramidSparseAttention(cfg, inference_num=inference_num, layer_num=len(first_blocks), model_type=model_type)
    for t in transformers:
        _install(t, module, text_first=is_cog)
    return module


def reset_wan_attention_to_dense(pipe, default_processor_factory=None):
    """Remove the sparse module again (modify_diffusers.py:649-678)."""
    for t in (getattr(pipe, "transformer", None), getattr(pipe, "transformer_2", None)):
        if t is None:
            continue
        for block in (getattr(t, "blocks", None) or getattr(t, "transformer_blocks")):
            if hasattr(block.attn1, "inner_attention"):
                block.attn1.inner_attention = None
            if default_processor_factory is not None:
                block.attn1.set_processor(default_processor_factory())
