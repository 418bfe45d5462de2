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


def rope_interleaved_pairs(x: torch.Tensor, freqs_cos: torch.Tensor, freqs_sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of the Wan transformer blocks: channels are (even, odd) pairs, the cosine table is read at its
    even entries and the sine table at its odd ones (modify_diffusers.py:260-271).  x: [B, S, H, D]; tables broadcast
    against it ([1, S, 1, D])."""
    even, odd = x[..., 0::2], x[..., 1::2]
    c, s = freqs_cos[..., 0::2], freqs_sin[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = even * c - odd * s
    out[..., 1::2] = even * s + odd * c
    return out.type_as(x)


def rope_real_pairs(x: torch.Tensor, image_rotary_emb) -> torch.Tensor:
    """Rotary embedding as the CogVideoX blocks apply it (diffusers' ``apply_rotary_emb`` with real tables, called at
    modify_diffusers.py:366-369): x [B, H, S, D], tables (cos, sin) of shape [S, D]; the pair (x0, x1) of neighbouring
    channels turns into (x0 cos - x1 sin, x1 cos + x0 sin), computed in fp32 and rounded once."""
    cos, sin = image_rotary_emb
    cos, sin = cos[None, None].to(x.device), sin[None, None].to(x.device)
    a, b = x.reshape(*x.shape[:-1], -1, 2).unbind(-1)
    turned = torch.stack([-b, a], dim=-1).flatten(3)
    return (x.float() * cos + turned.float() * sin).to(x.dtype)


_rotary_cache = {}


def _rotary_tables(kind: str, cos: torch.Tensor, sin: torch.Tensor, first: int):
    """ops.RotaryTables for the fused loads, built once per (cos, sin) pair - every layer of a step passes the same
    tables.  kind "wan": cos/sin broadcastable to [1, S, 1, D], cosine read at the even entries and sine at the odd
    ones (rope_interleaved_pairs); kind "real": cos/sin [S, D] (rope_real_pairs).  None if the tables carry a batch."""
    from . import ops
    key = (kind, cos.data_ptr(), sin.data_ptr(), tuple(cos.shape), cos.device, first, cos._version, sin._version)
    hit = _rotary_cache.get(key)
    if hit is not None:
        return hit
    if kind == "wan":
        D = cos.shape[-1]
        plain = cos.dim() == 2 or (cos.dim() == 4 and cos.shape[0] == 1 and cos.shape[2] == 1)
        if not plain or cos.shape != sin.shape:
            return None
        c2, s2 = cos.reshape(-1, D).float(), sin.reshape(-1, D).float()
        a = c2[:, 0::2].repeat_interleave(2, dim=1)
        b = s2[:, 1::2].repeat_interleave(2, dim=1)
    else:
        if cos.dim() != 2:
            return None
        a, b = cos.float(), sin.float()
    tables = ops.RotaryTables(a, b, first)
    if len(_rotary_cache) > 8:
        _rotary_cache.clear()
    _rotary_cache[key] = tables
    return tables


class SparseWanAttnProcessor:
    """Attention processor of the Wan 2.1 / 2.2 transformer blocks with the sparse module in place of the dense
    attention (modify_diffusers.py:192-315): separate or fused projections, q/k norms on the full hidden width,
    rotary tables given as a (cos, sin) tuple, the image-conditioning branch of the I2V models (dense attention over
    the added image keys, summed into the result), ``attn.inner_attention(q, k, v, layer_idx)`` on [B, H, S, D], then
    both output layers."""

    TEXT_CONTEXT = 512     # tokens of the text encoder; whatever precedes them in the context is image conditioning

    def __init__(self, idx: int):
        self.layer_idx = idx

    @staticmethod
    def _project(attn, hidden_states, context):
        if context is None:
            context = hidden_states
        if getattr(attn, "fused_projections", False):
            if getattr(attn, "cross_attention_dim_head", None) is None:
                return attn.to_qkv(hidden_states).chunk(3, dim=-1)
            k, v = attn.to_kv(context).chunk(2, dim=-1)
            return attn.to_q(hidden_states), k, v
        return attn.to_q(hidden_states), attn.to_k(context), attn.to_v(context)

    @staticmethod
    def _project_image(attn, image_context):
        if getattr(attn, "fused_projections", False):
            return attn.to_added_kv(image_context).chunk(2, dim=-1)
        return attn.add_k_proj(image_context), attn.add_v_proj(image_context)

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, attention_mask=None, rotary_emb=None,
                 numerical_timestep=None):
        image_context = None
        if getattr(attn, "add_k_proj", None) is not None:
            n_img = encoder_hidden_states.shape[1] - self.TEXT_CONTEXT
            image_context = encoder_hidden_states[:, :n_img]
            encoder_hidden_states = encoder_hidden_states[:, n_img:]
        q, k, v = self._project(attn, hidden_states, encoder_hidden_states)
        if getattr(attn, "norm_q", None) is not None:
            q = attn.norm_q(q)
        if getattr(attn, "norm_k", None) is not None:
            k = attn.norm_k(k)
        H = attn.heads
        q, k, v = (x.unflatten(2, (H, -1)) for x in (q, k, v))                  # [B, S, H, D]
        fused = None
        if rotary_emb is not None:
            # a module that rotates inside its kernels gets q and k as they are (self-attention: same length, same tables)
            if getattr(attn.inner_attention, "fuses_rotary", False) and q.is_cuda and q.shape[1] == k.shape[1]:
                fused = _rotary_tables("wan", rotary_emb[0], rotary_emb[1], 0)
            if fused is None:
                q = rope_interleaved_pairs(q, *rotary_emb)
                k = rope_interleaved_pairs(k, *rotary_emb)
        from_image = None
        if image_context is not None:
            k_img, v_img = self._project_image(attn, image_context)
            k_img = attn.norm_added_k(k_img)
            k_img, v_img = k_img.unflatten(2, (H, -1)), v_img.unflatten(2, (H, -1))
            from_image = torch.nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k_img.transpose(1, 2), v_img.transpose(1, 2)).transpose(1, 2).flatten(2, 3).type_as(q)
        if fused is not None:
            out = attn.inner_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), self.layer_idx, rotary=fused)
        else:
            out = attn.inner_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), self.layer_idx)
        out = out.transpose(1, 2).flatten(2, 3).type_as(q)
        if from_image is not None:
            out = out + from_image
        return attn.to_out[1](attn.to_out[0](out))


class SparseCogVideoXAttnProcessor:
    """Attention processor of the CogVideoX blocks (modify_diffusers.py:318-381): text and video tokens form one
    sequence (text first), q/k norms act per head (after the head split), the rotary tables arrive as
    ``image_rotary_emb`` and turn the video tokens only, and the result is split back into (video, text)."""

    def __init__(self, layer_idx: int):
        self.layer_idx = layer_idx

    def __call__(self, attn, hidden_states, encoder_hidden_states, attention_mask=None, image_rotary_emb=None):
        assert attention_mask is None, "Attention mask is not supported"
        n_text = encoder_hidden_states.size(1)
        x = torch.cat([encoder_hidden_states, hidden_states], dim=1)
        B = x.shape[0]
        H = attn.heads
        q, k, v = attn.to_q(x), attn.to_k(x), attn.to_v(x)
        D = k.shape[-1] // H
        q, k, v = (y.view(B, -1, H, D).transpose(1, 2) for y in (q, k, v))      # [B, H, S, D]
        if getattr(attn, "norm_q", None) is not None:
            q = attn.norm_q(q).to(dtype=v.dtype)
        if getattr(attn, "norm_k", None) is not None:
            k = attn.norm_k(k).to(dtype=v.dtype)
        fused = None
        if image_rotary_emb is not None:
            if (getattr(attn.inner_attention, "fuses_rotary", False) and q.is_cuda
                    and not getattr(attn, "is_cross_attention", False)):
                fused = _rotary_tables("real", image_rotary_emb[0], image_rotary_emb[1], n_text)
            if fused is None:
                q = torch.cat([q[:, :, :n_text], rope_real_pairs(q[:, :, n_text:], image_rotary_emb)], dim=2)
                if not getattr(attn, "is_cross_attention", False):
                    k = torch.cat([k[:, :, :n_text], rope_real_pairs(k[:, :, n_text:], image_rotary_emb)], dim=2)
        if fused is not None:
            out = attn.inner_attention(q, k, v, self.layer_idx, rotary=fused)
        else:
            out = attn.inner_attention(q, k, v, self.layer_idx)
        out = out.transpose(1, 2).reshape(B, -1, H * D)
        out = attn.to_out[1](attn.to_out[0](out))
        return out[:, n_text:], out[:, :n_text]


def _swap_processors(blocks, module: PyramidSparseAttention, make_processor, verbose: bool) -> None:
    for idx, block in enumerate(blocks):
        a = block.attn1
        a.verbose = verbose
        a.inner_attention = module
        previous = a.get_processor() if hasattr(a, "get_processor") else getattr(a, "processor", None)
        a.set_processor(make_processor(idx))
        if not hasattr(a, "origin_processor"):
            a.origin_processor = previous


def set_block_sparse_attn_wan(model, model_name: str, inference_num: int, attention_info: Dict[str, Any],
                              verbose: bool = False) -> PyramidSparseAttention:
    """One PyramidSparseAttention shared by every ``blocks[i].attn1`` of a Wan transformer
    (modify_diffusers.py:480-548).  The configuration banner of the reference is not printed."""
    cfg = AttentionConfig(**attention_info["params"])
    module = PyramidSparseAttention(config=cfg, inference_num=inference_num, layer_num=len(model.blocks),
                                    model_type=model_name)
    _swap_processors(model.blocks, module, SparseWanAttnProcessor, verbose)
    return module


def set_block_sparse_attn_cogvideox(model, model_name: str, inference_num: int, attention_info: Dict[str, Any],
                                    verbose: bool = False) -> PyramidSparseAttention:
    """The same for ``transformer_blocks[i].attn1`` of a CogVideoX transformer, with that model's defaults for the
    fields a preset may leave out (modify_diffusers.py:384-477)."""
    dims = attention_info.get("video_dims", {})
    p = attention_info.get("params", {})
    cfg = AttentionConfig(
        width=dims.get("width"), height=dims.get("height"), depth=dims.get("depth"),
        text_length=p.get("text_length", 226), use_rearrange=p.get("use_rearrange", True),
        block_m=p.get("block_m", 128), block_n=p.get("block_n", 128), tile_n=p.get("tile_n", 32),
        use_sim_mask=p.get("use_sim_mask", False), mask_ratios=p.get("mask_ratios", {}),
        mask_mode=p.get("mask_mode", "thresholdbound"), attn_impl=p.get("attn_impl", "new_mask_type"),
        tile_size=p.get("tile_size"), rearrange_method=p.get("rearrange_method", "Gilbert"),
        warmup_steps=p.get("warmup_steps", 12), verbose=verbose,
        sim_2x_threshold=p.get("sim_2x_threshold", 0), sim_4x_threshold=p.get("sim_4x_threshold", 0),
        sim_8x_threshold=p.get("sim_8x_threshold", -1))
    module = PyramidSparseAttention(config=cfg, inference_num=inference_num, layer_num=len(model.transformer_blocks),
                                    model_type="cogvideo")
    _swap_processors(model.transformer_blocks, module, SparseCogVideoXAttnProcessor, verbose)
    return module


def set_adaptive_sparse_attention(pipe, model_name: str, inference_num: int = 50, video_shape=None,
                                  attention_type: Optional[str] = "PSA", attention_preset: Optional[str] = None,
                                  verbose: bool = False, config_path: Optional[str] = None):
    """Resolve the preset for (model, video shape) and route every self-attention of the pipeline's transformer(s)
    through ONE shared PyramidSparseAttention (modify_diffusers.py:551-646).  Returns the resolved preset dictionary, as
    the reference does; the installed module is ``pipe.transformer.blocks[0].attn1.inner_attention``.  Dense presets
    and attention_type "dense"/"none" leave the pipeline untouched."""
    if video_shape is None:
        raise ValueError("Please provide video_shape=[width, height, depth] for configuring attention.")
    low = model_name.lower()
    is_cog, is_wan = "cogvideo" in low, "wan" in low
    if not is_cog and not is_wan:
        raise ValueError(f"Unsupported model: {model_name}. "
                         f"Supported models: {list(SUPPORTED_MODELS['CogVideo']) + list(SUPPORTED_MODELS['Wan'])}")
    kind = (attention_type or "psa").lower()
    if kind not in {"psa", "dense", "none"}:
        raise ValueError(f"Unsupported attention_type '{attention_type}'.")
    info = WanAttentionConfigLoader(config_path).get_attention_config(model_name, attention_preset, video_shape)
    if info["type"] == "dense" or kind in {"dense", "none"}:
        return info
    if is_cog:
        transformer = pipe.transformer if hasattr(pipe, "transformer") else pipe
        set_block_sparse_attn_cogvideox(transformer, model_name, inference_num, info, verbose)
        return info
    module = set_block_sparse_attn_wan(pipe.transformer, model_name, inference_num, info, verbose)
    second = getattr(pipe, "transformer_2", None)
    if second is not None:
        # the second expert of the Wan 2.2 pipelines shares module AND processors with the first, layer by layer
        for idx, block in enumerate(second.blocks):
            first = pipe.transformer.blocks[idx].attn1
            block.attn1.verbose = verbose
            block.attn1.inner_attention = module
            block.attn1.set_processor(first.processor)
            if not hasattr(block.attn1, "origin_processor"):
                block.attn1.origin_processor = first.origin_processor
    return info


def reset_wan_attention_to_dense(pipe, include_transformer_2: bool = True):
    """Put the stock processors back and drop the sparse module (modify_diffusers.py:649-678).  ``pipe`` is a pipeline
    (``transformer`` / ``transformer_2``) or a transformer itself (``blocks``)."""
    if hasattr(pipe, "blocks"):
        targets = [pipe]
    else:
        targets = [getattr(pipe, "transformer", None)]
        if include_transformer_2:
            targets.append(getattr(pipe, "transformer_2", None))
    for t in targets:
        for block in (getattr(t, "blocks", None) or []):
            a = getattr(block, "attn1", None)
            if a is None:
                continue
            if hasattr(a, "origin_processor"):
                a.set_processor(a.origin_processor)
            if hasattr(a, "inner_attention"):
                a.inner_attention = None
            a.verbose = False
