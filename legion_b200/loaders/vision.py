"""Vision towers from checkpoints: the ``model.visual.*`` tensors of a Hugging Face Qwen3-VL-style checkpoint and
``clip`` mmproj GGUF files (``qwen3vl_merger`` projector), mapped to the flat names of ``vision.tower``; and a
writer of tiny random mmproj files for tests.

Reference counterparts: ``src/hf/vision.rs`` (HF tensors as the converter would write them), ``src/vision/mod.rs``
(``VisionHparams::from_gguf``), ``src/vision/tiny.rs`` (tiny mmproj for tests)."""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple

import torch

from ..vision.preprocess import VisionHparams
from ..vision.tower import VisionConfig, VisionTower, random_vision_weights

# flat name -> (HF suffix under "model.visual." / "visual.", GGUF clip name)
_BLOCK = {
    "ln1.w": ("norm1.weight", "ln1.weight"), "ln1.b": ("norm1.bias", "ln1.bias"),
    "qkv.w": ("attn.qkv.weight", "attn_qkv.weight"), "qkv.b": ("attn.qkv.bias", "attn_qkv.bias"),
    "proj.w": ("attn.proj.weight", "attn_out.weight"), "proj.b": ("attn.proj.bias", "attn_out.bias"),
    "ln2.w": ("norm2.weight", "ln2.weight"), "ln2.b": ("norm2.bias", "ln2.bias"),
    "fc1.w": ("mlp.linear_fc1.weight", "ffn_up.weight"), "fc1.b": ("mlp.linear_fc1.bias", "ffn_up.bias"),
    "fc2.w": ("mlp.linear_fc2.weight", "ffn_down.weight"), "fc2.b": ("mlp.linear_fc2.bias", "ffn_down.bias"),
}
_MERGER_HF = {"ln.w": "norm.weight", "ln.b": "norm.bias", "fc1.w": "linear_fc1.weight", "fc1.b": "linear_fc1.bias",
              "fc2.w": "linear_fc2.weight", "fc2.b": "linear_fc2.bias"}


def hf_names(cfg: VisionConfig, prefix: str = "model.visual.") -> Dict[str, str]:
    """flat tower name -> checkpoint tensor name."""
    out = {"patch.w": prefix + "patch_embed.proj.weight", "patch.b": prefix + "patch_embed.proj.bias",
           "pos": prefix + "pos_embed.weight"}
    for i in range(cfg.depth):
        for k, (hf, _) in _BLOCK.items():
            out[f"blk{i}.{k}"] = f"{prefix}blocks.{i}.{hf}"
    for k, hf in _MERGER_HF.items():
        out[f"merger.{k}"] = f"{prefix}merger.{hf}"
        for j in range(len(cfg.deepstack_layers)):
            out[f"ds{j}.{k}"] = f"{prefix}deepstack_merger_list.{j}.{hf}"
    return out


def gguf_names(cfg: VisionConfig) -> Dict[str, str]:
    """flat tower name -> ``clip`` mmproj tensor name (the two frames of the temporal patch are two tensors there)."""
    out = {"patch.b": "v.patch_embd.bias", "pos": "v.position_embd.weight",
           "merger.ln.w": "v.post_ln.weight", "merger.ln.b": "v.post_ln.bias",
           "merger.fc1.w": "mm.0.weight", "merger.fc1.b": "mm.0.bias",
           "merger.fc2.w": "mm.2.weight", "merger.fc2.b": "mm.2.bias"}
    for i in range(cfg.depth):
        for k, (_, gg) in _BLOCK.items():
            out[f"blk{i}.{k}"] = f"v.blk.{i}.{gg}"
    for j, layer in enumerate(cfg.deepstack_layers):
        for k, gg in (("ln.w", "norm.weight"), ("ln.b", "norm.bias"), ("fc1.w", "fc1.weight"), ("fc1.b", "fc1.bias"),
                      ("fc2.w", "fc2.weight"), ("fc2.b", "fc2.bias")):
            out[f"ds{j}.{k}"] = f"v.deepstack.{layer}.{gg}"
    return out


def config_from_hf(vc: dict, lm_hidden: Optional[int] = None) -> VisionConfig:
    """``vision_config`` of a Hugging Face ``config.json``."""
    act = {"gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu", "silu": "silu"}.get(vc.get("hidden_act", "gelu_pytorch_tanh"),
                                                                                "gelu_tanh")
    return VisionConfig(depth=int(vc["depth"]), hidden=int(vc["hidden_size"]), n_head=int(vc["num_heads"]),
                        intermediate=int(vc["intermediate_size"]), out_hidden=int(vc.get("out_hidden_size", lm_hidden or 0)),
                        patch_size=int(vc.get("patch_size", 16)), temporal_patch_size=int(vc.get("temporal_patch_size", 2)),
                        spatial_merge_size=int(vc.get("spatial_merge_size", 2)),
                        num_pos=int(vc.get("num_position_embeddings", 2304)),
                        deepstack_layers=tuple(vc.get("deepstack_visual_indexes", ())), act=act)


def load_vision_hf(path: str, device="cpu", dtype=torch.float32) -> Optional[Tuple[VisionTower, VisionHparams]]:
    """The tower a Hugging Face checkpoint directory ships, or None when it has none."""
    from .safetensors_io import Checkpoint
    with open(os.path.join(path, "config.json")) as f:
        conf = json.load(f)
    vc = conf.get("vision_config")
    if not vc:
        return None
    lm = conf.get("text_config", conf)
    if vc.get("model_type") == "gemma4_vision":
        return load_gemma4_vision_hf(path, vc, int(lm["hidden_size"]), device, dtype)
    cfg = config_from_hf(vc, lm.get("hidden_size"))
    ck = Checkpoint(path)
    prefix = next((p for p in ("model.visual.", "visual.") if ck.has(p + "pos_embed.weight")), None)
    if prefix is None:
        return None
    w = {}
    for flat, name in hf_names(cfg, prefix).items():
        t = ck.get(name)
        if flat == "patch.w":
            t = t.reshape(t.shape[0], -1)            # the 3-D convolution kernel, flattened over (3, temporal, P, P)
        w[flat] = t.to(device=device, dtype=dtype)
    pp = {}
    ppath = os.path.join(path, "preprocessor_config.json")
    if os.path.exists(ppath):
        with open(ppath) as f:
            pp = json.load(f)
    size = pp.get("size", {}) if isinstance(pp.get("size"), dict) else {}
    hp = VisionHparams(patch_size=cfg.patch_size, spatial_merge_size=cfg.spatial_merge_size,
                       temporal_patch_size=cfg.temporal_patch_size,
                       image_min_pixels=int(size.get("shortest_edge", 0) or 0),
                       image_max_pixels=int(size.get("longest_edge", 0) or 0),
                       image_mean=tuple(pp.get("image_mean", (0.5, 0.5, 0.5))),
                       image_std=tuple(pp.get("image_std", (0.5, 0.5, 0.5))), resize="stretch")
    return VisionTower(cfg, w), hp


def load_mmproj(path: str, device="cpu", dtype=torch.float32) -> Tuple[VisionTower, VisionHparams]:
    """A ``clip`` mmproj GGUF with the ``qwen3vl_merger`` or the ``gemma4v`` projector."""
    from .gguf import GgufFile
    g = GgufFile(path)
    md = g.metadata
    arch = md.get("general.architecture", "")
    proj = md.get("clip.vision.projector_type", md.get("clip.projector_type", ""))
    if arch == "clip" and proj == "gemma4v":
        return _load_gemma4v_mmproj(g, device, dtype)
    if arch != "clip" or proj != "qwen3vl_merger":
        raise ValueError(f"unsupported vision architecture / projector: {arch}/{proj}")

    def need(key):
        if f"clip.vision.{key}" not in md:
            raise ValueError(f"missing vision metadata: clip.vision.{key}")
        return md[f"clip.vision.{key}"]

    hidden, depth = int(need("embedding_length")), int(need("block_count"))
    deep = md.get("clip.vision.is_deepstack_layers")
    layers = tuple(i for i, f in enumerate(deep) if f) if deep is not None else ()
    pos = g.torch("v.position_embd.weight")
    cfg = VisionConfig(depth=depth, hidden=hidden, n_head=int(need("attention.head_count")),
                       intermediate=int(need("feed_forward_length")), out_hidden=int(need("projection_dim")),
                       patch_size=int(need("patch_size")), temporal_patch_size=2,
                       spatial_merge_size=int(md.get("clip.vision.spatial_merge_size", 2)), num_pos=int(pos.shape[0]),
                       deepstack_layers=layers, ln_eps=float(md.get("clip.vision.attention.layer_norm_epsilon", 1e-6)),
                       act="gelu_tanh" if md.get("clip.use_gelu", True) else "silu")
    w = {}
    for flat, name in gguf_names(cfg).items():
        w[flat] = g.torch(name).to(device=device, dtype=dtype)
    # the temporal patch: frame 0 in v.patch_embd.weight, frame 1 in v.patch_embd.weight.1, each [hidden, 3, P, P]
    f0 = g.torch("v.patch_embd.weight").reshape(hidden, 3, 1, cfg.patch_size, cfg.patch_size)
    f1 = g.torch("v.patch_embd.weight.1").reshape(hidden, 3, 1, cfg.patch_size, cfg.patch_size)
    w["patch.w"] = torch.cat([f0, f1], dim=2).reshape(hidden, -1).to(device=device, dtype=dtype)
    hp = VisionHparams(patch_size=cfg.patch_size, spatial_merge_size=cfg.spatial_merge_size,
                       image_min_pixels=int(md.get("clip.vision.image_min_pixels", 0) or 0),
                       image_max_pixels=int(md.get("clip.vision.image_max_pixels", 0) or 0),
                       image_mean=tuple(float(v) for v in need("image_mean")[:3]),
                       image_std=tuple(float(v) for v in need("image_std")[:3]), resize="pad")
    return VisionTower(cfg, w), hp


def write_tiny_mmproj(path: str, cfg: Optional[VisionConfig] = None, seed: int = 0) -> VisionConfig:
    """A tiny random ``qwen3vl_merger`` mmproj as a GGUF file (tests)."""
    from .gguf import GgufWriter
    cfg = cfg or VisionConfig()
    w = random_vision_weights(cfg, seed=seed)
    md = {"clip.projector_type": "qwen3vl_merger", "clip.has_vision_encoder": True,
          "clip.use_gelu": True, "clip.vision.embedding_length": cfg.hidden, "clip.vision.block_count": cfg.depth,
          "clip.vision.attention.head_count": cfg.n_head, "clip.vision.feed_forward_length": cfg.intermediate,
          "clip.vision.projection_dim": cfg.out_hidden, "clip.vision.patch_size": cfg.patch_size,
          "clip.vision.spatial_merge_size": cfg.spatial_merge_size,
          "clip.vision.attention.layer_norm_epsilon": cfg.ln_eps,
          "clip.vision.image_mean": [0.5, 0.5, 0.5], "clip.vision.image_std": [0.5, 0.5, 0.5],
          "clip.vision.is_deepstack_layers": [i in cfg.deepstack_layers for i in range(cfg.depth)]}
    wr = GgufWriter(path, "clip")
    for k, v in md.items():
        wr.add(k, v)
    for flat, name in gguf_names(cfg).items():
        wr.add_tensor(name, w[flat].float())
    pw = w["patch.w"].float().reshape(cfg.hidden, 3, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)
    wr.add_tensor("v.patch_embd.weight", pw[:, :, 0].contiguous())
    wr.add_tensor("v.patch_embd.weight.1", pw[:, :, 1].contiguous())
    wr.write()
    return cfg


def load_gemma4_vision_hf(path: str, vc: dict, lm_hidden: int, device="cpu", dtype=torch.float32):
    """The Gemma 4 tower of a Hugging Face checkpoint directory (``model.vision_tower.*`` and the projection
    ``model.embed_vision.*``). The patch projection's columns go from the checkpoint's (row, column, channel) order
    inside a patch to the channel-major order the preprocessor emits. Pixels stay in [0, 1] (the tower rescales);
    the grid is aligned to the pooling kernel."""
    from ..vision.gemma4v import Gemma4VisionConfig, Gemma4VisionTower
    from .safetensors_io import Checkpoint
    if vc.get("use_clipped_linears"):
        raise ValueError("gemma4 vision: towers with clipped linears are not supported")
    rope = vc.get("rope_parameters") or {}
    nh = int(vc["num_attention_heads"])
    cfg = Gemma4VisionConfig(depth=int(vc["num_hidden_layers"]), hidden=int(vc["hidden_size"]), n_head=nh,
                             n_kv_head=int(vc.get("num_key_value_heads") or nh),
                             head_dim=int(vc.get("head_dim") or int(vc["hidden_size"]) // nh),
                             intermediate=int(vc["intermediate_size"]), out_hidden=lm_hidden,
                             patch_size=int(vc.get("patch_size", 16)), spatial_merge_size=int(vc.get("pooling_kernel_size", 3)),
                             num_pos=int(vc.get("position_embedding_size", 10240)),
                             act={"gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu", "silu": "silu"}.get(
                                 vc.get("hidden_activation", "gelu_pytorch_tanh"), "gelu_tanh"),
                             ln_eps=float(vc.get("rms_norm_eps", 1e-6)), rope_theta=float(rope.get("rope_theta", 100.0)),
                             standardize=bool(vc.get("standardize", False)))
    ck = Checkpoint(path)
    V = next((p for p in ("model.vision_tower.", "vision_tower.") if ck.has(p + "patch_embedder.input_proj.weight")), None)
    if V is None:
        return None
    E = V.replace("vision_tower.", "embed_vision.")
    to = lambda t: t.to(device=device, dtype=dtype)           # noqa: E731
    P = cfg.patch_size
    pw = ck.get(V + "patch_embedder.input_proj.weight")
    table = ck.get(V + "patch_embedder.position_embedding_table")
    w = {"patch.w": to(pw.reshape(pw.shape[0], P, P, 3).permute(0, 3, 1, 2).reshape(pw.shape[0], -1).contiguous()),
         "pos.x": to(table[0]), "pos.y": to(table[1]), "proj.w": to(ck.get(E + "embedding_projection.weight"))}
    if cfg.standardize:
        w["std.bias"], w["std.scale"] = to(ck.get(V + "std_bias")), to(ck.get(V + "std_scale"))
    names = {"q.w": "self_attn.q_proj.linear.weight", "k.w": "self_attn.k_proj.linear.weight",
             "v.w": "self_attn.v_proj.linear.weight", "o.w": "self_attn.o_proj.linear.weight",
             "q_norm.w": "self_attn.q_norm.weight", "k_norm.w": "self_attn.k_norm.weight",
             "ln1.w": "input_layernorm.weight", "post_attn.w": "post_attention_layernorm.weight",
             "ln2.w": "pre_feedforward_layernorm.weight", "post_ffn.w": "post_feedforward_layernorm.weight",
             "gate.w": "mlp.gate_proj.linear.weight", "up.w": "mlp.up_proj.linear.weight",
             "down.w": "mlp.down_proj.linear.weight"}
    for i in range(cfg.depth):
        for ours, theirs in names.items():
            w[f"blk{i}.{ours}"] = to(ck.get(f"{V}encoder.layers.{i}.{theirs}"))
    k = cfg.spatial_merge_size
    hp = VisionHparams(patch_size=P, spatial_merge_size=k, temporal_patch_size=1, image_mean=(0.0, 0.0, 0.0),
                       image_std=(1.0, 1.0, 1.0), resize="stretch", min_tokens=1, max_tokens=280)
    return Gemma4VisionTower(cfg, w), hp


_G4V_BLOCK = {"ln1.w": "ln1", "ln2.w": "ln2", "post_attn.w": "attn_post_norm", "post_ffn.w": "ffn_post_norm", "q.w": "attn_q",
              "k.w": "attn_k", "v.w": "attn_v", "o.w": "attn_out", "q_norm.w": "attn_q_norm", "k_norm.w": "attn_k_norm",
              "gate.w": "ffn_gate", "up.w": "ffn_up", "down.w": "ffn_down"}


def _load_gemma4v_mmproj(g, device, dtype):
    """The ``gemma4v`` projector of a ``clip`` mmproj (tensor names as the reference lists them,
    ``src/vision/gemma4v.rs::names``): the patch convolution kernel is the patch projection, the position tensor
    holds the column table and the row table, ``mm.input_projection`` maps the pooled rows to the model's width."""
    from ..vision.gemma4v import Gemma4VisionConfig, Gemma4VisionTower
    md = g.metadata
    if any(n.endswith(".input_min") or n.endswith(".output_min") for n in g.tensors):
        raise ValueError("gemma4v with clipped linears is not supported")

    def need(key):
        if f"clip.vision.{key}" not in md:
            raise ValueError(f"missing vision metadata: clip.vision.{key}")
        return md[f"clip.vision.{key}"]

    hidden, depth, nh = int(need("embedding_length")), int(need("block_count")), int(need("attention.head_count"))
    pos = g.torch("v.position_embd.weight")
    if pos.dim() != 3 or pos.shape[0] != 2:
        raise ValueError("v.position_embd.weight: not two tables")
    proj = g.torch("mm.input_projection.weight")
    kw = g.torch("v.blk.0.attn_k.weight")
    cfg = Gemma4VisionConfig(depth=depth, hidden=hidden, n_head=nh, n_kv_head=kw.shape[0] // (hidden // nh),
                             head_dim=hidden // nh, intermediate=int(need("feed_forward_length")),
                             out_hidden=int(proj.shape[0]), patch_size=int(need("patch_size")),
                             spatial_merge_size=int(md.get("clip.vision.projector.scale_factor", 3)),
                             num_pos=int(pos.shape[1]), ln_eps=float(md.get("clip.vision.attention.layer_norm_epsilon", 1e-6)),
                             standardize="v.std_bias" in g.tensors)
    to = lambda t: t.to(device=device, dtype=dtype)           # noqa: E731
    w = {"patch.w": to(g.torch("v.patch_embd.weight").reshape(hidden, -1)), "pos.x": to(pos[0]), "pos.y": to(pos[1]),
         "proj.w": to(proj)}
    if cfg.standardize:
        w["std.bias"], w["std.scale"] = to(g.torch("v.std_bias")), to(g.torch("v.std_scale"))
    for i in range(depth):
        for ours, theirs in _G4V_BLOCK.items():
            w[f"blk{i}.{ours}"] = to(g.torch(f"v.blk.{i}.{theirs}.weight"))
    # the tower takes pixels in [0, 1] and rescales them itself; 70 .. 1120 rows per image
    hp = VisionHparams(patch_size=cfg.patch_size, spatial_merge_size=cfg.spatial_merge_size, temporal_patch_size=1,
                       image_mean=(0.0, 0.0, 0.0), image_std=(1.0, 1.0, 1.0), resize="stretch", min_tokens=70,
                       max_tokens=1120)
    return Gemma4VisionTower(cfg, w), hp


def write_tiny_gemma4v_mmproj(path: str, cfg=None, seed: int = 0):
    """A small ``gemma4v`` mmproj with random weights (tests and demos)."""
    from ..vision.gemma4v import Gemma4VisionConfig, random_gemma4v_weights
    from .gguf import GgufWriter
    cfg = cfg or Gemma4VisionConfig(standardize=True)
    w = random_gemma4v_weights(cfg, seed=seed)
    wr = GgufWriter(path, "clip")
    wr.add("clip.vision.projector_type", "gemma4v")
    for k, v in (("embedding_length", cfg.hidden), ("block_count", cfg.depth), ("attention.head_count", cfg.n_head),
                 ("feed_forward_length", cfg.intermediate), ("patch_size", cfg.patch_size),
                 ("projector.scale_factor", cfg.spatial_merge_size)):
        wr.add(f"clip.vision.{k}", int(v))
    wr.add("clip.vision.attention.layer_norm_epsilon", float(cfg.ln_eps))
    P = cfg.patch_size
    wr.add_tensor("v.patch_embd.weight", w["patch.w"].float().reshape(cfg.hidden, 3, P, P).contiguous())
    wr.add_tensor("v.position_embd.weight", torch.stack([w["pos.x"], w["pos.y"]]).float().contiguous())
    wr.add_tensor("mm.input_projection.weight", w["proj.w"])
    if cfg.standardize:
        wr.add_tensor("v.std_bias", w["std.bias"])
        wr.add_tensor("v.std_scale", w["std.scale"])
    for i in range(cfg.depth):
        for ours, theirs in _G4V_BLOCK.items():
            wr.add_tensor(f"v.blk.{i}.{theirs}.weight", w[f"blk{i}.{ours}"])
    wr.write()
    return cfg, w
