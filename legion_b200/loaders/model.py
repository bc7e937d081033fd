"""One entry point to open a model: a ``.gguf`` file, an HF checkpoint directory (safetensors, BF16 / FP8 /
NVFP4), or ``random:<preset>`` for random-init weights of a named shape (benchmarks and tests).

Returns the hyper-parameters, canonical weights (this rank's shard under TP / EP) and a tokenizer, the way
the reference's ``LmEngine::load`` opens GGUF directly and HF directories through its converter
(``src/engine/lm.rs:3932``, ``src/hf/mod.rs:64``).
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from ..config import PRESETS, ModelConfig
from ..models.weights import Shard, random_weights
from .tokenizer import BpeTokenizer, ByteTokenizer, Tokenizer, tokenizer_from_gguf_metadata


def load_model(path: str, device="cpu", dtype=None, rank: int = 0, world: int = 1, expert_parallel: bool = False,
               seed: int = 0, keep_layers=None, dp_attention: bool = False,
               keep_quant: bool = False, read_threads: int = 0) -> Tuple[ModelConfig, Dict[str, torch.Tensor], Tokenizer, dict]:
    """``keep_layers(il)``: a pipeline stage keeps only the layers it owns (plus embeddings and head).
    ``keep_quant`` (HF directories on a GPU): NVFP4 / FP8 tensors stay in their shipped encoding; with expert
    parallelism every rank reads only its own experts from the files, straight to its GPU."""
    from ..models.weights import layer_of
    keep = None
    if keep_layers is not None:
        keep = lambda name: layer_of(name) is None or keep_layers(layer_of(name))   # noqa: E731
    dev = torch.device(device)
    if dtype is None:
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    info: dict = {"source": path}
    if path.startswith("random:"):
        cfg = PRESETS[path.split(":", 1)[1]]()
        shard = Shard(cfg, rank, world, expert_parallel, dp_attention) if world > 1 else None
        w = random_weights(cfg, dev, dtype, seed=seed, shard=shard, keep=keep)
        return cfg, w, ByteTokenizer(cfg.vocab), info
    if os.path.isdir(path):
        from .hf_map import load_hf
        local_experts = None
        if keep_quant and dev.type == "cuda" and world > 1 and (expert_parallel or dp_attention):
            from .safetensors_io import Checkpoint
            from .hf_map import config_from_hf
            c0 = config_from_hf(Checkpoint(path).config)
            if c0.n_expert and c0.n_expert % world == 0:
                per = c0.n_expert // world
                local_experts = (rank * per, (rank + 1) * per)
        if local_experts is not None:
            # sharded read: this rank's experts only, encoded, straight to the GPU; the rest is sliced below
            cfg, w, ck = load_hf(path, dev, dtype, keep_quant=True, expert_range=local_experts,
                                 keep_quant_dense=dp_attention, read_threads=read_threads)
        else:
            cfg, w, ck = load_hf(path, "cpu" if world > 1 else dev, dtype,
                                 keep_quant=keep_quant and world == 1 and dev.type == "cuda", read_threads=read_threads)
        info["quant_method"] = ck.quant_method()
        info["local_experts"] = local_experts
        tok: Tokenizer
        if os.path.exists(os.path.join(path, "tokenizer.json")):
            tok = BpeTokenizer.from_hf_dir(path)
        else:
            tok = ByteTokenizer(cfg.vocab)
    elif path.endswith(".gguf"):
        from .gguf_map import load_gguf
        cfg, w, md = load_gguf(path, "cpu" if world > 1 else dev, dtype)
        info["gguf_arch"] = md.get("general.architecture")
        kind = md.get("tokenizer.ggml.model", "gpt2")
        if "tokenizer.ggml.tokens" in md and ((kind in ("gpt2", "gemma4") and "tokenizer.ggml.merges" in md)
                                              or (kind == "llama" and "tokenizer.ggml.scores" in md)):
            tok = tokenizer_from_gguf_metadata(md)
        else:
            tok = ByteTokenizer(cfg.vocab)
            if md.get("tokenizer.chat_template"):
                tok.chat_template = md["tokenizer.chat_template"]
    else:
        raise ValueError(f"cannot tell what kind of model {path!r} is (expected .gguf, an HF directory or random:<preset>)")
    if keep is not None:
        w = {k: v for k, v in w.items() if keep(k)}
    if world > 1:
        sh = Shard(cfg, rank, world, expert_parallel, dp_attention)
        pre_sliced = info.get("local_experts") is not None

        def place(k, v):
            if pre_sliced and k.endswith(("moe.gate_up", "moe.down")):
                return v                         # read as this rank's experts already
            if not isinstance(v, torch.Tensor):
                return v
            return sh.slice(k, v).to(dev)
        w = {k: place(k, v) for k, v in w.items()}
    return cfg, w, tok, info
