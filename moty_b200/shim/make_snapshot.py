"""Write a synthetic Qwen3-shaped snapshot the reference's `qwen` engine can load: config.json, one
bf16 model.safetensors and a REF file (prompt ids + placeholders for the ids to generate).

    python -m moty_b200.shim.make_snapshot <dir> [--layers 28] [--prompt 64] [--gen 128]

Defaults are the Qwen3-0.6B shape: 28 layers, hidden 1024, 16 query / 8 KV heads of 128 with QK-norm,
RoPE theta 1e6, SwiGLU FFN 3072, vocabulary 151936, tied embeddings.  Every matrix is N(0, 0.02) from
seed 0 rounded to bf16, norm gains are 1.0, the prompt is uniform random ids from seed 1.  Tensor
names are the ones the engine's loader asks for (engines/qwen.c:439-501).  No tokenizer is written:
REF= mode needs none (runtime/rt_gen_loop.h:46-84).
"""
from __future__ import annotations

import argparse
import json
import os
import struct

import numpy as np


def _bf16(a: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_snapshot(path: str, layers: int = 28, hidden: int = 1024, heads: int = 16, kv_heads: int = 8, head_dim: int = 128,
                   inter: int = 3072, vocab: int = 151936, prompt: int = 64, gen: int = 128, seed: int = 0) -> dict:
    os.makedirs(path, exist_ok=True)
    cfg = {"model_type": "qwen3", "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": heads,
           "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter, "vocab_size": vocab,
           "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True,
           "eos_token_id": vocab - 1}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = [("model.embed_tokens.weight", (vocab, hidden), "m"), ("model.norm.weight", (hidden,), "1")]
    for i in range(layers):
        p = f"model.layers.{i}."
        names += [(p + "input_layernorm.weight", (hidden,), "1"), (p + "post_attention_layernorm.weight", (hidden,), "1"),
                  (p + "self_attn.q_proj.weight", (heads * head_dim, hidden), "m"),
                  (p + "self_attn.k_proj.weight", (kv_heads * head_dim, hidden), "m"),
                  (p + "self_attn.v_proj.weight", (kv_heads * head_dim, hidden), "m"),
                  (p + "self_attn.o_proj.weight", (hidden, heads * head_dim), "m"),
                  (p + "self_attn.q_norm.weight", (head_dim,), "1"), (p + "self_attn.k_norm.weight", (head_dim,), "1"),
                  (p + "mlp.gate_proj.weight", (inter, hidden), "m"), (p + "mlp.up_proj.weight", (inter, hidden), "m"),
                  (p + "mlp.down_proj.weight", (hidden, inter), "m")]
    header, off = {}, 0
    for name, shape, _ in names:
        n = int(np.prod(shape)) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    rng = np.random.default_rng(seed)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj))); f.write(hj)
        for name, shape, kind in names:
            if kind == "1":
                f.write(_bf16(np.ones(shape, np.float32)).tobytes())
            else:
                f.write(_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).tobytes())
    ids = np.random.default_rng(1).integers(0, vocab, prompt).tolist()
    with open(os.path.join(path, "ref.json"), "w") as f:
        json.dump({"prompt_ids": ids, "full_ids": ids + [0] * gen}, f)
    return cfg


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("dir")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--gen", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=151936)
    a = ap.parse_args()
    write_snapshot(a.dir, layers=a.layers, prompt=a.prompt, gen=a.gen, vocab=a.vocab)
    print(a.dir)
