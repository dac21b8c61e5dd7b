"""Seeded synthetic safetensors checkpoints for the converter tests: small models whose key sets make upstream's
architecture detection fire, with tensors that exercise every branch of the planner (1-D, small, high-precision keys,
skipped keys, ignored keys, widths that do not divide the block size, the SD1/SDXL shape fix, F32 / F16 / BF16 sources)."""
from __future__ import annotations

import json
import struct

import numpy as np


def _bf16_bits(x: np.ndarray) -> np.ndarray:
    return (x.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)


def write_safetensors(path: str, tensors: list[tuple[str, str, np.ndarray]], metadata: dict | None = None) -> None:
    """tensors: (name, dtype "F32" | "F16" | "BF16", fp32 values of the wanted shape)."""
    header, blobs, offset = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dtype, values in tensors:
        if dtype == "F32":
            raw = values.astype(np.float32).tobytes()
        elif dtype == "F16":
            raw = values.astype(np.float16).tobytes()
        else:
            raw = _bf16_bits(values).tobytes()
        header[name] = {"dtype": dtype, "shape": list(values.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def _values(rng, shape):
    return (rng.standard_normal(shape) * 0.05).astype(np.float32)


def flux_like(seed: int = 0, dtype: str = "BF16", layers: int = 3):
    rng = np.random.default_rng(seed)
    t = [("model.diffusion_model.img_in.weight", dtype, _values(rng, (256, 64))),
         ("model.diffusion_model.time_in.in_layer.weight", dtype, _values(rng, (256, 256))),
         ("model.diffusion_model.final_layer.linear.weight", dtype, _values(rng, (64, 256)))]
    for i in range(layers):
        p = f"model.diffusion_model.double_blocks.{i}."
        t += [(p + "img_attn.qkv.weight", dtype, _values(rng, (768, 256))),
              (p + "img_attn.qkv.bias", dtype, _values(rng, (768,))),
              (p + "img_attn.proj.weight", dtype, _values(rng, (256, 256))),
              (p + "img_attn.norm.query_norm.scale", dtype, _values(rng, (32,))),
              (p + "img_mlp.0.weight", dtype, _values(rng, (1024, 256))),
              (p + "img_mlp.2.weight", dtype, _values(rng, (256, 1024))),
              (p + "img_mod.lin.weight", "F32", _values(rng, (1536, 256))),
              (p + "odd_width.weight", dtype, _values(rng, (64, 96)))]
    t.append(("unrelated.weight", dtype, _values(rng, (256, 256))))  # lacks the prefix: dropped
    return t


def wan_like(seed: int = 1, dtype: str = "F16", layers: int = 30):
    rng = np.random.default_rng(seed)
    t = [("text_embedding.2.weight", dtype, _values(rng, (256, 256))), ("head.modulation", "F32", _values(rng, (1, 2, 256))),
         ("head.head.weight", dtype, _values(rng, (64, 256))), ("patch_embedding.weight", dtype, _values(rng, (256, 16, 1, 2, 2)))]
    for i in range(layers):
        p = f"blocks.{i}."
        t += [(p + "self_attn.norm_q.weight", dtype, _values(rng, (256,))),
              (p + "self_attn.q.weight", dtype, _values(rng, (256, 256))),
              (p + "self_attn.v.weight", dtype, _values(rng, (256, 256))),
              (p + "self_attn.o.weight", dtype, _values(rng, (256, 256))),
              (p + "ffn.0.weight", dtype, _values(rng, (512, 256))),
              (p + "ffn.2.weight", dtype, _values(rng, (256, 512))),
              (p + "modulation", "F32", _values(rng, (1, 6, 256)))]
    return t


def sd1_like(seed: int = 2, dtype: str = "F16"):
    rng = np.random.default_rng(seed)
    t = [("model.diffusion_model.input_blocks.0.0.weight", dtype, _values(rng, (64, 4, 3, 3)))]
    for i in (3, 6, 9):
        t.append((f"model.diffusion_model.input_blocks.{i}.0.op.weight", dtype, _values(rng, (64, 64, 3, 3))))
    for name in ("output_blocks.2.1.conv.weight", "output_blocks.5.2.conv.weight", "output_blocks.8.2.conv.weight"):
        t.append(("model.diffusion_model." + name, dtype, _values(rng, (64, 64, 3, 3))))
    for i in range(2):
        p = f"model.diffusion_model.input_blocks.{i + 1}.1.transformer_blocks.0."
        t += [(p + "attn1.to_q.weight", dtype, _values(rng, (256, 256))), (p + "attn1.to_v.weight", dtype, _values(rng, (256, 256))),
              (p + "attn1.to_out.0.weight", dtype, _values(rng, (256, 256))), (p + "ff.net.2.weight", dtype, _values(rng, (256, 1024))),
              (p + "norm1.weight", dtype, _values(rng, (256,)))]
    t.append(("model.diffusion_model.time_embed.0.weight", dtype, _values(rng, (256, 64))))
    t.append(("first_stage_model.decoder.conv_in.weight", dtype, _values(rng, (8, 4, 3, 3))))
    return t


def cosmos_like(seed: int = 3, dtype: str = "BF16"):
    rng = np.random.default_rng(seed)
    t = [("net.pos_embedder.seq", dtype, _values(rng, (64, 32))), ("net.accum_video_sample_counter", "F32", _values(rng, (1,))),
         ("net.final_layer.linear.weight", dtype, _values(rng, (64, 256)))]
    for i in range(3):
        p = f"net.blocks.{i}."
        t += [(p + "mlp.layer1.weight", dtype, _values(rng, (512, 256))), (p + "mlp.layer2.weight", dtype, _values(rng, (256, 512))),
              (p + "adaln_modulation_cross_attn.1.weight", dtype, _values(rng, (768, 256))),
              (p + "self_attn.q_proj.weight", dtype, _values(rng, (256, 256))), (p + "self_attn.v_proj.weight", dtype, _values(rng, (256, 256))),
              (p + "self_attn.output_proj.weight", dtype, _values(rng, (256, 256))), (p + "self_attn._extra_state", "F32", _values(rng, (4,)))]
    return t


def llama_like(seed: int = 4, dtype: str = "BF16", layers: int = 8):
    rng = np.random.default_rng(seed)
    t = [("model.embed_tokens.weight", dtype, _values(rng, (512, 256))), ("model.norm.weight", dtype, _values(rng, (256,))),
         ("lm_head.weight", dtype, _values(rng, (512, 256)))]
    for i in range(layers):
        p = f"model.layers.{i}."
        t += [(p + "self_attn.q_proj.weight", dtype, _values(rng, (256, 256))), (p + "self_attn.k_proj.weight", dtype, _values(rng, (64, 256))),
              (p + "self_attn.v_proj.weight", dtype, _values(rng, (64, 256))), (p + "self_attn.o_proj.weight", dtype, _values(rng, (256, 256))),
              (p + "mlp.gate_proj.weight", dtype, _values(rng, (768, 256))), (p + "mlp.up_proj.weight", dtype, _values(rng, (768, 256))),
              (p + "mlp.down_proj.weight", dtype, _values(rng, (256, 768))), (p + "input_layernorm.weight", dtype, _values(rng, (256,)))]
    return t


# name -> (builder, list of (case name, extra command line options))
CASES = {
    "flux_bf16": (lambda: flux_like(), [("q4_k_m", ["--qtype", "Q4_K_M"]), ("q8_0", ["--qtype", "Q8_0"]),
                                        ("q3_k_m_dynamic", ["--qtype", "Q3_K_M", "--policy", "dynamic"]),
                                        ("q5_k_s_uniform", ["--qtype", "Q5_K_S", "--policy", "uniform"]),
                                        ("q4_0_overrides", ["--qtype", "Q4_0", "--tensor-type", "*img_mlp.0.weight=Q6_K", "--tensor-type",
                                                            "*proj.weight=F16", "--include", "img_in.weight", "--exclude", "*img_mod*"])]),
    "flux_f32": (lambda: flux_like(seed=5, dtype="F32", layers=2), [("q2_k", ["--qtype", "Q2_K"]), ("q6_k", ["--qtype", "Q6_K"])]),
    "wan_f16": (lambda: wan_like(), [("q4_k_s", ["--qtype", "Q4_K_S"]), ("q4_k_m_dynamic", ["--qtype", "Q4_K_M", "--policy", "dynamic"]),
                                     ("q5_k_m_dynamic", ["--qtype", "Q5_K_M", "--policy", "dynamic"]), ("q5_1", ["--qtype", "Q5_1"])]),
    "sd1_f16": (lambda: sd1_like(), [("q4_k_m", ["--qtype", "Q4_K_M"]), ("q5_0", ["--qtype", "Q5_0"])]),
    "cosmos_bf16": (lambda: cosmos_like(), [("q3_k_l", ["--qtype", "Q3_K_L"]), ("q1_0", ["--qtype", "Q1_0"])]),
}
