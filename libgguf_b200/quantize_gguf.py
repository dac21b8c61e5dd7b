"""safetensors -> GGUF conversion with every tensor encoded on the GPUs.

    python -m libgguf_b200.quantize_gguf --src model.safetensors --qtype Q4_K_M [--dst out.gguf] [--gpus N | --gpus 0,2,3] ...

Planning follows upstream's native converter (csrc/quantize_gguf.cpp): header parse (:919-984), key prefix
stripping (:986-1021), architecture detection (:1023-1070), which tensors may be quantized (:1072-1105), the mixed
"comfy" policy (:1107-1138) and the layer-aware "dynamic" policy (:1140-1199), storage types of the tensors that stay
unquantized (:1201-1210), the SD1/SDXL shape fix (:1212-1224), overrides / include / exclude and the block-size
fallback (:1235-1316), GGUF metadata (:1336-1363, :2436-2439).  For the same input and options the output file is
byte-identical to upstream's.  The tensor loop (:1990-2223) is replaced: instead of one tensor at a time through one
GPU, all tensors whose bytes are not a plain copy of the source go, batch by batch, through the multi-GPU streaming
pipeline (libgguf_cuda_pipeline_*), 16-bit sources travelling as 16-bit values.

Additions over upstream, all opt-in by input: Llama-style checkpoints (keys `model.layers.N.self_attn.q_proj.weight`
...) are accepted as architecture "llama" with the Q4_K_M / Q5_K_M "more bits for half of attn_v and ffn_down, Q6_K
output" rule, and the IQ / TQ / MXFP4 families are accepted as --qtype (upstream rejects them, :584-586); types that need
importance weights derive them from each tensor.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
from dataclasses import dataclass, field

import numpy as np

from . import GGMLQuantizationType as Q
from . import row_size
from .gguf_file import DEFAULT_ALIGNMENT, T_ARRAY, T_INT64, T_STRING, T_UINT32, TensorInfo, header_bytes, pad_to

QUANT_VERSION = 2
QUANTIZATION_THRESHOLD = 1024
REARRANGE_THRESHOLD = 512
MAX_TENSOR_NAME_LENGTH = 127

BLOCK_SIZE = {"F32": 1, "F16": 1, "BF16": 1, "Q4_0": 32, "Q4_1": 32, "Q5_0": 32, "Q5_1": 32, "Q8_0": 32, "Q1_0": 128,
              "Q2_K": 256, "Q3_K": 256, "Q4_K": 256, "Q5_K": 256, "Q6_K": 256}
# accepted here, rejected by upstream's converter
EXTRA_BLOCK_SIZE = {"IQ2_XXS": 256, "IQ2_XS": 256, "IQ2_S": 256, "IQ3_XXS": 256, "IQ3_S": 256, "IQ1_S": 256, "IQ1_M": 256,
                    "IQ4_NL": 32, "IQ4_XS": 256, "TQ1_0": 256, "TQ2_0": 256, "MXFP4": 32, "NVFP4": 64}
FILE_TYPE_VALUE = {"Q4_0": 2, "Q4_1": 3, "Q8_0": 7, "Q5_0": 8, "Q5_1": 9, "Q2_K": 10, "Q3_K_S": 11, "Q3_K_M": 12, "Q3_K_L": 13,
                   "Q4_K_S": 14, "Q4_K_M": 15, "Q5_K_S": 16, "Q5_K_M": 17, "Q6_K": 18, "Q2_K_S": 21, "Q1_0": 27}
# llama.cpp's file type numbers for the families upstream's converter does not write
EXTRA_FILE_TYPE_VALUE = {"IQ2_XXS": 19, "IQ2_XS": 20, "IQ3_XXS": 23, "IQ1_S": 24, "IQ4_NL": 25, "IQ3_S": 26, "IQ2_S": 28,
                         "IQ4_XS": 30, "IQ1_M": 31, "TQ1_0": 36, "TQ2_0": 37, "MXFP4": 38}
SOURCE_DTYPES = {"F32": (np.float32, 0, 4), "F16": (np.float16, 1, 2), "BF16": (np.uint16, 2, 2)}


class ConversionError(RuntimeError):
    pass


def fail(message: str):
    raise ConversionError(message)


# ---- names and patterns -------------------------------------------------------------------------------------------
def fnmatch_case(pattern: str, text: str) -> bool:
    """`*` and `?` only, case sensitive, no character classes (upstream :636-668)."""
    p = t = 0
    star_p = star_t = -1
    while t < len(text):
        if p < len(pattern) and pattern[p] == "*":
            while p < len(pattern) and pattern[p] == "*":
                p += 1
            if p == len(pattern):
                return True
            star_p, star_t = p, t
        elif p < len(pattern) and (pattern[p] == "?" or pattern[p] == text[t]):
            p += 1
            t += 1
        elif star_p >= 0:
            star_t += 1
            p, t = star_p, star_t
        else:
            return False
    while p < len(pattern) and pattern[p] == "*":
        p += 1
    return p == len(pattern)


def matches_any(name: str, patterns) -> bool:
    return any(fnmatch_case(p, name) for p in patterns)


def contains_any(name: str, markers) -> bool:
    return any(m in name for m in markers)


_BLOCK_NAMES = {"blocks", "double_blocks", "double_layers", "double_stream_blocks", "input_blocks", "joint_blocks", "layers",
                "output_blocks", "single_blocks", "single_stream_blocks", "transformer_blocks"}


def dynamic_layer_index(key: str) -> int:
    parts = key.split(".")
    for a, b in zip(parts, parts[1:]):
        if a in _BLOCK_NAMES and b.isascii() and b.isdigit():
            return int(b)
    for a, b in zip(parts, parts[1:]):
        if a in ("context_refiner", "noise_refiner") and b.isascii() and b.isdigit():
            return int(b)
    return -1


_K_ORDER = ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_0"]


def promote_k_qtype(qtype: str, steps: int = 1) -> str:
    if qtype in _K_ORDER:
        return _K_ORDER[min(_K_ORDER.index(qtype) + steps, len(_K_ORDER) - 1)]
    return qtype


# ---- architectures ------------------------------------------------------------------------------------------------
@dataclass
class ModelTemplate:
    arch: str
    shape_fix: bool = False
    keys_detect: list = field(default_factory=list)
    keys_banned: list = field(default_factory=list)
    keys_hiprec: list = field(default_factory=list)
    keys_ignore: list = field(default_factory=list)


MODEL_TEMPLATES = [
    ModelTemplate("flux", False, [["transformer_blocks.0.attn.norm_added_k.weight"], ["double_blocks.0.img_attn.proj.weight"]],
                  ["transformer_blocks.0.attn.norm_added_k.weight"]),
    ModelTemplate("sd3", False, [["transformer_blocks.0.attn.add_q_proj.weight"], ["joint_blocks.0.x_block.attn.qkv.weight"]],
                  ["transformer_blocks.0.attn.add_q_proj.weight"]),
    ModelTemplate("aura", False, [["double_layers.3.modX.1.weight"], ["joint_transformer_blocks.3.ff_context.out_projection.weight"]],
                  ["joint_transformer_blocks.3.ff_context.out_projection.weight"]),
    ModelTemplate("hidream", False, [["caption_projection.0.linear.weight", "double_stream_blocks.0.block.ff_i.shared_experts.w3.weight"]],
                  [], [".ff_i.gate.weight", "img_emb.emb_pos"]),
    ModelTemplate("cosmos", False, [["blocks.0.mlp.layer1.weight", "blocks.0.adaln_modulation_cross_attn.1.weight"]],
                  [], ["pos_embedder"], ["_extra_state", "accum_"]),
    ModelTemplate("hyvid", False, [["double_blocks.0.img_attn_proj.weight", "txt_in.individual_token_refiner.blocks.1.self_attn_qkv.weight"]]),
    ModelTemplate("wan", False, [["blocks.0.self_attn.norm_q.weight", "text_embedding.2.weight", "head.modulation"]], [], [".modulation"]),
    ModelTemplate("ltxv", False, [["adaln_single.emb.timestep_embedder.linear_2.weight", "transformer_blocks.27.scale_shift_table",
                                   "caption_projection.linear_2.weight"]], [], ["scale_shift_table"]),
    ModelTemplate("sdxl", True, [["down_blocks.0.downsamplers.0.conv.weight", "add_embedding.linear_1.weight"],
                                 ["input_blocks.3.0.op.weight", "input_blocks.6.0.op.weight", "output_blocks.2.2.conv.weight",
                                  "output_blocks.5.2.conv.weight"], ["label_emb.0.0.weight"]]),
    ModelTemplate("sd1", True, [["down_blocks.0.downsamplers.0.conv.weight"],
                                ["input_blocks.3.0.op.weight", "input_blocks.6.0.op.weight", "input_blocks.9.0.op.weight",
                                 "output_blocks.2.1.conv.weight", "output_blocks.5.2.conv.weight", "output_blocks.8.2.conv.weight"]]),
    ModelTemplate("lumina2", False, [["cap_embedder.1.weight", "context_refiner.0.attention.qkv.weight"]]),
]

_UNET_SKIP = ["class_embedding.*", "time_embedding.*", "add_embedding.*", "time_embed.*", "label_emb.*", "conv_in.*", "conv_out.*",
              "input_blocks.0.0.weight", "out.2.weight"]
ARCH_SKIP_PATTERNS = {
    "flux": ["txt_in.*", "img_in.*", "time_in.*", "vector_in.*", "guidance_in.*", "final_layer.*"],
    "sd1": _UNET_SKIP,
    "sdxl": _UNET_SKIP,
    "sd3": ["final_layer.*", "time_text_embed.*", "context_embedder.*", "t_embedder.*", "y_embedder.*", "x_embedder.*", "proj_out.weight",
            "pos_embed"],
    "aura": ["t_embedder.*", "init_x_linear.*", "modF.1.weight", "cond_seq_linear.weight", "final_linear.weight", "positional_encoding",
             "register_tokens"],
    "ltxv": ["adaln_single.*", "caption_projection.*", "patchify_proj.*", "proj_out.*", "*scale_shift_table*"],
    "hyvid": ["txt_in.*", "img_in.*", "time_in.*", "vector_in.*", "guidance_in.*", "final_layer.*"],
    "wan": ["*modulation.*", "patch_embedding.*", "text_embedding.*", "time_projection.*", "time_embedding.*", "img_emb.*", "head.*"],
    "hidream": ["p_embedder.*", "t_embedder.*", "x_embedder.*", "final_layer.*", "*.ff_i.gate.weight", "caption_projection.*"],
    "cosmos": ["p_embedder.*", "t_embedder.*", "t_embedding_norm.*", "x_embedder.*", "pos_embedder.*", "final_layer.*"],
    "lumina2": ["t_embedder.*", "x_embedder.*", "final_layer.*", "cap_embedder.*", "context_refiner.*", "noise_refiner.*"],
}

# Addition: decoder-only language models in the Hugging Face key layout.  Keys are kept as they are.
LLAMA_DETECT = ["model.layers.0.self_attn.q_proj.weight", "model.layers.0.mlp.down_proj.weight"]


@dataclass
class SourceTensor:
    source_key: str
    key: str
    dtype: str
    shape: list
    data_begin: int
    data_end: int


def parse_safetensors_header(path: str) -> list[SourceTensor]:
    size = os.path.getsize(path)
    if size < 8:
        fail("invalid safetensors file")
    with open(path, "rb") as f:
        (header_len,) = struct.unpack("<Q", f.read(8))
        if header_len > size - 8:
            fail("invalid safetensors header length")
        raw = f.read(header_len)
    data_start = 8 + header_len
    try:
        root = json.loads(raw.decode("utf-8"), object_pairs_hook=list)
    except (ValueError, UnicodeDecodeError):
        fail("invalid JSON: unsupported value")
    if not isinstance(root, list):
        fail("invalid safetensors header")
    tensors = []
    for name, info in root:
        if name == "__metadata__":
            continue
        entry = dict(info) if isinstance(info, list) else {}
        dtype, shape, offsets = entry.get("dtype"), entry.get("shape"), entry.get("data_offsets")
        if not isinstance(dtype, str) or not isinstance(shape, list) or not isinstance(offsets, list) or len(offsets) != 2:
            fail("invalid safetensors tensor entry for " + name)
        if any(not isinstance(d, int) or isinstance(d, bool) or d < 0 for d in shape):
            fail("invalid safetensors shape for " + name)
        if any(not isinstance(o, int) or isinstance(o, bool) or o < 0 for o in offsets):
            fail("invalid safetensors data_offsets for " + name)
        values = product_shape(shape)
        if dtype not in SOURCE_DTYPES:
            fail("unsupported source dtype: " + dtype)
        begin, end = data_start + offsets[0], data_start + offsets[1]
        if end < begin or end - begin != values * SOURCE_DTYPES[dtype][2]:
            fail("safetensors byte length does not match shape/dtype for " + name)
        if end > size:
            fail("safetensors byte range exceeds file size for " + name)
        tensors.append(SourceTensor(name, name, dtype, list(shape), begin, end))
    return tensors


def product_shape(shape) -> int:
    total = 1
    for dim in shape:
        if dim <= 0:
            fail("shape dimensions must be positive")
        total *= dim
    return total


def strip_prefix(tensors: list[SourceTensor]) -> list[SourceTensor]:
    for prefix in ("model.diffusion_model.", "model."):
        if any(t.key.startswith(prefix) for t in tensors):
            kept = [t for t in tensors if t.key.startswith(prefix)]
            for t in kept:
                t.key = t.key[len(prefix):]
            return kept
    if tensors and all(t.key.startswith("net.") for t in tensors):
        for t in tensors:
            t.key = t.key[4:]
    return tensors


def detect_arch(tensors: list[SourceTensor]) -> ModelTemplate:
    keys = {t.key for t in tensors}
    for model in MODEL_TEMPLATES:
        if any(all(k in keys for k in match) for match in model.keys_detect):
            if any(k in keys for k in model.keys_banned):
                fail("Model architecture not allowed for conversion; use the reference checkpoint key format")
            return model
    fail("Unknown model architecture")


# ---- policies -----------------------------------------------------------------------------------------------------
_ATTENTION_VALUE = ["*attn_v.weight*", "*.to_v.weight*", "*.v.weight*", "*.attn.w1v.weight*", "*.attn.w2v.weight*", "*_attn.v_proj.weight*"]
_FUSED_QKV = ["*attn_qkv.weight*", "*attn.qkv.weight*", "*attention.qkv.weight*"]
_FFN_DOWN = ["*ffn_down*", "*experts.*.w2.weight*", "*shared_experts.w2.weight*", "*.ffn.2.weight*", "*.ff.net.2.weight*",
             "*.mlp.layer2.weight*", "*.adaln_modulation_mlp.2.weight*", "*.feed_forward.w2.weight*"]
_ATTENTION_OUT = ["*.to_out.0.weight", "*.to_out.weight", "*.o_proj.weight", "*.out_proj.weight", "*.proj_out.weight", "*_attn.proj.weight"]
_ATTENTION_QKO = ["*.to_q.weight", "*.q_proj.weight", "*.query_proj.weight", "*_attn.q_proj.weight", "*attn_q.weight",
                  "*.to_k.weight", "*.k_proj.weight", "*.key_proj.weight", "*_attn.k_proj.weight", "*attn_k.weight"] + _ATTENTION_OUT
_FFN_UP_DOWN = _FFN_DOWN + ["*.mlp.linear_fc2.weight", "*.linear_fc2.weight", "*.down_proj.weight", "*.c_proj.weight",
                            "*.out_projection.weight", "*.mlp.up_proj.weight", "*.up_proj.weight", "*.w3.weight", "*.fc1.weight",
                            "*.linear_fc1.weight", "*.mlp.layer1.weight"]
_FFN = _FFN_UP_DOWN + ["*.mlp.gate_proj.weight", "*.gate_proj.weight", "*.w1.weight"]


def policy_allows_quant_shape(key: str, shape, model: ModelTemplate, policy: str) -> bool:
    if len(shape) != 2 or not key.endswith("weight"):
        return False
    if policy == "uniform":
        return True
    return not matches_any(key, ARCH_SKIP_PATTERNS.get(model.arch, []))


def mixed_policy_qtype(file_type: str, base: str, key: str, model: ModelTemplate, counters: dict) -> str:
    qtype = base
    if matches_any(key, _ATTENTION_VALUE):
        if file_type == "Q2_K":
            qtype = "Q3_K"
        elif file_type == "Q3_K_M":
            qtype = "Q5_K" if counters["attention_value"] < 2 else "Q4_K"
        elif file_type == "Q3_K_L":
            qtype = "Q5_K"
        elif file_type in ("Q4_K_M", "Q5_K_M"):
            qtype = "Q6_K"
        elif file_type == "Q4_K_S" and counters["attention_value"] < 4:
            qtype = "Q5_K"
        counters["attention_value"] += 1
    elif matches_any(key, _FUSED_QKV):
        if file_type in ("Q3_K_M", "Q3_K_L"):
            qtype = "Q4_K"
        elif file_type == "Q4_K_M":
            qtype = "Q5_K"
        elif file_type == "Q5_K_M":
            qtype = "Q6_K"
    elif matches_any(key, _FFN_DOWN):
        qtype = {"Q3_K_M": "Q4_K", "Q3_K_L": "Q5_K", "Q4_K_S": "Q5_K", "Q4_K_M": "Q6_K", "Q5_K_M": "Q6_K", "Q4_0": "Q4_1",
                 "Q5_0": "Q5_1"}.get(file_type, qtype)
        counters["ffn_down"] += 1
    elif model.arch == "aura" and file_type == "Q3_K_M" and fnmatch_case("double_layers.*.mlp?.c_proj.weight", key):
        qtype = "Q4_K"
    return qtype


def dynamic_policy_qtype(file_type: str, comfy: str, key: str, max_layer: int) -> str:
    layer = dynamic_layer_index(key)
    if layer < 0:
        return comfy
    early = layer <= 1
    final_tail = max_layer >= 0 and layer >= max_layer - 1
    low = file_type in ("Q2_K", "Q3_K_M", "Q4_K_M")
    if matches_any(key, _ATTENTION_VALUE):
        if file_type in ("Q2_K", "Q3_K_M", "Q3_K_L"):
            return "Q6_K"
        if file_type in ("Q4_K_S", "Q4_K_M", "Q5_K_S", "Q5_K_M"):
            return "Q8_0"
        return promote_k_qtype(comfy)
    if matches_any(key, _FUSED_QKV):
        return promote_k_qtype(comfy, 2 if early else 1)
    if matches_any(key, _ATTENTION_QKO):
        qtype = promote_k_qtype(comfy, 2 if early else 1)
        if matches_any(key, _ATTENTION_OUT):
            if low and (15 <= layer <= 24 or (layer >= 28 and not final_tail)):
                qtype = promote_k_qtype(qtype)
            elif file_type == "Q5_K_M" and (layer in (3, 24) or (layer >= 31 and not final_tail)):
                qtype = "Q8_0"
        return qtype
    if matches_any(key, _FFN):
        qtype = promote_k_qtype(comfy, 2 if early and file_type in ("Q4_K_M", "Q5_K_M") else 1)
        if matches_any(key, _FFN_UP_DOWN):
            if low and (layer in (7, 21) or (layer >= 23 and not final_tail)):
                qtype = promote_k_qtype(qtype)
            elif file_type == "Q5_K_M" and (layer == 7 or (layer >= 27 and not final_tail)):
                qtype = "Q8_0"
        return qtype
    return comfy


def llama_use_more_bits(layer: int, n_layers: int) -> bool:
    """llama.cpp's rule for the tensors that get the next-larger type in the *_M mixes: half of the layers."""
    return layer < n_layers // 8 or layer >= 7 * n_layers // 8 or (layer - n_layers // 8) % 3 == 2


def llama_policy_qtype(file_type: str, base: str, key: str, n_layers: int) -> str:
    if key in ("lm_head.weight", "output.weight"):
        return "Q6_K" if base in _K_ORDER[:4] else base
    if file_type in ("Q4_K_M", "Q5_K_M") and (key.endswith("self_attn.v_proj.weight") or key.endswith("mlp.down_proj.weight")):
        layer = dynamic_layer_index(key)
        if layer >= 0 and llama_use_more_bits(layer, n_layers):
            return "Q6_K"
    return base


# ---- planning -----------------------------------------------------------------------------------------------------
def parse_qtype(text: str, allow_extra: bool = True) -> tuple[str, str]:
    file_type = text.upper()
    if file_type == "Q8_K":
        fail("Q8_K output is not supported: this repo has metadata for Q8_K but no output quantizer")
    if file_type in EXTRA_BLOCK_SIZE:
        if not allow_extra or file_type not in EXTRA_FILE_TYPE_VALUE:
            fail("non-Q/K quantization families are not supported by this native executable yet")
        return file_type, file_type
    file_type = {"Q3_K": "Q3_K_M", "Q4_K": "Q4_K_M", "Q5_K": "Q5_K_M"}.get(file_type, file_type)
    tensor_qtype = file_type
    for prefix in ("Q3_K", "Q4_K", "Q5_K", "Q2_K"):
        if file_type.startswith(prefix + "_"):
            tensor_qtype = prefix
    if tensor_qtype not in BLOCK_SIZE or tensor_qtype in ("F32", "F16", "BF16"):
        fail("unsupported direct quantization type: " + text)
    if file_type not in FILE_TYPE_VALUE:
        fail("unsupported output file type: " + file_type)
    return file_type, tensor_qtype


def parse_tensor_qtype_name(text: str) -> str:
    name = text.upper()
    if name == "Q8_K":
        fail("Q8_K tensor output is not supported")
    name = {"Q3_K_S": "Q3_K", "Q3_K_M": "Q3_K", "Q3_K_L": "Q3_K", "Q4_K_S": "Q4_K", "Q4_K_M": "Q4_K", "Q5_K_S": "Q5_K",
            "Q5_K_M": "Q5_K", "Q2_K_S": "Q2_K"}.get(name, name)
    if name not in BLOCK_SIZE and name not in EXTRA_BLOCK_SIZE:
        fail("unsupported GGML tensor type: " + text)
    return name


def block_size_of(name: str) -> int:
    return BLOCK_SIZE.get(name) or EXTRA_BLOCK_SIZE[name]


def is_quantized(name: str) -> bool:
    return name not in ("F32", "F16", "BF16")


@dataclass
class TensorPlan:
    key: str
    source_dtype: str
    qtype: str
    source_shape: list
    write_shape: list
    data_begin: int
    data_end: int
    n_rows: int
    n_per_row: int
    nbytes: int


@dataclass
class Options:
    src: str
    qtype: str = "Q4_K_S"
    dst: str = ""
    policy: str = "comfy"
    tensor_overrides: list = field(default_factory=list)   # (pattern, type name)
    include: list = field(default_factory=list)
    exclude: list = field(default_factory=list)
    overwrite: bool = False
    gpus: int = 0                                            # 0 = all visible
    devices: tuple = ()                                      # explicit device list (--gpus 0,2 or LIBGGUF_CUDA_DEVICES); wins over gpus
    chunk_bytes: int = 128 << 20
    batch_bytes: int = 4 << 30
    timings: bool = False


def qtype_nbytes(shape, name: str) -> int:
    values = product_shape(shape)
    if values % block_size_of(name) != 0:
        fail("Tensor with incompatible shape cannot be stored as " + name)
    n_per_row = shape[-1] if shape else 1
    rs = row_size(int(Q[name]), n_per_row)
    if rs == 0:
        fail("unsupported qtype or row width for " + name)
    return values // n_per_row * rs


def prepare_plans(tensors, model: ModelTemplate, file_type: str, base: str, options: Options, kv: list, result: dict) -> list[TensorPlan]:
    plans = []
    counters = {"attention_value": 0, "ffn_down": 0}
    max_layer = max((dynamic_layer_index(t.key) for t in tensors), default=-1)
    for t in tensors:
        if contains_any(t.key, model.keys_ignore):
            continue
        if len(t.key.encode("utf-8")) > MAX_TENSOR_NAME_LENGTH:
            fail("Can only handle tensor names up to 127 characters: " + t.key)
        n_params = product_shape(t.shape)
        storage = "BF16" if t.dtype == "BF16" else "F16"
        if t.dtype in ("F32", "BF16") and (len(t.shape) == 1 or n_params <= QUANTIZATION_THRESHOLD or contains_any(t.key, model.keys_hiprec)):
            storage = "F32"
        write_shape = list(t.shape)
        if model.shape_fix and len(t.shape) > 1 and n_params >= REARRANGE_THRESHOLD and n_params % 256 == 0 and t.shape[-1] % 256 != 0:
            kv.append(("comfy.gguf.orig_shape." + t.key, T_ARRAY, (T_INT64, list(t.shape))))
            write_shape = [n_params // 256, 256]
        if model.arch == "llama":
            quantize = len(write_shape) == 2 and t.key.endswith("weight")
        else:
            quantize = policy_allows_quant_shape(t.key, write_shape, model, options.policy)
        if matches_any(t.key, options.include) and len(write_shape) == 2:
            quantize = True
        if matches_any(t.key, options.exclude):
            quantize = False
        target = storage
        forced = next((name for pattern, name in options.tensor_overrides if fnmatch_case(pattern, t.key)), "")
        if forced:
            target = parse_tensor_qtype_name(forced)
            quantize = is_quantized(target)
        elif quantize:
            target = base
            if model.arch == "llama":
                if options.policy != "uniform":
                    target = llama_policy_qtype(file_type, base, t.key, max_layer + 1)
            elif options.policy in ("comfy", "dynamic"):
                target = mixed_policy_qtype(file_type, base, t.key, model, counters)
                if options.policy == "dynamic":
                    target = dynamic_policy_qtype(file_type, target, t.key, max_layer)
        if quantize and is_quantized(target) and write_shape[-1] % block_size_of(target) != 0:
            result["fallbacks"][target] = result["fallbacks"].get(target, 0) + 1
            target, quantize = "F16", False
        n_per_row = write_shape[-1] if write_shape else 1
        plans.append(TensorPlan(t.key, t.dtype, target, list(t.shape), write_shape, t.data_begin, t.data_end,
                                product_shape(write_shape) // n_per_row, n_per_row, qtype_nbytes(write_shape, target)))
        result["tensor_types"][target] = result["tensor_types"].get(target, 0) + 1
    return plans


# ---- conversion ---------------------------------------------------------------------------------------------------
def default_output_path(src: str, file_type: str) -> str:
    slash = max(src.rfind("/"), src.rfind("\\"))
    dot = src.rfind(".")
    if dot < 0 or dot < slash:
        dot = len(src)
    return src[:dot] + "-" + file_type + ".gguf"


def plan_file(options: Options):
    """Everything up to the payload: returns (dst, file_type, model, kv, plans, result)."""
    file_type, base = parse_qtype(options.qtype)
    dst = options.dst or default_output_path(options.src, file_type)
    if os.path.isfile(dst) and not options.overwrite:
        fail("Output exists and overwriting is disabled: " + dst)
    if options.policy not in ("comfy", "dynamic", "uniform"):
        fail("--policy must be 'comfy', 'dynamic', or 'uniform'")
    try:
        tensors = parse_safetensors_header(options.src)
    except OSError as exc:
        fail(f"failed to open input file: {exc.strerror}")
    if all(k in {t.key for t in tensors} for k in LLAMA_DETECT):
        model = ModelTemplate("llama")
    else:
        tensors = strip_prefix(tensors)
        model = detect_arch(tensors)
    result = {"output_path": dst, "arch": model.arch, "file_type": "MOSTLY_" + file_type, "tensor_types": {}, "fallbacks": {}}
    value = FILE_TYPE_VALUE.get(file_type, EXTRA_FILE_TYPE_VALUE.get(file_type))
    kv = [("general.architecture", T_STRING, model.arch), ("general.quantization_version", T_UINT32, QUANT_VERSION),
          ("general.file_type", T_UINT32, value)]
    plans = prepare_plans(tensors, model, file_type, base, options, kv, result)
    return dst, file_type, model, kv, plans, result


class _PinnedArena:
    """A page-locked host buffer from the library (the GPUs copy from / to it directly), seen as a numpy byte array."""

    def __init__(self, lib, ctx, size: int):
        import ctypes
        self._lib, self._ctx, self._handle = lib, ctx, ctypes.c_void_p()
        if lib.libgguf_cuda_host_buffer_create(ctx, size, ctypes.byref(self._handle)) != 0:
            fail("cannot allocate pinned host memory: " + lib.libgguf_cuda_last_error(ctx).decode())
        pointer = ctypes.cast(lib.libgguf_cuda_host_buffer_data(self._handle), ctypes.POINTER(ctypes.c_ubyte))
        self.array = np.ctypeslib.as_array(pointer, shape=(size,))

    def close(self):
        if self._handle:
            self.array = None
            self._lib.libgguf_cuda_host_buffer_destroy(self._ctx, self._handle)
            self._handle = None


# The pinned arenas of the last conversion, kept for the next one in this process (page-locking a gigabyte takes a few
# tenths of a second, as long as the conversion of a small model): {"key": (device, size, pairs), "ctx": ..., "pairs": [...]}
_ARENA_CACHE: dict = {}


def _release_arena_cache() -> None:
    from ._native import lib
    for pair in _ARENA_CACHE.get("pairs", []):
        for arena in pair:
            arena.close()
    if _ARENA_CACHE.get("ctx"):
        lib.libgguf_cuda_context_destroy(_ARENA_CACHE["ctx"])
    _ARENA_CACHE.clear()


def _arenas(lib, device: int, size: int, pairs: int):
    """`pairs` (input, output) arena pairs of `size` bytes each, page-locked through a library context on `device`."""
    import atexit
    import ctypes
    key = (device, size, pairs)
    if _ARENA_CACHE.get("key") == key:
        return _ARENA_CACHE["pairs"]
    first_use = not _ARENA_CACHE
    _release_arena_cache()
    ctx = ctypes.c_void_p()
    if lib.libgguf_cuda_context_create(device, ctypes.byref(ctx)) != 0:
        fail("no CUDA device is available")
    _ARENA_CACHE.update(key=key, ctx=ctx, pairs=[])
    for _ in range(pairs):
        _ARENA_CACHE["pairs"].append((_PinnedArena(lib, ctx, size), _PinnedArena(lib, ctx, size)))
    if first_use:
        atexit.register(_release_arena_cache)
    return _ARENA_CACHE["pairs"]


def _align(n: int, to: int = 256) -> int:
    return (n + to - 1) // to * to


@dataclass
class _Piece:
    plan: TensorPlan
    row0: int
    rows: int
    last: bool      # last piece of its tensor: the alignment padding follows it

    @property
    def convert(self) -> bool:
        return self.plan.qtype != self.plan.source_dtype


def _pieces(plans, cap: int):
    """Row ranges of the tensors to convert, none larger than `cap` bytes on either side; other tensors stay whole."""
    for p in plans:
        if p.qtype == p.source_dtype:
            yield _Piece(p, 0, p.n_rows, True)
            continue
        row_in = p.n_per_row * SOURCE_DTYPES[p.source_dtype][2]
        row_out = p.nbytes // p.n_rows
        per = max(1, min(cap // row_in, cap // row_out))
        for row0 in range(0, p.n_rows, per):
            rows = min(per, p.n_rows - row0)
            yield _Piece(p, row0, rows, row0 + rows == p.n_rows)


def _batches(pieces, cap: int):
    """Consecutive pieces grouped so that their source bytes and their encoded bytes each fit `cap`."""
    batch, used_in, used_out = [], 0, 0
    for piece in pieces:
        p = piece.plan
        need_in = _align(piece.rows * p.n_per_row * SOURCE_DTYPES[p.source_dtype][2]) if piece.convert else 0
        need_out = _align(piece.rows * (p.nbytes // p.n_rows)) if piece.convert else 0
        if batch and (used_in + need_in > cap or used_out + need_out > cap):
            yield batch
            batch, used_in, used_out = [], 0, 0
        batch.append(piece)
        used_in += need_in
        used_out += need_out
    if batch:
        yield batch


def convert(options: Options) -> dict:
    """Runs the plan: row ranges of the source tensors are read from the file straight into pinned memory by a pool of
    reader threads (one batch ahead of the GPUs), encoded by the multi-GPU pipeline into pinned memory, and written out
    in plan order."""
    import ctypes
    from concurrent.futures import ThreadPoolExecutor

    import time

    from ._native import lib
    from .convert import ConversionPipeline, whole_tensor_imatrix   # needs the CUDA library; planning above does not

    clock = time.perf_counter
    began = clock()
    # wall-clock seconds of the calling thread per stage; the reads and the host<->device copies overlap the encode
    spent = {"metadata": 0.0, "setup": 0.0, "read": 0.0, "cuda_quant": 0.0, "write": 0.0, "close": 0.0}
    dst, _, _, kv, plans, result = plan_file(options)
    infos = [TensorInfo(p.key, tuple(p.write_shape), int(Q[p.qtype]), p.nbytes) for p in plans]
    head = header_bytes(kv, infos)
    spent["metadata"] = clock() - began
    source = np.memmap(options.src, dtype=np.uint8, mode="r")
    count = ctypes.c_int(0)
    if lib.libgguf_cuda_device_count(ctypes.byref(count)) != 0 or count.value < 1:
        fail("no CUDA device is available")
    devices = resolve_devices(options.gpus, options.devices, count.value)
    n_gpus = len(devices)
    # two pinned arenas per direction; large enough to keep every GPU's slots busy, small enough to allocate quickly
    cap = max(1 << 16, min(options.batch_bytes // 4, max(256 << 20, n_gpus * (128 << 20))))
    # a piece is at least one row: the arenas must hold the widest row of the plan on either side
    for p in plans:
        if p.qtype != p.source_dtype:
            cap = max(cap, _align(p.n_per_row * SOURCE_DTYPES[p.source_dtype][2]), _align(p.nbytes // p.n_rows))
    chunk = max(1 << 12, min(options.chunk_bytes, cap // (3 * n_gpus)))
    fd, out_fd = os.open(options.src, os.O_RDONLY), -1
    readers = ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1))
    writers = ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1))
    READ_PIECE = 16 << 20
    # where every tensor's bytes go in the output file: known before anything is encoded, so finished pieces are
    # written at their place by a pool of writer threads while the GPUs work on the next batch
    data_start = pad_to(len(head))
    tensor_at, at = {}, data_start
    for p in plans:
        tensor_at[p.key] = at
        at += pad_to(p.nbytes)
    file_size = at

    # The output is written through a shared mapping: writer threads copy finished pieces to their place, so the
    # pages of a new file are allocated by all of them at once (write() calls on one file take turns on its lock:
    # 1.8 GB to a RAM-backed file system took 0.36 s with eight threads calling pwrite).  A file system that is too
    # full is an OSError before anything is written (free space is checked first) or from the reservation that runs
    # beside the first batches (posix_fallocate on a thread of its own); waiting for the reservation before the first
    # copy cost 0.1 s, since it touches every page once by itself.
    out_map = None
    reserved = None

    def reserve():
        import errno
        try:
            os.posix_fallocate(out_fd, 0, file_size)
        except OSError as e:
            if e.errno not in (errno.EOPNOTSUPP, errno.EINVAL, errno.ENOSYS):
                raise

    def write_at(view, file_offset: int):
        buffer = memoryview(view).cast("B")
        if out_map is not None:
            out_map[file_offset:file_offset + len(buffer)] = np.frombuffer(buffer, np.uint8)
            return
        done, total = 0, len(buffer)
        while done < total:
            done += os.pwrite(out_fd, buffer[done:total], file_offset + done)

    def read_into(view: np.ndarray, file_offset: int):
        done, total = 0, view.size
        buffer = memoryview(view)
        while done < total:
            got = os.preadv(fd, [buffer[done:total]], file_offset + done)
            if got <= 0:
                fail("unexpected end of input file")
            done += got

    def stage(batch, arena_pair):
        """Starts the reads of one batch; returns (entries for the pipeline, output view per piece, futures)."""
        arena_in, arena_out = arena_pair
        entries, outputs, futures, at_in, at_out = [], [], [], 0, 0
        for piece in batch:
            if not piece.convert:
                outputs.append(None)
                continue
            p = piece.plan
            np_dtype, _, esize = SOURCE_DTYPES[p.source_dtype]
            nbytes_in, nbytes_out = piece.rows * p.n_per_row * esize, piece.rows * (p.nbytes // p.n_rows)
            file_at = p.data_begin + piece.row0 * p.n_per_row * esize
            raw = arena_in.array[at_in:at_in + nbytes_in]
            for start in range(0, nbytes_in, READ_PIECE):
                futures.append(readers.submit(read_into, raw[start:min(start + READ_PIECE, nbytes_in)], file_at + start))
            enc = arena_out.array[at_out:at_out + nbytes_out]
            entries.append((int(Q[p.qtype]), raw.view(np_dtype).reshape(piece.rows, p.n_per_row), split_weights.get(p.key), enc))
            outputs.append(enc)
            at_in += _align(nbytes_in)
            at_out += _align(nbytes_out)
        return entries, outputs, futures

    counts = {"cuda_chunks": 0, "cuda_max_input": 0, "cuda_max_output": 0}
    split_weights: dict[str, np.ndarray] = {}
    finished = False
    try:
        out_fd = os.open(dst, os.O_RDWR | os.O_CREAT | os.O_TRUNC, 0o644)
        room = os.fstatvfs(out_fd)
        if room.f_blocks > 0 and room.f_bavail * room.f_frsize < file_size:   # (a file system that reports no sizes is not judged)
            import errno
            raise OSError(errno.ENOSPC, f"{dst}: {file_size} bytes needed, {room.f_bavail * room.f_frsize} free")
        os.ftruncate(out_fd, file_size)       # the padding between tensors is the zeros of the extended file
        reserved = writers.submit(reserve)
        try:
            out_map = np.memmap(dst, dtype=np.uint8, mode="r+", shape=(file_size,))
        except (OSError, ValueError):
            out_map = None                    # a file system without shared mappings: positioned writes
        pieces = list(_pieces(plans, cap))
        # A type that needs importance weights derives them from the WHOLE tensor (upstream compute_auto_imatrix,
        # csrc/_libgguf_module.cpp:1210-1242).  A tensor that goes through in one piece gets them inside the pipeline;
        # one that was cut gets them here, once, from the mapped source, and every piece is encoded with them, so the
        # bytes do not depend on --gpus or --batch-mb.
        for piece in pieces:
            p = piece.plan
            if piece.convert and not (piece.row0 == 0 and piece.last) and p.key not in split_weights \
                    and lib.libgguf_quantize_requires_imatrix(int(Q[p.qtype])):
                np_dtype = SOURCE_DTYPES[p.source_dtype][0]
                whole = source[p.data_begin:p.data_end].view(np_dtype).reshape(p.n_rows, p.n_per_row)
                split_weights[p.key] = whole_tensor_imatrix(whole)
        batches = list(_batches(pieces, cap))
        arenas = _arenas(lib, devices[0], cap + 4096, 2)
        head_written = writers.submit(write_at, head, 0)   # behind the reservation, like every other write
        writes = [[], []]                      # write futures of the batch that last used each arena pair
        with ConversionPipeline(devices, slots=3, chunk_bytes=chunk) as pipe:
            staged = stage(batches[0], arenas[0]) if batches else None
            spent["setup"] = clock() - began - spent["metadata"]   # devices, arenas, pipeline, output file
            for i, batch in enumerate(batches):
                entries, outputs, futures = staged
                t0 = clock()
                for f in futures:
                    f.result()
                t1 = clock()
                if i + 1 < len(batches):   # the next batch's reads run while this one is encoded and written
                    staged = stage(batches[i + 1], arenas[(i + 1) & 1])
                for f in writes[i & 1]:    # this pair's output arena is free once batch i - 2 has reached the file
                    f.result()
                t2 = clock()
                if entries:
                    pipe.quantize(entries)
                t3 = clock()
                writes[i & 1] = []
                for piece, enc in zip(batch, outputs):
                    p = piece.plan
                    data = enc if enc is not None else source[p.data_begin:p.data_end]
                    base = tensor_at[p.key] + piece.row0 * (p.nbytes // p.n_rows)
                    for start in range(0, len(data), READ_PIECE):
                        writes[i & 1].append(writers.submit(write_at, data[start:min(start + READ_PIECE, len(data))], base + start))
                spent["read"] += t1 - t0
                spent["write"] += t2 - t1
                spent["cuda_quant"] += t3 - t2
                for entry in entries:
                    counts["cuda_chunks"] += 1
                    counts["cuda_max_input"] = max(counts["cuda_max_input"], entry[1].nbytes)
                    counts["cuda_max_output"] = max(counts["cuda_max_output"], entry[3].nbytes)
            t4 = clock()
            for pending in writes:
                for f in pending:
                    f.result()
            head_written.result()
            reserved.result()
            spent["write"] += clock() - t4
            t5 = clock()
        spent["close"] = clock() - t5   # the pipeline's streams and buffers
        finished = True
    finally:
        readers.shutdown(wait=True)
        writers.shutdown(wait=True)
        out_map = None   # unmaps; the dirty pages belong to the file
        os.close(fd)
        if out_fd >= 0:
            os.close(out_fd)
        if not finished:   # never leave a half-written file behind
            try:
                os.unlink(dst)
            except OSError:
                pass
    result["timings"] = dict(spent, total=clock() - began, tensors=len(plans), cuda_tensors=sum(1 for p in plans if p.qtype != p.source_dtype),
                             threads=min(16, os.cpu_count() or 1), scratch=cap, cuda_vram=chunk, **counts)
    return result


def timings_line(result: dict) -> str:
    """The stderr line of upstream's --timings (csrc/quantize_gguf.cpp:2527-2547), same tokens in the same order.  The
    reads, the host<->device copies and the encode overlap here: `read` is the time the writer waited for source
    bytes, `cuda_quant` the time it waited for the GPUs (copies included, hence h2d = d2h = 0), nothing is converted
    on the CPU and nothing is verified against a second backend."""
    t = result["timings"]
    return ("Timings: total=%.3fs metadata=%.3fs read=%.3fs cpu_convert=%.3fs h2d=%.3fs cuda_quant=%.3fs d2h=%.3fs write=%.3fs "
            "tensors=%d cuda_tensors=%d cuda_verified=%d cuda_chunks=%d threads=%d scratch=%d cuda_vram=%d cuda_pipeline=%d "
            "cuda_max_input=%d cuda_max_output=%d" % (
                t["total"], t["metadata"], t["read"], 0.0, 0.0, t["cuda_quant"], 0.0, t["write"], t["tensors"], t["cuda_tensors"], 0,
                t["cuda_chunks"], t["threads"], t["scratch"], t["cuda_vram"], 1, t["cuda_max_input"], t["cuda_max_output"]))


def summary_lines(result: dict) -> list[str]:
    lines = [f"Wrote {result['output_path']}", f"Architecture: {result['arch']}", f"File type: {result['file_type']}",
             "Tensor types: " + ", ".join(f"{k}={v}" for k, v in sorted(result["tensor_types"].items()))]
    if result["fallbacks"]:
        lines.append("Fallbacks: " + ", ".join(f"{k}={v}" for k, v in sorted(result["fallbacks"].items())))
    return lines


def parse_device_spec(text: str) -> tuple[int, tuple]:
    """'--gpus' / LIBGGUF_CUDA_DEVICES value -> (count, explicit device list): '4' -> (4, ()), '0,2,3' -> (0, (0, 2, 3)).
    A single number is a count; a list (a trailing comma makes one: '2,') names devices."""
    text = text.strip()
    if not text:
        return 0, ()
    try:
        if "," in text:
            devices = tuple(int(t) for t in text.split(",") if t.strip())
            if not devices or any(d < 0 for d in devices) or len(set(devices)) != len(devices):
                raise ValueError
            return 0, devices
        n = int(text)
        if n < 0:
            raise ValueError
        return n, ()
    except ValueError:
        fail(f"invalid GPU selection '{text}': expected a count or a comma-separated list of distinct device numbers")


def resolve_devices(gpus: int, devices: tuple, visible: int) -> list[int]:
    """The device list a conversion uses, given the number of visible CUDA devices."""
    if devices:
        bad = [d for d in devices if d >= visible]
        if bad:
            fail(f"CUDA device {bad[0]} requested, but only {visible} device(s) are visible")
        return list(devices)
    if gpus > visible:
        fail(f"{gpus} GPUs requested, but only {visible} device(s) are visible")
    return list(range(gpus if gpus > 0 else visible))


def parse_args(argv) -> Options:
    ap = argparse.ArgumentParser(prog="libgguf_b200.quantize_gguf", description="safetensors -> GGUF on the GPU pipeline")
    ap.add_argument("--src", required=True)
    ap.add_argument("--qtype", default="Q4_K_S")
    ap.add_argument("--dst", default="")
    ap.add_argument("--overwrite", action="store_true")
    ap.add_argument("--policy", default="comfy", choices=["comfy", "dynamic", "uniform"])
    ap.add_argument("--tensor-type", action="append", default=[], metavar="PATTERN=TYPE")
    ap.add_argument("--include", action="append", default=[])
    ap.add_argument("--exclude", action="append", default=[])
    # options of upstream's command that choose how its own CPU / single-GPU loop runs: accepted so that existing command
    # lines keep working; the ones with an equivalent here are mapped, the rest have nothing to configure
    ap.add_argument("--imatrix", default="", help="accepted for command line parity; the Q/K quantizers do not use it")
    ap.add_argument("--scratch-bytes", "--cpu-ram-bytes", dest="scratch_bytes", type=int, default=0, help="ignored (no CPU loop)")
    ap.add_argument("--threads", type=int, default=0, help="ignored (no CPU loop)")
    ap.add_argument("--backend", default="auto", choices=["auto", "cuda", "cpu"], help="'cpu' is refused: there is no CPU path")
    ap.add_argument("--cuda-fallback", default="", help="ignored (every type is supported on the GPU)")
    ap.add_argument("--verify-cuda-tensors", default="", help="ignored (parity is a test-suite matter here)")
    ap.add_argument("--verify-cuda-large-tensors", default="", help="ignored")
    ap.add_argument("--verify-cuda-random-tensors", default="", help="ignored")
    ap.add_argument("--seed", default="", help="ignored")
    ap.add_argument("--cuda-vram-bytes", type=int, default=0, help="largest shard in bytes (same as --chunk-mb)")
    ap.add_argument("--cuda-batch-mb", type=int, default=0, help="largest shard in MiB (same as --chunk-mb)")
    ap.add_argument("--cuda-pipeline", default="1", help="ignored (always pipelined)")
    ap.add_argument("--timings", action="store_true", help="print the wall-clock time of the conversion to stderr")
    ap.add_argument("--gpus", default="", help="GPUs to stream through: a count N (devices 0..N-1) or a comma-separated device "
                    "list such as 0,2,3 (default: the list in LIBGGUF_CUDA_DEVICES, else all visible devices)")
    ap.add_argument("--chunk-mb", type=int, default=128, help="largest shard, MiB of source bytes")
    ap.add_argument("--batch-mb", type=int, default=4096, help="host memory held between file writes, MiB")
    a = ap.parse_args(argv)
    gpu_count, gpu_list = parse_device_spec(str(a.gpus) if str(a.gpus).strip() else os.environ.get("LIBGGUF_CUDA_DEVICES", ""))
    if a.backend == "cpu":
        fail("CPU backend requested, but this converter encodes on CUDA devices only")
    if a.cuda_vram_bytes > 0:
        a.chunk_mb = max(1, a.cuda_vram_bytes >> 20)
    if a.cuda_batch_mb > 0:
        a.chunk_mb = a.cuda_batch_mb
    overrides = []
    for item in a.tensor_type:
        pattern, eq, name = item.partition("=")
        if not eq or not pattern or not name:
            fail("expected PATTERN=QTYPE for --tensor-type")
        overrides.append((pattern, parse_tensor_qtype_name(name)))
    return Options(src=a.src, qtype=a.qtype, dst=a.dst, policy=a.policy, tensor_overrides=overrides, include=a.include,
                   exclude=a.exclude, overwrite=a.overwrite, gpus=gpu_count, devices=gpu_list, chunk_bytes=a.chunk_mb << 20, batch_bytes=a.batch_mb << 20,
                   timings=a.timings)


def main(argv=None) -> int:
    try:
        options = parse_args(sys.argv[1:] if argv is None else argv)
        result = convert(options)
        if options.timings:
            print(timings_line(result), file=sys.stderr)
    except ConversionError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    print("\n".join(summary_lines(result)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
