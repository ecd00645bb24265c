"""Seeded synthetic checkpoint with the tensor names and shapes of Qwen3-TTS VoiceDesign.

There is no real checkpoint on the machines this runs on, so benchmarks and tests load
random weights of the exact architecture the library validates at finalize (404 tensors,
the names of the reference's talker.cu:495-562 and :704-747).  Decode matrices are drawn as
int8-valued rows times a per-row scale, scale ~ U(0.5, 1.5) / (73.6 * sqrt(K)), so that a
unit-RMS input gives a roughly unit-RMS output and hidden states stay O(1) through 28 layers
(73.6 is the RMS of a uniform integer in [-127, 127]).  Norm weights are 1 + 0.02 N(0,1),
embeddings and biases 0.02 N(0,1).  Values never influence timing.
"""
from __future__ import annotations

import zlib
from typing import Dict, Iterator, Tuple

import numpy as np
import torch

TALKER_LAYERS = 28
PREDICTOR_LAYERS = 5
H = 2048
I = 6144
VOCAB = 3072
TEXT_VOCAB = 151936
PH = 1024
PI = 3072
PVOCAB = 2048
GROUPS = 15


def tensor_shapes(predictor_head_dim: int = 128) -> Dict[str, Tuple[int, ...]]:
    """name -> shape for all 404 tensors."""
    shapes: Dict[str, Tuple[int, ...]] = {}

    def layer(prefix, hidden, inter, qw, kvw, hd):
        shapes[prefix + ".input_layernorm.weight"] = (hidden,)
        shapes[prefix + ".self_attn.q_proj.weight"] = (qw, hidden)
        shapes[prefix + ".self_attn.k_proj.weight"] = (kvw, hidden)
        shapes[prefix + ".self_attn.v_proj.weight"] = (kvw, hidden)
        shapes[prefix + ".self_attn.o_proj.weight"] = (hidden, qw)
        shapes[prefix + ".self_attn.q_norm.weight"] = (hd,)
        shapes[prefix + ".self_attn.k_norm.weight"] = (hd,)
        shapes[prefix + ".post_attention_layernorm.weight"] = (hidden,)
        shapes[prefix + ".mlp.gate_proj.weight"] = (inter, hidden)
        shapes[prefix + ".mlp.up_proj.weight"] = (inter, hidden)
        shapes[prefix + ".mlp.down_proj.weight"] = (hidden, inter)

    shapes["talker.model.codec_embedding.weight"] = (VOCAB, H)
    shapes["talker.model.text_embedding.weight"] = (TEXT_VOCAB, H)
    shapes["talker.text_projection.linear_fc1.weight"] = (H, H)
    shapes["talker.text_projection.linear_fc1.bias"] = (H,)
    shapes["talker.text_projection.linear_fc2.weight"] = (H, H)
    shapes["talker.text_projection.linear_fc2.bias"] = (H,)
    shapes["talker.model.norm.weight"] = (H,)
    shapes["talker.codec_head.weight"] = (VOCAB, H)
    for l in range(TALKER_LAYERS):
        layer(f"talker.model.layers.{l}", H, I, 2048, 1024, 128)
    shapes["talker.code_predictor.small_to_mtp_projection.weight"] = (PH, H)
    shapes["talker.code_predictor.small_to_mtp_projection.bias"] = (PH,)
    shapes["talker.code_predictor.model.norm.weight"] = (PH,)
    hd = predictor_head_dim
    for l in range(PREDICTOR_LAYERS):
        layer(f"talker.code_predictor.model.layers.{l}", PH, PI, 16 * hd, 8 * hd, hd)
    for g in range(GROUPS):
        shapes[f"talker.code_predictor.model.codec_embedding.{g}.weight"] = (PVOCAB, H)
        shapes[f"talker.code_predictor.lm_head.{g}.weight"] = (PVOCAB, PH)
    return shapes


def _kind(name: str) -> str:
    if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        return "norm"
    if name.endswith(".bias") or "embedding" in name:
        return "small"
    return "matrix"


def make_tensor(name: str, shape: Tuple[int, ...], seed: int = 0, exact_int8: bool = False) -> np.ndarray:
    """bf16 bit patterns (uint16) of one tensor; depends only on (name, shape, seed, exact_int8).

    exact_int8: every decode matrix is int8-representable as a bf16 tensor: row = q * 2^e with
    integer q in [-127, 127], one |q| = 127 per row and a power-of-two scale.  The per-row int8
    quantizer (scale = absmax / 127, q = round(w / scale)) then returns exactly q and 2^e, so a bf16
    GEMM over the tensor and an int8 GEMM over its quantized form multiply the same numbers."""
    g = torch.Generator()
    g.manual_seed((zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF)
    kind = _kind(name)
    if kind == "norm":
        t = 1.0 + 0.02 * torch.randn(shape, generator=g)
    elif kind == "small":
        t = 0.02 * torch.randn(shape, generator=g)
    else:
        rows, cols = shape
        q = torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)
        if exact_int8:
            q[:, 0] = 127
            exponent = torch.round(torch.log2((0.5 + torch.rand((rows, 1), generator=g))
                                              / (73.6 * float(cols) ** 0.5)))
            scale = torch.pow(2.0, exponent)
        else:
            scale = (0.5 + torch.rand((rows, 1), generator=g)) / (73.6 * float(cols) ** 0.5)
        t = q.to(torch.float32) * scale
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def checkpoint_cuda(device: int, seed: int = 0,
                    predictor_head_dim: int = 128) -> Iterator[Tuple[str, np.ndarray]]:
    """Same distributions as checkpoint(), drawn with the GPU's generator (seconds instead of
    a minute on a busy host; values differ from checkpoint()'s).  For benchmarks only: tests
    that compare against the oracle use checkpoint(), whose values do not depend on the GPU."""
    dev = torch.device("cuda", device)
    g = torch.Generator(device=dev)
    for name, shape in tensor_shapes(predictor_head_dim).items():
        g.manual_seed((zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF)
        kind = _kind(name)
        if kind == "norm":
            t = 1.0 + 0.02 * torch.randn(shape, generator=g, device=dev)
        elif kind == "small":
            t = 0.02 * torch.randn(shape, generator=g, device=dev)
        else:
            rows, cols = shape
            q = torch.randint(-127, 128, shape, generator=g, device=dev, dtype=torch.int8)
            scale = (0.5 + torch.rand((rows, 1), generator=g, device=dev)) / (73.6 * float(cols) ** 0.5)
            t = q.to(torch.float32) * scale
        yield name, t.to(torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)


def checkpoint(seed: int = 0, predictor_head_dim: int = 128,
               exact_int8: bool = False) -> Iterator[Tuple[str, np.ndarray]]:
    """Yields (name, bf16 bits) for all 404 tensors, one at a time (about 3.8 GB in total)."""
    for name, shape in tensor_shapes(predictor_head_dim).items():
        yield name, make_tensor(name, shape, seed, exact_int8)
