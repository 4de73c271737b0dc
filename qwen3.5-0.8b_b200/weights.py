"""Seeded random-init weights of the Qwen3.5-0.8B text tower (+ MTP block).

The tensor names and shapes are the checkpoint's, i.e. the ones the reference's
torch implementation looks up (speccheck/specimpl.py:92-127, speccheck/mtp.py:33,65-77),
so one dict feeds the reference, the CPU oracle and the device engine alike.

Distributions (the benchmark's synthetic stand-in for the real checkpoint):
linear / embedding weights N(0, 0.02); every RMSNorm weight 1.0; A_log = log(U[1,16]);
dt_bias ~ U[-4,-2]; conv1d weights N(0, 0.1).  Everything is rounded to bf16 once,
because the reference holds all parameters in bf16 (speccheck/specimpl.py:85).

Each tensor has its own generator seeded from (seed, crc32(name)), so a single layer
can be produced without generating the 1.5 GB model.
"""
from __future__ import annotations

import zlib

import torch

D_MODEL = 1024
N_LAYERS = 24
N_Q, N_KV, D_HEAD = 8, 2, 256
D_FF = 3584
VOCAB = 248320
H_V = 16
D_K = D_V = 128
K_CONV = 4
KEY_DIM = H_V * D_K          # 2048
VAL_DIM = H_V * D_V          # 2048
CONV_CH = 2 * KEY_DIM + VAL_DIM   # 6144
Q_WIDTH = N_Q * D_HEAD       # 2048
QPROJ_WIDTH = 2 * Q_WIDTH    # 4096
KV_WIDTH = N_KV * D_HEAD     # 512
LM = "model.language_model."
MTP = "mtp."


def is_attn_layer(l: int) -> bool:
    """Full attention at layers 3, 7, ..., 23 (engine/state.h:67)."""
    return l % 4 == 3


GDN_LAYERS = [l for l in range(N_LAYERS) if not is_attn_layer(l)]
ATTN_LAYERS = [l for l in range(N_LAYERS) if is_attn_layer(l)]


def _attn_block(pre: str) -> dict:
    return {
        pre + "self_attn.q_proj.weight": ("lin", (QPROJ_WIDTH, D_MODEL)),
        pre + "self_attn.k_proj.weight": ("lin", (KV_WIDTH, D_MODEL)),
        pre + "self_attn.v_proj.weight": ("lin", (KV_WIDTH, D_MODEL)),
        pre + "self_attn.q_norm.weight": ("one", (D_HEAD,)),
        pre + "self_attn.k_norm.weight": ("one", (D_HEAD,)),
        pre + "self_attn.o_proj.weight": ("lin", (D_MODEL, Q_WIDTH)),
    }


def _mlp_block(pre: str) -> dict:
    return {
        pre + "mlp.gate_proj.weight": ("lin", (D_FF, D_MODEL)),
        pre + "mlp.up_proj.weight": ("lin", (D_FF, D_MODEL)),
        pre + "mlp.down_proj.weight": ("lin", (D_MODEL, D_FF)),
    }


def layer_spec(l: int) -> dict:
    """name -> (kind, shape) for one text-tower layer."""
    pre = f"{LM}layers.{l}."
    spec = {
        pre + "input_layernorm.weight": ("one", (D_MODEL,)),
        pre + "post_attention_layernorm.weight": ("one", (D_MODEL,)),
    }
    spec.update(_mlp_block(pre))
    if is_attn_layer(l):
        spec.update(_attn_block(pre))
    else:
        spec.update({
            pre + "linear_attn.in_proj_qkv.weight": ("lin", (CONV_CH, D_MODEL)),
            pre + "linear_attn.in_proj_z.weight": ("lin", (VAL_DIM, D_MODEL)),
            pre + "linear_attn.in_proj_b.weight": ("lin", (H_V, D_MODEL)),
            pre + "linear_attn.in_proj_a.weight": ("lin", (H_V, D_MODEL)),
            pre + "linear_attn.conv1d.weight": ("conv", (CONV_CH, 1, K_CONV)),
            pre + "linear_attn.A_log": ("alog", (H_V,)),
            pre + "linear_attn.dt_bias": ("dtb", (H_V,)),
            pre + "linear_attn.norm.weight": ("one", (D_V,)),
            pre + "linear_attn.out_proj.weight": ("lin", (D_MODEL, VAL_DIM)),
        })
    return spec


def mtp_spec() -> dict:
    pre = MTP + "layers.0."
    spec = {
        MTP + "fc.weight": ("lin", (D_MODEL, 2 * D_MODEL)),
        MTP + "pre_fc_norm_embedding.weight": ("one", (D_MODEL,)),
        MTP + "pre_fc_norm_hidden.weight": ("one", (D_MODEL,)),
        MTP + "norm.weight": ("one", (D_MODEL,)),
        pre + "input_layernorm.weight": ("one", (D_MODEL,)),
        pre + "post_attention_layernorm.weight": ("one", (D_MODEL,)),
    }
    spec.update(_attn_block(pre))
    spec.update(_mlp_block(pre))
    return spec


def top_spec(vocab: int = VOCAB) -> dict:
    return {
        LM + "embed_tokens.weight": ("lin", (vocab, D_MODEL)),
        LM + "norm.weight": ("one", (D_MODEL,)),
    }


def full_spec(vocab: int = VOCAB, layers=None, mtp: bool = True) -> dict:
    spec = top_spec(vocab)
    for l in (range(N_LAYERS) if layers is None else layers):
        spec.update(layer_spec(l))
    if mtp:
        spec.update(mtp_spec())
    return spec


def make_tensor(name: str, kind: str, shape, seed: int = 0) -> torch.Tensor:
    """One bf16 parameter, reproducible from (seed, name) alone."""
    g = torch.Generator(device="cpu")
    g.manual_seed((seed << 32) ^ zlib.crc32(name.encode()))
    if kind == "one":
        t = torch.ones(shape, dtype=torch.float32)
    elif kind == "lin":
        t = torch.empty(shape, dtype=torch.float32).normal_(0.0, 0.02, generator=g)
    elif kind == "conv":
        t = torch.empty(shape, dtype=torch.float32).normal_(0.0, 0.1, generator=g)
    elif kind == "alog":
        t = torch.empty(shape, dtype=torch.float32).uniform_(1.0, 16.0, generator=g).log()
    elif kind == "dtb":
        t = torch.empty(shape, dtype=torch.float32).uniform_(-4.0, -2.0, generator=g)
    else:
        raise ValueError(kind)
    return t.to(torch.bfloat16)


def make_weights(seed: int = 0, vocab: int = VOCAB, layers=None, mtp: bool = True) -> dict:
    """dict name -> bf16 CPU tensor for the whole model (or the `layers` subset)."""
    return {n: make_tensor(n, k, s, seed) for n, (k, s) in full_spec(vocab, layers, mtp).items()}
