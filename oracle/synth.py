"""Seeded synthetic checkpoints and inputs with the shapes of a converted Pi0 / Pi05 checkpoint.

TEST INFRASTRUCTURE ONLY (see vla_oracle.py).  Real checkpoints, camera frames and the tokenizer are
not available offline, so every benchmark configuration is stood in for by seeded random tensors:
weights bf16 N(0, 0.02) drawn in dict order from torch.Generator().manual_seed(seed), LayerNorm
scales 1 / shifts 0, Pi05 timestep table sinusoidal.  Key names and shapes follow
pi0_infer.py:1245-1287 and pi05_infer.py:563-611 of the reference.
"""
from __future__ import annotations

import torch

from .vla_oracle import sincos_time_table

BF16 = torch.bfloat16


def vision_shapes(nl=27):
    return {
        "vision_patch_embedding_w": (14, 14, 3, 1152),
        "vision_patch_embedding_b": (1152,),
        "vision_position_embedding": (256, 1152),
        "vision_attn_qkv_w": (nl, 1152, 3456),
        "vision_attn_qkv_b": (nl, 3456),
        "vision_attn_o_w": (nl, 1152, 1152),
        "vision_attn_o_b": (nl, 1152),
        "vision_ffn_up_w": (nl, 1152, 4304),
        "vision_ffn_up_b": (nl, 4304),
        "vision_ffn_down_w": (nl, 4304, 1152),
        "vision_ffn_down_b": (nl, 1152),
        "vision_pre_attn_norm_w": (nl, 1152),
        "vision_pre_attn_norm_b": (nl, 1152),
        "vision_pre_ffn_norm_w": (nl, 1152),
        "vision_pre_ffn_norm_b": (nl, 1152),
        "vision_final_norm_w": (1152,),
        "vision_final_norm_b": (1152,),
    }


def encoder_shapes(nl=18):
    return {
        "encoder_multi_modal_projector_w": (1152, 2048),
        "encoder_multi_modal_projector_b": (2048,),
        "encoder_attn_qkv_w": (nl, 2048, 2560),
        "encoder_attn_o_w": (nl, 2048, 2048),
        "encoder_ffn_gate_w": (nl, 2048, 16384),
        "encoder_ffn_up_w": (nl, 2048, 16384),
        "encoder_ffn_down_w": (nl, 16384, 2048),
    }


def pi0_decoder_shapes(nl=18):
    return {
        "decoder_state_in_proj_w": (32, 1024),
        "decoder_state_in_proj_b": (1024,),
        "decoder_action_fused_in_proj_w": (32, 1024),
        "decoder_action_fused_time_biases": (10, 1024),
        "decoder_action_mlp_w": (1024, 1024),
        "decoder_action_mlp_b": (1024,),
        "decoder_attn_qkv_w": (nl, 1024, 2560),
        "decoder_attn_o_w": (nl, 2048, 1024),
        "decoder_ffn_gate_w": (nl, 1024, 4096),
        "decoder_ffn_up_w": (nl, 1024, 4096),
        "decoder_ffn_down_w": (nl, 4096, 1024),
        "decoder_action_fused_out_proj_w": (1024, 32),
        "decoder_action_fused_out_proj_b": (32,),
    }


def pi05_decoder_shapes(nl=18):
    return {
        "decoder_time_embeds": (10, 1024),
        "decoder_time_mlp_in_w": (1024, 1024),
        "decoder_time_mlp_in_b": (1024,),
        "decoder_time_mlp_out_w": (1024, 1024),
        "decoder_time_mlp_out_b": (1024,),
        "decoder_action_in_proj_w": (32, 1024),
        "decoder_action_in_proj_b": (1024,),
        "decoder_pre_attn_norm_mod_w": (nl, 1024, 3072),
        "decoder_pre_attn_norm_mod_b": (nl, 3072),
        "decoder_pre_ffn_norm_mod_w": (nl, 1024, 3072),
        "decoder_pre_ffn_norm_mod_b": (nl, 3072),
        "decoder_attn_qkv_w": (nl, 1024, 2560),
        "decoder_attn_o_w": (nl, 2048, 1024),
        "decoder_ffn_gate_w": (nl, 1024, 4096),
        "decoder_ffn_up_w": (nl, 1024, 4096),
        "decoder_ffn_down_w": (nl, 4096, 1024),
        "decoder_action_out_proj_w": (1024, 32),
        "decoder_action_out_proj_b": (32,),
        "decoder_final_norm_mod_w": (1024, 3072),
        "decoder_final_norm_mod_b": (3072,),
    }


def _fill(shapes, gen, std=0.02):
    out = {}
    for k, shp in shapes.items():
        if k.endswith("_norm_w"):
            out[k] = torch.ones(shp, dtype=BF16)
        elif k.endswith("_norm_b"):
            out[k] = torch.zeros(shp, dtype=BF16)
        elif k == "decoder_time_embeds":
            out[k] = sincos_time_table(shp[0])
        else:
            t = torch.empty(shp, dtype=torch.float32)
            t.normal_(0.0, std, generator=gen)
            if k.startswith("decoder_action_fused_out_proj"):
                # a converted Pi0 checkpoint holds dt = -0.1 folded into this projection
                # (convert_from_jax.py:192-194); without it the synthetic actions are O(10), not O(1)
                t *= 0.1
            out[k] = t.to(BF16)
    return out


def prompt_embeds(ids, dim=2048, std=0.02):
    """language_embeds for token ids: row(id) ~ N(0,std) seeded by the id, times sqrt(dim)
    (pi05_infer.py:784 scales the embedding gather by sqrt(2048))."""
    rows = []
    for i in ids:
        g = torch.Generator().manual_seed(1_000_003 + int(i))
        rows.append(torch.empty(dim).normal_(0.0, std, generator=g))
    if not rows:
        return torch.empty(0, dim, dtype=BF16)
    return (torch.stack(rows).to(BF16) * (dim ** 0.5)).to(BF16)


def make_checkpoint(model="pi0", seed=0, prompt_ids=(), n_vit_layers=27, n_layers=18):
    """Full synthetic converted checkpoint (CPU bf16 tensors)."""
    gen = torch.Generator().manual_seed(seed)
    shapes = {}
    shapes.update(vision_shapes(n_vit_layers))
    shapes.update(encoder_shapes(n_layers))
    shapes.update(pi0_decoder_shapes(n_layers) if model == "pi0" else pi05_decoder_shapes(n_layers))
    ck = _fill(shapes, gen)
    ck["language_embeds"] = prompt_embeds(prompt_ids)
    return ck


def make_inputs(num_views, chunk=50, seed=0):
    """images U[-1,1] (nv,224,224,3), state N(0,1) (32,), noise N(0,1) (chunk,32); bf16."""
    g = torch.Generator().manual_seed(10_000 + seed)
    images = (torch.rand(num_views, 224, 224, 3, generator=g) * 2 - 1).to(BF16)
    state = torch.randn(32, generator=g).to(BF16)
    noise = torch.randn(chunk, 32, generator=g).to(BF16)
    return images, state, noise


def prompt_ids(n, seed=0, vocab=257152):
    g = torch.Generator().manual_seed(20_000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def config(n: int, **kw):
    """The benchmark configurations by number (1..3): returns dict(model, num_views, chunk, checkpoint, inputs)."""
    if n == 1:
        ck = make_checkpoint("pi0", seed=0, **kw)
        return dict(model="pi0", num_views=1, chunk=50, checkpoint=ck, inputs=make_inputs(1, 50, 0))
    if n == 2:
        ck = make_checkpoint("pi0", seed=0, prompt_ids=prompt_ids(20, 0), **kw)
        return dict(model="pi0", num_views=3, chunk=50, checkpoint=ck, inputs=make_inputs(3, 50, 0))
    if n == 3:
        g = torch.Generator().manual_seed(30_000)
        ids = prompt_ids(20, 1) + torch.randint(0, 256, (32,), generator=g).tolist()
        ck = make_checkpoint("pi05", seed=1, prompt_ids=ids, **kw)
        return dict(model="pi05", num_views=2, chunk=50, checkpoint=ck, inputs=make_inputs(2, 50, 1))
    raise ValueError(n)
