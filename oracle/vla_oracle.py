"""Eager fp32 PyTorch restatement of the realtime-vla Pi0 / Pi05 single-observation forward.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA path is compared against; it is
never imported by the product package.  Only the tests, the smoke check and the CPU-baseline leg of
the benchmark may use it.

Parity status: the reference ships no golden vectors and no executable test for this path, so the
restatement is pinned against outputs of the reference's own Triton kernels executed by the Triton
CPU interpreter on small shapes (fixtures under tests/golden/, made by tests/golden/make_golden.py).
Full-model parity against a real checkpoint is unpinned (no checkpoint exists offline).

Everything is evaluated in fp32 from the converted-checkpoint dict.  Weights and inputs are the bf16
values up-cast; no intermediate bf16 rounding of the reference is imitated, except weight
preparation steps that the reference performs once at construction time (Pi05 out-projection
scaling, done in bf16 there).

Reference call graph followed (file:line in the reference project):
  pi0_infer.py:348-364    patch embedding (patch vector order py,px,c) + position embedding
  pi0_infer.py:366-382    LayerNorm eps 1e-5
  pi0_infer.py:588-646    27 SigLIP blocks (16 heads x 72, default SDPA scale)
  pi0_infer.py:753-775    final LayerNorm + 1152->2048 projector
  pi0_infer.py:648-663    RMS norm without learned scale, eps 1e-6
  pi0_infer.py:777-810    QKV (8 Q heads + 1 K + 1 V, head 256) with interleaved-pair RoPE
  pi0_infer.py:819-824    prefix attention, bidirectional, scale 256^-0.5
  pi0_infer.py:841-884    18 prefix layers, layer 17 stops after K/V
  pi0_infer.py:1069-1095  suffix softmax mask: the state token (8 head rows) sees keys j <= P
  pi0_infer.py:1165-1230  state projection, 10 Euler steps of the action expert
  pi0_infer.py:1319-1335  RoPE tables (theta 10000), suffix positions P..P+S-1
  pi05_infer.py:78-113    adaRMS: rms(x)*(1+scale)+shift, gate; style row = [scale|shift|gate]
  pi05_infer.py:282-309, 382-416  key masks by valid prefix length
  pi05_infer.py:418-523   Pi05 decoder (no state token, gated residuals)
  pi05_infer.py:655-722   out-projection scaling by -1/10, time MLP and style precompute
  pi05_infer.py:787-790   suffix RoPE positions start at valid_len-1
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

F32 = torch.float32

N_VIT_LAYERS = 27
N_LAYERS = 18
N_STEPS = 10
VIT_D = 1152
VIT_HEADS = 16
VIT_HD = 72
ENC_D = 2048
DEC_D = 1024
HD = 256
NQ = 8


def _f(t: torch.Tensor, device=None) -> torch.Tensor:
    return t.detach().to(device=device or t.device, dtype=F32)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    # pi0_infer.py:285, 689 — x * sigmoid(2*sqrt(2/pi) * x * (1 + 0.044715 x^2))
    return x * torch.sigmoid(1.5957691216057308 * x * (1.0 + 0.044715 * x * x))


def layer_norm(x, w, b, eps=1e-5):
    mean = x.mean(-1, keepdim=True)
    xc = x - mean
    var = (xc * xc).mean(-1, keepdim=True)
    return xc / torch.sqrt(var + eps) * w + b


def rms_norm(x, eps=1e-6):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)


def rope_table(positions: torch.Tensor):
    """cos/sin (n,128) for integer positions; pi0_infer.py:1319-1323."""
    inv_freq = 1.0 / (10000 ** (torch.arange(0, HD, 2, dtype=F32, device=positions.device) / HD))
    phase = inv_freq[None, :] * positions.to(F32)[:, None]
    return torch.cos(phase), torch.sin(phase)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (..., n, 256) rotated on adjacent pairs (2i, 2i+1); cos/sin (n,128). pi0_infer.py:795-800."""
    x0 = x[..., 0::2]
    x1 = x[..., 1::2]
    y0 = x0 * cos - x1 * sin
    y1 = x1 * cos + x0 * sin
    return torch.stack([y0, y1], dim=-1).flatten(-2)


def patchify(images: torch.Tensor) -> torch.Tensor:
    """(nv,224,224,3) -> (nv*256, 588), patch vector order (py,px,c). pi0_infer.py:350."""
    nv = images.shape[0]
    return images.reshape(nv, 16, 14, 16, 14, 3).permute(0, 1, 3, 2, 4, 5).reshape(nv * 256, 588)


def vit_block(x, n1w, n1b, qkv_w, qkv_b, o_w, o_b, n2w, n2b, up_w, up_b, down_w, down_b):
    """One SigLIP block on x (nv*256,1152); returns (x_out, qkv). pi0_infer.py:608-646."""
    nv = x.shape[0] // 256
    xn = layer_norm(x, n1w, n1b)
    qkv_flat = xn @ qkv_w + qkv_b
    qkv = qkv_flat.reshape(nv, 256, 3, VIT_HEADS, VIT_HD).permute(2, 0, 3, 1, 4)      # (3,nv,h,256,72)
    logits = (qkv[0] @ qkv[1].transpose(-1, -2)) * (VIT_HD ** -0.5)
    attn = torch.softmax(logits, dim=-1) @ qkv[2]                                     # (nv,h,256,72)
    attn = attn.permute(0, 2, 1, 3).reshape(nv * 256, VIT_D)
    x = x + attn @ o_w + o_b
    xn = layer_norm(x, n2w, n2b)
    h = gelu_tanh(xn @ up_w + up_b)
    return x + h @ down_w + down_b, qkv_flat


def vision_encoder(w: Dict[str, torch.Tensor], images: torch.Tensor, n_layers: int = N_VIT_LAYERS) -> torch.Tensor:
    """images (nv,224,224,3) fp32 -> vision_x (nv*256,1152). pi0_infer.py:598-646."""
    nv = images.shape[0]
    x = patchify(images) @ w["vision_patch_embedding_w"].reshape(588, VIT_D)
    x = x + w["vision_patch_embedding_b"] + w["vision_position_embedding"].repeat(nv, 1)
    for i in range(n_layers):
        x, _ = vit_block(x, w["vision_pre_attn_norm_w"][i], w["vision_pre_attn_norm_b"][i],
                         w["vision_attn_qkv_w"][i], w["vision_attn_qkv_b"][i],
                         w["vision_attn_o_w"][i], w["vision_attn_o_b"][i],
                         w["vision_pre_ffn_norm_w"][i], w["vision_pre_ffn_norm_b"][i],
                         w["vision_ffn_up_w"][i], w["vision_ffn_up_b"][i],
                         w["vision_ffn_down_w"][i], w["vision_ffn_down_b"][i])
    return x


def project_vision(w, vision_x):
    """final LayerNorm + projector. pi0_infer.py:753-775."""
    xn = layer_norm(vision_x, w["vision_final_norm_w"], w["vision_final_norm_b"])
    return xn @ w["encoder_multi_modal_projector_w"] + w["encoder_multi_modal_projector_b"]


def prefix_layer(x, cos, sin, valid_len: int, last: bool, qkv_w, o_w=None, gate_w=None, up_w=None, down_w=None):
    """One Gemma-2B prefix layer. Returns (x_out, K, V). pi0_infer.py:852-884; pi05_infer.py:321-380."""
    P = x.shape[0]
    qkv = rms_norm(x) @ qkv_w
    q = apply_rope(qkv[:, : NQ * HD].reshape(P, NQ, HD).transpose(0, 1), cos, sin)   # (8,P,256)
    k = apply_rope(qkv[:, NQ * HD: (NQ + 1) * HD], cos, sin)
    v = qkv[:, (NQ + 1) * HD:]
    if last:
        return x, k, v
    logits = (q @ k.t()) * (HD ** -0.5)                                              # (8,P,P)
    if valid_len < P:
        logits[:, :, valid_len:] = float("-inf")
    attn = (torch.softmax(logits, dim=-1) @ v).transpose(0, 1).reshape(P, NQ * HD)
    x = x + attn @ o_w
    xn = rms_norm(x)
    h = gelu_tanh(xn @ gate_w) * (xn @ up_w)
    x = x + h @ down_w
    return x, k, v


def prefix_encoder(w, encoder_x: torch.Tensor, valid_len: Optional[int] = None, n_layers: int = N_LAYERS):
    """encoder_x (P,2048) -> K,V caches (n_layers,P,256). Layer n_layers-1 only produces K/V."""
    P = encoder_x.shape[0]
    valid_len = P if valid_len is None else valid_len
    cos, sin = rope_table(torch.arange(P, device=encoder_x.device))
    x = encoder_x
    Ks, Vs = [], []
    for i in range(n_layers):
        x, k, v = prefix_layer(x, cos, sin, valid_len, i == n_layers - 1, w["encoder_attn_qkv_w"][i],
                               w["encoder_attn_o_w"][i], w["encoder_ffn_gate_w"][i],
                               w["encoder_ffn_up_w"][i], w["encoder_ffn_down_w"][i])
        Ks.append(k)
        Vs.append(v)
    return torch.stack(Ks), torch.stack(Vs)


def _suffix_attention(q, k_all, v_all, mask):
    """q (8,S,256); k_all/v_all (T,256); mask (S,T) bool (True = visible)."""
    logits = (q @ k_all.t()) * (HD ** -0.5)
    logits = logits.masked_fill(~mask[None], float("-inf"))
    return (torch.softmax(logits, dim=-1) @ v_all).transpose(0, 1).reshape(q.shape[1], NQ * HD)


def pi0_suffix_mask(P, S, device=None):
    """(S, P+S) visibility: the state token (row 0) sees keys j <= P, action tokens see everything.
    pi0_infer.py:1084-1085."""
    mask = torch.ones(S, P + S, dtype=torch.bool, device=device)
    mask[0, P + 1:] = False
    return mask


def pi0_decoder_layer(x, Kp, Vp, cos, sin, mask, qkv_w, o_w, gate_w, up_w, down_w):
    """One action-expert layer; returns (x_out, k_new, v_new). pi0_infer.py:1187-1223."""
    S = x.shape[0]
    qkv = (x @ qkv_w) * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    q = apply_rope(qkv[:, : NQ * HD].reshape(S, NQ, HD).transpose(0, 1), cos, sin)
    k = apply_rope(qkv[:, NQ * HD: (NQ + 1) * HD], cos, sin)
    v = qkv[:, (NQ + 1) * HD:]
    attn = _suffix_attention(q, torch.cat([Kp, k], 0), torch.cat([Vp, v], 0), mask)
    x = x + attn @ o_w
    xn = rms_norm(x)
    h = gelu_tanh(xn @ gate_w) * (xn @ up_w)
    return x + h @ down_w, k, v


def pi0_decoder(w, K, V, state, noise, n_layers: int = N_LAYERS, n_steps: int = N_STEPS):
    """Pi0 action expert. K,V (n_layers,P,256); state (32,); noise (C,32). pi0_infer.py:1165-1230."""
    P = K.shape[1]
    C = noise.shape[0]
    S = C + 1
    dev = noise.device
    cos, sin = rope_table(torch.arange(S, device=dev) + P)
    mask = pi0_suffix_mask(P, S, dev)
    state_tok = state[None, :] @ w["decoder_state_in_proj_w"] + w["decoder_state_in_proj_b"]
    noise = noise.clone()
    for step in range(n_steps):
        a = torch.nn.functional.silu(noise @ w["decoder_action_fused_in_proj_w"]
                                     + w["decoder_action_fused_time_biases"][step])
        a = a @ w["decoder_action_mlp_w"] + w["decoder_action_mlp_b"]
        x = torch.cat([state_tok, a], 0)
        for i in range(n_layers):
            x, _, _ = pi0_decoder_layer(x, K[i], V[i], cos, sin, mask, w["decoder_attn_qkv_w"][i],
                                        w["decoder_attn_o_w"][i], w["decoder_ffn_gate_w"][i],
                                        w["decoder_ffn_up_w"][i], w["decoder_ffn_down_w"][i])
        xn = rms_norm(x[1:])
        noise = noise + xn @ w["decoder_action_fused_out_proj_w"] + w["decoder_action_fused_out_proj_b"]
    return noise


def pi05_styles(w, n_layers: int = N_LAYERS, n_steps: int = N_STEPS):
    """time_emb and the adaRMS style rows per (step, layer). pi05_infer.py:673-722."""
    silu = torch.nn.functional.silu
    te = silu(w["decoder_time_embeds"][:n_steps] @ w["decoder_time_mlp_in_w"] + w["decoder_time_mlp_in_b"])
    te = silu(te @ w["decoder_time_mlp_out_w"] + w["decoder_time_mlp_out_b"])            # (steps,1024)
    attn = torch.einsum("sk,lkn->sln", te, w["decoder_pre_attn_norm_mod_w"][:n_layers]) \
        + w["decoder_pre_attn_norm_mod_b"][:n_layers][None]
    ffn = torch.einsum("sk,lkn->sln", te, w["decoder_pre_ffn_norm_mod_w"][:n_layers]) \
        + w["decoder_pre_ffn_norm_mod_b"][:n_layers][None]
    fin = te @ w["decoder_final_norm_mod_w"] + w["decoder_final_norm_mod_b"]
    return attn, ffn, fin


def ada_rms(x, style):
    """pi05_infer.py:99-113. style (3072,) = [scale|shift|gate]. Returns (normed, gate)."""
    scale, shift, gate = style[:DEC_D], style[DEC_D: 2 * DEC_D], style[2 * DEC_D:]
    return rms_norm(x) * (1.0 + scale) + shift, gate


def pi05_decoder_layer(x, Kp, Vp, cos, sin, mask, style_attn, style_ffn, qkv_w, o_w, gate_w, up_w, down_w):
    """One adaRMS action-expert layer; returns (x_out, k_new, v_new). pi05_infer.py:428-509."""
    S = x.shape[0]
    xn, gate = ada_rms(x, style_attn)
    qkv = xn @ qkv_w
    q = apply_rope(qkv[:, : NQ * HD].reshape(S, NQ, HD).transpose(0, 1), cos, sin)
    k = apply_rope(qkv[:, NQ * HD: (NQ + 1) * HD], cos, sin)
    v = qkv[:, (NQ + 1) * HD:]
    attn = _suffix_attention(q, torch.cat([Kp, k], 0), torch.cat([Vp, v], 0), mask)
    x = x + gate * (attn @ o_w)
    xn, gate = ada_rms(x, style_ffn)
    h = gelu_tanh(xn @ gate_w) * (xn @ up_w)
    return x + gate * (h @ down_w), k, v


def pi05_decoder(w, K, V, noise, valid_len: int, n_layers: int = N_LAYERS, n_steps: int = N_STEPS):
    """Pi05 action expert. K,V (n_layers,P_alloc,256). pi05_infer.py:418-523."""
    P = K.shape[1]
    S = noise.shape[0]
    dev = noise.device
    cos, sin = rope_table(torch.arange(S, device=dev) + (valid_len - 1))        # pi05_infer.py:788
    mask = torch.ones(S, P + S, dtype=torch.bool, device=dev)
    mask[:, valid_len:P] = False
    st_attn, st_ffn, st_fin = pi05_styles(w, n_layers, n_steps)
    # The reference scales the out-projection once, in place, in bf16 (pi05_infer.py:670-671).
    wo = (w["decoder_action_out_proj_w"].to(torch.bfloat16) * (-1.0 / N_STEPS)).to(F32)
    bo = (w["decoder_action_out_proj_b"].to(torch.bfloat16) * (-1.0 / N_STEPS)).to(F32)
    noise = noise.clone()
    for step in range(n_steps):
        x = noise @ w["decoder_action_in_proj_w"] + w["decoder_action_in_proj_b"]
        for i in range(n_layers):
            x, _, _ = pi05_decoder_layer(x, K[i], V[i], cos, sin, mask, st_attn[step, i], st_ffn[step, i],
                                         w["decoder_attn_qkv_w"][i], w["decoder_attn_o_w"][i],
                                         w["decoder_ffn_gate_w"][i], w["decoder_ffn_up_w"][i],
                                         w["decoder_ffn_down_w"][i])
        xn, _ = ada_rms(x, st_fin[step])
        noise = noise + xn @ wo + bo
    return noise


def _weights_f32(checkpoint, device):
    return {k: _f(v, device) for k, v in checkpoint.items() if k != "embedding_weight"}


@torch.no_grad()
def pi0_forward(checkpoint, images, state, noise, device="cpu", return_intermediates=False):
    """Oracle for Pi0Inference(checkpoint, nv, C).forward(images, state, noise). pi0_infer.py:1232-1361."""
    w = _weights_f32(checkpoint, device)
    images, state, noise = _f(images, device), _f(state, device), _f(noise, device)
    vx = vision_encoder(w, images)
    enc = torch.cat([project_vision(w, vx), w["language_embeds"].reshape(-1, ENC_D)], 0)
    K, V = prefix_encoder(w, enc)
    out = pi0_decoder(w, K, V, state, noise)
    if return_intermediates:
        return out, {"vision_x": vx, "encoder_x": enc, "K": K, "V": V}
    return out


def pi05_prompt_from_ids(embedding_weight, ids):
    """Prompt embeddings of token ids: embedding(ids) * sqrt(2048), rounded to bf16 as in the reference
    (pi05_infer.py:726-743 builds the bf16 table, :783-785 gathers and scales).  Returns fp32 values."""
    table = torch.as_tensor(embedding_weight).to(torch.bfloat16)
    ids = torch.as_tensor(ids).long().cpu()
    return (table.cpu()[ids] * float(table.shape[1] ** 0.5)).to(torch.bfloat16).float()


@torch.no_grad()
def pi05_forward(checkpoint, images, noise, device="cpu", prompt_embeds=None, max_prompt_len=None,
                 return_intermediates=False):
    """Oracle for Pi05Inference(..., discrete_state_input=False).forward(images, noise), or with explicit
    prompt embeddings shorter than the allocated prompt window. pi05_infer.py:525-528, 804-826."""
    w = _weights_f32(checkpoint, device)
    images, noise = _f(images, device), _f(noise, device)
    nv = images.shape[0]
    prompt = w["language_embeds"].reshape(-1, ENC_D) if prompt_embeds is None else _f(prompt_embeds, device)
    max_prompt_len = prompt.shape[0] if max_prompt_len is None else max_prompt_len
    valid_len = nv * 256 + prompt.shape[0]
    pad = torch.zeros(max_prompt_len - prompt.shape[0], ENC_D, dtype=F32, device=prompt.device)
    vx = vision_encoder(w, images)
    enc = torch.cat([project_vision(w, vx), prompt, pad], 0)
    K, V = prefix_encoder(w, enc, valid_len=valid_len)
    out = pi05_decoder(w, K, V, noise, valid_len)
    if return_intermediates:
        return out, {"vision_x": vx, "encoder_x": enc, "K": K, "V": V}
    return out


def sincos_time_table(n_steps: int = N_STEPS) -> torch.Tensor:
    """decoder_time_embeds of a converted Pi05 checkpoint: [sin|cos] of t*2pi/period, periods 4e-3..4,
    t = 1.0, 0.9, ... (convert_from_jax_pi05.py:214-228)."""
    frac = torch.linspace(0.0, 1.0, DEC_D // 2)
    period = 4e-3 * (4.0 / 4e-3) ** frac
    rows = []
    t = torch.tensor(1.0)
    for _ in range(n_steps):
        arg = t * (1.0 / period) * 2 * math.pi
        rows.append(torch.cat([torch.sin(arg), torch.cos(arg)]).to(torch.bfloat16))
        t = t + (-1.0 / n_steps)
    return torch.stack(rows)
