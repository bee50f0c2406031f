"""The fp32 oracle against known answers produced by the reference's own Triton kernels
(fixtures made by tests/golden/make_golden.py through the Triton CPU interpreter).

The reference rounds every kernel output to bf16, the oracle does not, so agreement is at the level of
bf16 rounding of the values involved: a few ulp (2^-8 relative) of the largest magnitudes."""
import os

import pytest
import torch

from oracle import vla_oracle as O
from tests.golden.make_golden import weights_for

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(case):
    path = os.path.join(GOLD, case + ".pt")
    if not os.path.exists(path):
        pytest.skip("fixture %s missing" % case)
    g = torch.load(path)
    return g, weights_for(case, g["seed"])


def close(got, want, rel=1.5e-2, what=""):
    want = want.float()
    err = (got - want).abs()
    scale = want.abs().max().item()
    assert err.max().item() <= rel * scale, "%s max-abs %.3e vs scale %.3e" % (what, err.max().item(), scale)
    assert err.mean().item() <= 0.25 * rel * scale, "%s mean-abs %.3e" % (what, err.mean().item())


def test_patch_embed():
    g, w = load("patch_embed")
    x = O.patchify(w["images"]) @ w["w"].reshape(588, 1152) + w["b"] + w["pos"]
    close(x[::8], g["vision_x"], what="vision_x")


def test_vit_block():
    g, w = load("vit_block")
    x, qkv = O.vit_block(w["x"], w["n1w"], w["n1b"], w["qkv_w"], w["qkv_b"], w["o_w"], w["o_b"],
                         w["n2w"], w["n2b"], w["up_w"], w["up_b"], w["down_w"], w["down_b"])
    close(qkv[::32], g["qkv"], what="qkv")
    close(x[::8], g["x_out"], what="x_out")


def test_prefix_layer():
    g, w = load("prefix_layer")
    cos, sin = O.rope_table(torch.arange(5))
    x, k, v = O.prefix_layer(w["x"], cos, sin, 5, False, w["qkv_w"], w["o_w"], w["gate_w"], w["up_w"], w["down_w"])
    close(k, g["K"], what="K")
    close(v, g["V"], what="V")
    close(x, g["x_out"], what="x_out")


def test_pi0_decoder_layer():
    g, w = load("pi0_decoder_layer")
    P, S = 6, 4
    cos, sin = O.rope_table(torch.arange(S) + P)
    mask = O.pi0_suffix_mask(P, S)
    x, k, v = O.pi0_decoder_layer(w["x"], w["K"], w["V"], cos, sin, mask,
                                  w["qkv_w"], w["o_w"], w["gate_w"], w["up_w"], w["down_w"])
    close(k, g["K_new"], what="K_new")
    close(v, g["V_new"], what="V_new")
    close(x, g["x_out"], what="x_out")
    # the state token's 8 head rows must put exactly zero weight on keys beyond index P
    assert g["probs"].float()[:8, P + 1:].abs().max().item() == 0.0
    assert g["probs"].float()[8:, P + 1:].abs().max().item() > 0.0


def test_pi05_decoder_layer():
    g, w = load("pi05_decoder_layer")
    PA, PV, S = 7, 5, 4
    cos, sin = O.rope_table(torch.arange(S) + (PV - 1))
    mask = torch.ones(S, PA + S, dtype=torch.bool)
    mask[:, PV:PA] = False
    x, k, v = O.pi05_decoder_layer(w["x"], w["K"], w["V"], cos, sin, mask, w["style_attn"], w["style_ffn"],
                                   w["qkv_w"], w["o_w"], w["gate_w"], w["up_w"], w["down_w"])
    close(k, g["K_new"], what="K_new")
    close(v, g["V_new"], what="V_new")
    close(x, g["x_out"], what="x_out")
    assert g["probs"].float()[:, PV:PA].abs().max().item() == 0.0


def test_projector():
    """Final LayerNorm + projector into the prefix stream (pi0_infer.py:753-775)."""
    g, w = load("projector")
    enc = O.project_vision(dict(vision_final_norm_w=w["nw"], vision_final_norm_b=w["nb"],
                                encoder_multi_modal_projector_w=w["pw"], encoder_multi_modal_projector_b=w["pb"]), w["x"])
    close(enc[::8], g["encoder_x"], rel=1e-2, what="encoder_x")


def test_pi0_decoder_steps():
    """The Euler loop of the action expert (pi0_infer.py:1165-1230) over two steps of one layer: state projection, action
    in-projection with a different time bias per step, action MLP, the layer, and the fused norm + out-projection +
    update of the noise.  Pins the loop structure and the three small operators no single-layer fixture covers."""
    g, w = load("pi0_decoder_steps")
    ck = dict(decoder_state_in_proj_w=w["state_w"], decoder_state_in_proj_b=w["state_b"],
              decoder_action_fused_in_proj_w=w["in_w"], decoder_action_fused_time_biases=w["time_b"],
              decoder_action_mlp_w=w["mlp_w"], decoder_action_mlp_b=w["mlp_b"],
              decoder_attn_qkv_w=w["qkv_w"][None], decoder_attn_o_w=w["o_w"][None], decoder_ffn_gate_w=w["gate_w"][None],
              decoder_ffn_up_w=w["up_w"][None], decoder_ffn_down_w=w["down_w"][None],
              decoder_action_fused_out_proj_w=w["out_w"], decoder_action_fused_out_proj_b=w["out_b"])
    K, V = w["K"][None], w["V"][None]
    one = O.pi0_decoder(ck, K, V, w["state"], w["noise"], n_layers=1, n_steps=1)
    two = O.pi0_decoder(ck, K, V, w["state"], w["noise"], n_layers=1, n_steps=2)
    # the update per step is what the operators produce; compare it, not the noise it is added to
    close(one - w["noise"], g["noise_step1"].float() - w["noise"], rel=2e-2, what="update of step 1")
    close(two - one, g["noise_step2"].float() - g["noise_step1"].float(), rel=3e-2, what="update of step 2")
    close(two, g["noise_step2"], rel=1e-2, what="noise after two steps")
    # the two steps used different time biases: the updates differ
    assert (g["noise_step2"].float() - 2 * g["noise_step1"].float() + w["noise"]).abs().max().item() > 1e-3


def test_pi05_prefix_layer_valid_length_mask():
    """One Pi05 prefix layer with 7 allocated and 5 valid tokens (pi05_infer.py:321-380): keys beyond the valid length
    get exactly zero probability in every row, padded rows included, and K / V / the stream follow the oracle."""
    g, w = load("pi05_prefix_layer")
    PA, PV = 7, 5
    cos, sin = O.rope_table(torch.arange(PA))
    x, k, v = O.prefix_layer(w["x"], cos, sin, PV, False, w["qkv_w"], w["o_w"], w["gate_w"], w["up_w"], w["down_w"])
    assert g["probs"].float()[:, PV:].abs().max().item() == 0.0
    assert (g["probs"].float()[:, :PV].sum(-1) - 1).abs().max().item() < 2e-2
    close(k, g["K"], rel=1e-2, what="K")
    close(v, g["V"], rel=1e-2, what="V")
    close(x, g["x_out"], rel=1.5e-2, what="x_out")


def test_pi05_precompute():
    """Constructor-time work of Pi05 (pi05_infer.py:673-722): time MLP and the adaRMS style rows."""
    g, w = load("pi05_precompute")
    ck = dict(decoder_time_embeds=w["time_embeds"], decoder_time_mlp_in_w=w["in_w"], decoder_time_mlp_in_b=w["in_b"],
              decoder_time_mlp_out_w=w["out_w"], decoder_time_mlp_out_b=w["out_b"],
              decoder_pre_attn_norm_mod_w=w["attn_w"], decoder_pre_attn_norm_mod_b=w["attn_b"],
              decoder_pre_ffn_norm_mod_w=w["ffn_w"], decoder_pre_ffn_norm_mod_b=w["ffn_b"],
              decoder_final_norm_mod_w=w["fin_w"], decoder_final_norm_mod_b=w["fin_b"])
    attn, ffn, fin = O.pi05_styles(ck, n_layers=2, n_steps=2)
    close(attn, g["style_attn"], rel=1.5e-2, what="style_attn")
    close(ffn, g["style_ffn"], rel=1.5e-2, what="style_ffn")
    close(fin, g["style_fin"], rel=1.5e-2, what="style_fin")


def test_prompt_from_ids_matches_embedding_module():
    """The reference embeds prompt ids with nn.Embedding (bf16 table) and multiplies by the Python float
    sqrt(2048) (pi05_infer.py:735-743, 783-785); the oracle's gather must give the same bf16 values."""
    import torch
    from oracle import vla_oracle as O
    g = torch.Generator().manual_seed(3)
    table = (torch.randn(300, 2048, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, 300, (23,), generator=g)
    emb = torch.nn.Embedding(300, 2048, dtype=torch.bfloat16)
    with torch.no_grad():
        emb.weight.copy_(table)
        want = emb(ids) * float(2048 ** 0.5)
    assert want.dtype == torch.bfloat16
    assert torch.equal(O.pi05_prompt_from_ids(table, ids), want.float())
