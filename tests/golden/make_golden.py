"""Generate the known-answer fixtures in this directory from the reference's own kernels.

Run once, in a container that has the reference checkout, with
    python tests/golden/make_golden.py /path/to/reference [case ...]
It executes the reference's @triton.jit kernels through the Triton CPU interpreter
(TRITON_INTERPRET=1) on fp32 CPU tensors holding bf16-representable values (bf16 CPU tensors are not
reliable in the interpreter), by calling the reference's shape-specialised wrapper functions in the
same order as its model functions do.  The two torch.compile'd attention functions are called through
their undecorated bodies.  Weights are not stored: each fixture records the seed and the tests
regenerate them with weights_for(); inputs and the reference's outputs are stored (a few KB each).

Cases (reference file:line of the code sequence that is reproduced):
  patch_embed        pi0_infer.py:599-605   conv2d_embed_n256_1152_res
  vit_block          pi0_infer.py:608-646   one SigLIP block, one view
  prefix_layer       pi0_infer.py:852-884   one Gemma prefix layer, P=5
  pi0_decoder_layer  pi0_infer.py:1187-1223 one action-expert layer, P=6 prefix keys, S=4
  pi05_decoder_layer pi05_infer.py:428-509  one adaRMS layer, alloc 7 / valid 5 prefix keys, S=4
  projector          pi0_infer.py:753-775   final LayerNorm + 1152->2048 projector, one view
  pi0_decoder_steps  pi0_infer.py:1165-1230 the Euler loop itself: state projection, then two steps of (action in-projection
                                            with time_biases[step], action MLP, one expert layer, out-projection + update)
  pi05_prefix_layer  pi05_infer.py:321-380  one prefix layer with the valid-length softmax mask, alloc 7 / valid 5 tokens
  pi05_precompute    pi05_infer.py:673-722  constructor: time MLP and adaRMS style rows for 2 steps x 2 layers + final
"""
import os
import sys
import time

os.environ["TRITON_INTERPRET"] = "1"
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_values(shape, gen, std=0.02):
    return torch.empty(shape).normal_(0.0, std, generator=gen).to(torch.bfloat16).float()


def weights_for(case, seed):
    """Deterministic fp32 tensors with bf16-representable values, shared by generator and tests."""
    g = torch.Generator().manual_seed(seed)
    n = lambda *s, std=0.02: bf16_values(s, g, std)
    if case == "patch_embed":
        return dict(w=n(14, 14, 3, 1152), b=n(1152), pos=n(256, 1152), images=(torch.rand(1, 224, 224, 3, generator=g) * 2 - 1).to(torch.bfloat16).float())
    if case == "vit_block":
        return dict(x=n(256, 1152, std=0.5), n1w=1 + n(1152), n1b=n(1152), qkv_w=n(1152, 3456), qkv_b=n(3456),
                    o_w=n(1152, 1152), o_b=n(1152), n2w=1 + n(1152), n2b=n(1152),
                    up_w=n(1152, 4304), up_b=n(4304), down_w=n(4304, 1152), down_b=n(1152))
    if case == "prefix_layer":
        return dict(x=n(5, 2048, std=1.0), qkv_w=n(2048, 2560), o_w=n(2048, 2048), gate_w=n(2048, 16384),
                    up_w=n(2048, 16384), down_w=n(16384, 2048))
    if case == "pi0_decoder_layer":
        return dict(x=n(4, 1024, std=1.0), K=n(6, 256, std=1.0), V=n(6, 256, std=1.0), qkv_w=n(1024, 2560),
                    o_w=n(2048, 1024), gate_w=n(1024, 4096), up_w=n(1024, 4096), down_w=n(4096, 1024))
    if case == "pi05_decoder_layer":
        return dict(x=n(4, 1024, std=1.0), K=n(7, 256, std=1.0), V=n(7, 256, std=1.0), qkv_w=n(1024, 2560),
                    o_w=n(2048, 1024), gate_w=n(1024, 4096), up_w=n(1024, 4096), down_w=n(4096, 1024),
                    style_attn=n(3072, std=0.3), style_ffn=n(3072, std=0.3))
    if case == "projector":
        return dict(x=n(256, 1152, std=0.5), nw=1 + n(1152), nb=n(1152), pw=n(1152, 2048), pb=n(2048))
    if case == "pi0_decoder_steps":
        return dict(state=n(32, std=1.0), noise=n(3, 32, std=1.0), K=n(6, 256, std=1.0), V=n(6, 256, std=1.0),
                    state_w=n(32, 1024), state_b=n(1024), in_w=n(32, 1024), time_b=n(10, 1024), mlp_w=n(1024, 1024),
                    mlp_b=n(1024), qkv_w=n(1024, 2560), o_w=n(2048, 1024), gate_w=n(1024, 4096), up_w=n(1024, 4096),
                    down_w=n(4096, 1024), out_w=n(1024, 32), out_b=n(32))
    if case == "pi05_prefix_layer":
        return dict(x=n(7, 2048, std=1.0), qkv_w=n(2048, 2560), o_w=n(2048, 2048), gate_w=n(2048, 16384),
                    up_w=n(2048, 16384), down_w=n(16384, 2048))
    if case == "pi05_precompute":
        t = torch.linspace(0.0, 1.0, 512)
        period = 4e-3 * (4.0 / 4e-3) ** t
        te = torch.stack([torch.cat([torch.sin(tt / period * 6.283185307179586), torch.cos(tt / period * 6.283185307179586)])
                          for tt in (1.0, 0.9)]).to(torch.bfloat16).float()
        return dict(time_embeds=te, in_w=n(1024, 1024), in_b=n(1024), out_w=n(1024, 1024), out_b=n(1024),
                    attn_w=n(2, 1024, 3072), attn_b=n(2, 3072), ffn_w=n(2, 1024, 3072), ffn_b=n(2, 3072),
                    fin_w=n(1024, 3072), fin_b=n(3072))
    raise KeyError(case)


def rope_rows(positions):
    """Interleaved [cos0,sin0,cos1,sin1,...] rows rounded to bf16, as pi0_infer.py:1319-1326 builds them."""
    inv_freq = 1.0 / (10000 ** (torch.arange(0, 256, 2, dtype=torch.float32) / 256))
    ph = inv_freq[None, :] * positions.float()[:, None]
    c = torch.cos(ph).to(torch.bfloat16).float()
    s = torch.sin(ph).to(torch.bfloat16).float()
    return torch.cat([c[:, :, None], s[:, :, None]], 2).reshape(-1, 256).contiguous()


def padded(t, rows=128):
    """Copy of t backed by storage with `rows` rows, so that kernels that read unmasked rows stay in bounds."""
    buf = torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype)
    buf[: t.shape[0]] = t
    return buf[: t.shape[0]]


def run_case(case, ref, seed):
    import pi0_infer as R0
    w = weights_for(case, seed)
    out = {}
    if case == "patch_embed":
        vx = torch.zeros(1, 256, 1152)
        R0.conv2d_embed_n256_1152_res(w["images"], w["w"], w["b"], w["pos"], vx)
        out["vision_x"] = vx.reshape(256, 1152)[:: 8].clone()
    elif case == "vit_block":
        x = w["x"].clone().reshape(1, 256, 1152)
        xn = torch.zeros(1, 256, 1152)
        qkv = torch.zeros(1, 256, 3456)
        hid = torch.zeros(1, 256, 4304)
        buf = torch.zeros(256 * 1152 * 4 + 64 * 1152 * 4)
        attn_fn = getattr(R0.AttnMultiKey, "_torchdynamo_orig_callable", R0.AttnMultiKey)
        R0.layer_norm_QKV_matmul_n256_1152_3456_bias(x, w["n1w"], w["n1b"], w["qkv_w"], w["qkv_b"], qkv, xn)
        attn = attn_fn(qkv).contiguous()
        R0.matmul_n256_1152_1152_bias_res(attn, w["o_w"], w["o_b"], x, x, buf)
        R0.layer_norm_matmul_n256_1152_4304_bias_gelu(x, w["n2w"], w["n2b"], w["up_w"], w["up_b"], hid, xn)
        R0.matmul_n256_4304_1152_bias_res(hid, w["down_w"], w["down_b"], x, x, buf)
        out["x_out"] = x.reshape(256, 1152)[:: 8].clone()
        out["qkv"] = qkv.reshape(256, 3456)[:: 32].clone()
    elif case == "prefix_layer":
        P = 5
        x = padded(w["x"].clone())
        xn = padded(torch.zeros(P, 2048))
        Q = padded(torch.zeros(P * 8, 256), 1024)
        K = padded(torch.zeros(P, 256))
        V = padded(torch.zeros(P, 256))
        hid = padded(torch.zeros(P, 16384))
        rope = padded(rope_rows(torch.arange(P)))
        attn_fn = getattr(R0.AttnSingleKey, "_torchdynamo_orig_callable", R0.AttnSingleKey)
        R0.rms_matmul_n_2048_2560_qkv_rope(x, w["qkv_w"], rope, Q, K, V, xn)
        attn = attn_fn(Q, K, V, 1.0 / (256 ** 0.5)).contiguous()
        R0.matmul_n_2048_2048_res(padded(attn), w["o_w"], x)
        R0.rms_matmul_n_2048_16384_gate(x, w["gate_w"], w["up_w"], hid, xn)
        R0.matmul_n_16384_2048_res(hid, w["down_w"], x)
        out.update(x_out=x.clone(), K=K.clone(), V=V.clone())
    elif case == "pi0_decoder_layer":
        P, S = 6, 4
        x = padded(w["x"].clone())
        K = padded(torch.cat([w["K"], torch.zeros(S, 256)]))
        V = padded(torch.cat([w["V"], torch.zeros(S, 256)]))
        q = padded(torch.zeros(S * 8, 256))
        fac = padded(torch.zeros(S))
        att = padded(torch.zeros(S * 8, P + S))
        hid = padded(torch.zeros(S, 4096))
        rope = padded(rope_rows(torch.arange(S) + P))
        R0.rms_matmul_k_1024_2560_qkv_rope(x, w["qkv_w"], rope, q, K[P:], V[P:], fac)
        R0.matmul_k8_256_n_softmax_mask0(q, K, att, P)
        out["probs"] = att.clone()
        R0.matmul_k8_n_256(att, V, q)
        R0.matmul_k_2048_1024_res(q.view(-1, 2048), w["o_w"], x)
        R0.rms_matmul_k_1024_4096_gate(x, w["gate_w"], w["up_w"], hid, fac)
        R0.matmul_k_4096_1024_res(hid, w["down_w"], x)
        out.update(x_out=x.clone(), K_new=K[P:].clone(), V_new=V[P:].clone())
    elif case == "pi05_decoder_layer":
        import pi05_infer as R5
        PA, PV, S = 7, 5, 4
        x = padded(w["x"].clone())
        K = padded(torch.cat([w["K"], torch.zeros(S, 256)]))
        V = padded(torch.cat([w["V"], torch.zeros(S, 256)]))
        q = padded(torch.zeros(S * 8, 256))
        xn = padded(torch.zeros(S, 1024))
        gate = padded(torch.zeros(S, 1024))
        logits = padded(torch.zeros(S * 8, PA + S))
        att = padded(torch.zeros(S * 8, PA + S))
        hid = padded(torch.zeros(S, 4096))
        valid = torch.tensor([PV], dtype=torch.int32)
        rope = padded(rope_rows(torch.arange(S) + (PV - 1)))
        R5.adarms_norm_style_proj(x, None, None, None, xn, gate, w["style_attn"])
        R5.matmul_k_1024_2560_qkv_rope(xn, w["qkv_w"], rope, q, K[PA:PA + S], V[PA:PA + S])
        R0.matmul_abT_scale[(((S * 8 + 31) // 32) * ((PA + S + 31) // 32),)](
            q, K[:PA + S], logits, S * 8, PA + S, 256, 256 ** -0.5, BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=64)
        R5.softmax_kernel_prefix_suffix[((S * 8 + 3) // 4,)](
            logits, S * 8, PA, S, valid, att, BLOCK_SIZE_M=4, BLOCK_SIZE=1024)
        out["probs"] = att.clone()
        R0.matmul_k8_n_256(att, V[:PA + S], q)
        R5.matmul_k_2048_1024_gate(q.view(-1, 2048), w["o_w"], x, gate)
        R5.adarms_norm_style_proj(x, None, None, None, xn, gate, w["style_ffn"])
        R5.matmul_small_gate[((S + 127) // 128, (4096 + 63) // 64)](xn, w["gate_w"], w["up_w"], hid, S, 1024, 4096)
        R5.matmul_k_4096_1024_gate(hid, w["down_w"], x, gate)
        out.update(x_out=x.clone(), K_new=K[PA:PA + S].clone(), V_new=V[PA:PA + S].clone())
    elif case == "projector":
        out_buf = torch.zeros(256, 2048)
        R0.layer_norm_matmul_n256_1152_2048_bias(w["x"].clone().reshape(1, 256, 1152), w["nw"], w["nb"], w["pw"], w["pb"], out_buf,
                                                 torch.zeros(256, 1152))
        out["encoder_x"] = out_buf[:: 8].clone()
    elif case == "pi0_decoder_steps":
        P, C = 6, 3
        S = C + 1
        state_buf = padded(torch.zeros(1, 1024))
        x = padded(torch.zeros(S, 1024))
        x_buf = padded(torch.zeros(C, 1024))
        noise = padded(w["noise"].clone())
        K = padded(torch.cat([w["K"], torch.zeros(S, 256)]))
        V = padded(torch.cat([w["V"], torch.zeros(S, 256)]))
        q = padded(torch.zeros(S * 8, 256))
        fac = padded(torch.zeros(S))
        att = padded(torch.zeros(S * 8, P + S))
        hid = padded(torch.zeros(S, 4096))
        rope = padded(rope_rows(torch.arange(S) + P))
        R0.matmul_1_32_1024_bias(w["state"].clone(), w["state_w"], w["state_b"], state_buf)
        steps = []
        for step in range(2):
            x[:1].copy_(state_buf)
            R0.matmul_k_32_1024_bias_silu(noise, w["in_w"], w["time_b"][step % 10], x_buf)
            R0.matmul_k_1024_1024_bias(x_buf, w["mlp_w"], w["mlp_b"], x[1:])
            R0.rms_matmul_k_1024_2560_qkv_rope(x, w["qkv_w"], rope, q, K[P:], V[P:], fac)
            R0.matmul_k8_256_n_softmax_mask0(q, K, att, P)
            R0.matmul_k8_n_256(att, V, q)
            R0.matmul_k_2048_1024_res(q.view(-1, 2048), w["o_w"], x)
            R0.rms_matmul_k_1024_4096_gate(x, w["gate_w"], w["up_w"], hid, fac)
            R0.matmul_k_4096_1024_res(hid, w["down_w"], x)
            R0.rms_matmul_k_1024_32_bias_res(x[1:], w["out_w"], w["out_b"], noise, fac)
            steps.append(noise.clone())
        out.update(noise_step1=steps[0], noise_step2=steps[1], x_last=x.clone())
    elif case == "pi05_prefix_layer":
        import pi05_infer as R5
        PA, PV = 7, 5
        x = padded(w["x"].clone())
        xn = padded(torch.zeros(PA, 2048))
        Q = padded(torch.zeros(PA * 8, 256), 1024)
        K = padded(torch.zeros(PA, 256))
        V = padded(torch.zeros(PA, 256))
        logits = padded(torch.zeros(PA * 8, PA), 1024)
        att = padded(torch.zeros(PA * 8, PA), 1024)
        ctx = padded(torch.zeros(PA * 8, 256), 1024)
        hid = padded(torch.zeros(PA, 16384))
        valid = torch.tensor([PV], dtype=torch.int32)
        rope = padded(rope_rows(torch.arange(PA)))
        R0.rms_matmul_n_2048_2560_qkv_rope(x, w["qkv_w"], rope, Q, K, V, xn)
        R0.matmul_abT_scale[(((PA * 8 + 31) // 32) * ((PA + 31) // 32),)](
            Q, K, logits, PA * 8, PA, 256, 1.0 / (256 ** 0.5), BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=64)
        R5.softmax_kernel_masklen[((PA * 8 + 3) // 4,)](logits, PA * 8, PA, valid, att, BLOCK_SIZE_M=4, BLOCK_SIZE=1024)
        out["probs"] = att.clone()
        R0.matmul_k8_n_256(att, V, ctx)
        R0.matmul_n_2048_2048_res(ctx.view(-1, 2048), w["o_w"], x)
        R0.rms_matmul_n_2048_16384_gate(x, w["gate_w"], w["up_w"], hid, xn)
        R0.matmul_n_16384_2048_res(hid, w["down_w"], x)
        out.update(x_out=x.clone(), K=K.clone(), V=V.clone())
    elif case == "pi05_precompute":
        import pi05_infer as R5
        x_buf = padded(torch.zeros(1, 1024))
        time_emb = [padded(torch.zeros(1, 1024)) for _ in range(2)]
        style_attn = torch.zeros(2, 2, 3072)
        style_ffn = torch.zeros(2, 2, 3072)
        style_fin = torch.zeros(2, 3072)

        def style(dst, ww, bb, step):
            row = padded(torch.zeros(1, 3072))
            R0.matmul_small_bias[((1 + 31) // 32) * (3072 // 32),](time_emb[step], ww, row, bb, seq_len=1, features=1024,
                                                                  hidden=3072, BLOCK_SIZE_N=32, BLOCK_SIZE_M=32, BLOCK_SIZE_K=32)
            dst.copy_(row[0])
        for step in range(2):
            R5.matmul_1_1024_1024_bias_silu(padded(w["time_embeds"][step].clone().view(1, -1)), w["in_w"], w["in_b"], x_buf)
            R5.matmul_1_1024_1024_bias_silu(x_buf, w["out_w"], w["out_b"], time_emb[step])
            for i in range(2):
                style(style_attn[step, i], w["attn_w"][i], w["attn_b"][i], step)
                style(style_ffn[step, i], w["ffn_w"][i], w["ffn_b"][i], step)
            style(style_fin[step], w["fin_w"], w["fin_b"], step)
        out.update(time_emb=torch.cat([t[:1] for t in time_emb]).clone(), style_attn=style_attn, style_ffn=style_ffn, style_fin=style_fin)
    else:
        raise KeyError(case)
    return out


SEEDS = dict(patch_embed=11, vit_block=12, prefix_layer=13, pi0_decoder_layer=14, pi05_decoder_layer=15, projector=16,
             pi0_decoder_steps=17, pi05_prefix_layer=18, pi05_precompute=19)

if __name__ == "__main__":
    ref = sys.argv[1]
    sys.path.insert(0, ref)
    cases = sys.argv[2:] or list(SEEDS)
    for case in cases:
        t0 = time.time()
        res = run_case(case, ref, SEEDS[case])
        res = {k: v.to(torch.bfloat16) if v.dtype == torch.float32 else v for k, v in res.items()}
        res["seed"] = SEEDS[case]
        torch.save(res, os.path.join(HERE, case + ".pt"))
        print(case, "done in %.1fs" % (time.time() - t0), {k: tuple(v.shape) for k, v in res.items() if hasattr(v, "shape")}, flush=True)
