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
    else:
        raise KeyError(case)
    return out


SEEDS = dict(patch_embed=11, vit_block=12, prefix_layer=13, pi0_decoder_layer=14, pi05_decoder_layer=15)

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
