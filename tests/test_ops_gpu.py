"""Kernel-level parity on a B200: each CUDA kernel, called through the C ABI (vla_op_*), against the fp32
oracle arithmetic on the same seeded bf16 inputs.  Outputs are bf16, so the bound is bf16 rounding of the
result (2^-8 relative to the largest magnitude) plus fp32 accumulation-order noise."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import vla_oracle as O   # noqa: E402


def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda")


def rnd(shape, std, seed, d):
    g = torch.Generator().manual_seed(seed)
    return torch.empty(shape).normal_(0, std, generator=g).to(torch.bfloat16).to(d)


def assert_close(got, want, rel=6e-3, what=""):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all(), what + ": non-finite output"
    scale = want.abs().max().item() + 1e-6
    err = (got - want).abs().max().item()
    assert err <= rel * scale, "%s: max-abs %.4e vs scale %.4e (rel %.2e)" % (what, err, scale, err / scale)


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D,mode", [(1152, 0), (2048, 1), (1024, 1), (1024, 2)])
def test_norm(D, mode):
    import vla_ops as gpu_ops
    d = dev()
    x = rnd((51, D), 1.5, 1, d).float() + 0.3
    w = b = None
    if mode == 0:
        w, b = rnd((D,), 0.5, 2, d).float() + 1, rnd((D,), 0.5, 3, d).float()
        ref = O.layer_norm(x, w, b)
    elif mode == 1:
        ref = O.rms_norm(x)
    else:
        w = rnd((3 * D,), 0.3, 4, d).float()
        ref, _ = O.ada_rms(x, w)
    assert_close(gpu_ops.norm(x, mode, w, b), ref, what="norm")


# ---------------------------------------------------------------------------------------------------
def ref_attention(q, k, v, scale, mask=None):
    logits = (q.float() @ k.float().t()) * scale
    if mask is not None:
        logits = logits.masked_fill(~mask, float("-inf"))
    return torch.softmax(logits, -1) @ v.float()


@pytest.mark.parametrize("ksplit", [1, 2, 4])
def test_attention_vit(ksplit):
    import vla_ops as gpu_ops
    d = dev()
    nv = 2
    qkv = rnd((nv * 256, 3456), 1.0, 5, d)
    o = torch.zeros(nv * 256, 1152, dtype=torch.bfloat16, device=d)
    gpu_ops.attention(qkv, qkv[:, 1152:], qkv[:, 2304:], ldq=3456, ldk=3456, ldv=3456, ldo=1152, o=o,
                      groups_outer=nv, groups_inner=16,
                      strides=(256 * 3456, 72, 256 * 3456, 72, 256 * 3456, 72, 256 * 1152, 72),
                      n_q=256, n_keys=256, head_dim=72, scale=72 ** -0.5, ksplit=ksplit)
    x = qkv.float().reshape(nv, 256, 3, 16, 72).permute(2, 0, 3, 1, 4)
    ref = torch.softmax((x[0] @ x[1].transpose(-1, -2)) * 72 ** -0.5, -1) @ x[2]
    ref = ref.permute(0, 2, 1, 3).reshape(nv * 256, 1152)
    assert_close(o, ref, what="vit attention")


@pytest.mark.parametrize("P,valid,ksplit", [(256, 256, 1), (256, 256, 4), (300, 277, 2), (788, 788, 1), (20, 20, 1)])
def test_attention_prefix(P, valid, ksplit):
    import vla_ops as gpu_ops
    d = dev()
    q, k, v = rnd((P * 8, 256), 1.0, 6, d), rnd((P, 256), 1.0, 7, d), rnd((P, 256), 1.0, 8, d)
    o = torch.zeros(P * 8, 256, dtype=torch.bfloat16, device=d)
    gpu_ops.attention(q, k, v, ldq=256, ldk=256, ldv=256, ldo=256, o=o, n_q=P * 8, n_keys=P, head_dim=256,
                      prefix_alloc=P, valid_prefix=valid, scale=1 / 16, ksplit=ksplit)
    mask = torch.ones(P * 8, P, dtype=torch.bool, device=d)
    mask[:, valid:] = False
    assert_close(o, ref_attention(q, k, v, 1 / 16, mask), what="prefix attention")


@pytest.mark.parametrize("P,S,valid,restrict,ksplit", [(256, 51, 256, 8, 8), (788, 51, 788, 8, 0), (564, 50, 540, 0, 4),
                                                       (6, 4, 6, 8, 1)])
def test_attention_suffix(P, S, valid, restrict, ksplit):
    import vla_ops as gpu_ops
    d = dev()
    T = P + S
    q, k, v = rnd((S * 8, 256), 1.0, 9, d), rnd((T, 256), 1.0, 10, d), rnd((T, 256), 1.0, 11, d)
    o = torch.zeros(S * 8, 256, dtype=torch.bfloat16, device=d)
    gpu_ops.attention(q, k, v, ldq=256, ldk=256, ldv=256, ldo=256, o=o, n_q=S * 8, n_keys=T, head_dim=256,
                      prefix_alloc=P, valid_prefix=valid, restrict_rows=restrict, scale=1 / 16, ksplit=ksplit)
    mask = torch.ones(S * 8, T, dtype=torch.bool, device=d)
    mask[:, valid:P] = False
    mask[:restrict, P + 1:] = False
    assert_close(o, ref_attention(q, k, v, 1 / 16, mask), what="suffix attention")


@pytest.mark.parametrize("P,valid,ksplit", [(256, 256, 1), (256, 256, 2), (300, 277, 0), (788, 788, 0), (788, 788, 1), (20, 20, 1),
                                            (564, 540, 4)])
def test_attention_tc_prefix(P, valid, ksplit):
    import vla_ops
    d = dev()
    q, k, v = rnd((P * 8, 256), 1.0, 6, d), rnd((P + 51, 256), 1.0, 7, d), rnd((P + 51, 256), 1.0, 8, d)
    o = vla_ops.attention_tc(q, k, v, n_keys=P, prefix_alloc=P, valid_prefix=valid, scale=1 / 16, ksplit=ksplit)
    mask = torch.ones(P * 8, P, dtype=torch.bool, device=d)
    mask[:, valid:] = False
    assert_close(o, ref_attention(q, k[:P], v[:P], 1 / 16, mask), what="tcgen05 prefix attention")


@pytest.mark.parametrize("P,S,valid,restrict,ksplit", [(256, 51, 256, 8, 0), (788, 51, 788, 8, 0), (788, 51, 788, 8, 2),
                                                       (564, 50, 540, 0, 4), (6, 4, 6, 8, 1), (788, 51, 788, 8, 1)])
def test_attention_tc_suffix(P, S, valid, restrict, ksplit):
    import vla_ops
    d = dev()
    T = P + S
    q, k, v = rnd((S * 8, 256), 1.0, 9, d), rnd((T, 256), 1.0, 10, d), rnd((T, 256), 1.0, 11, d)
    o = vla_ops.attention_tc(q, k, v, prefix_alloc=P, valid_prefix=valid, restrict_rows=restrict, scale=1 / 16, ksplit=ksplit)
    mask = torch.ones(S * 8, T, dtype=torch.bool, device=d)
    mask[:, valid:P] = False
    mask[:restrict, P + 1:] = False
    assert_close(o, ref_attention(q, k, v, 1 / 16, mask), what="tcgen05 suffix attention")


# ---------------------------------------------------------------------------------------------------
GEMM_CASES = [
    # tokens, K, N, split, bn
    (51, 1024, 2560, 1, 64), (51, 1024, 2560, 4, 64), (51, 2048, 1024, 8, 64), (51, 4096, 1024, 8, 0),
    (1, 1024, 1024, 1, 0), (50, 32, 1024, 1, 0), (10, 1024, 3072, 2, 64),
    (256, 1152, 3456, 4, 256), (256, 1152, 4304, 2, 0), (256, 640, 1152, 1, 0), (512, 4304, 1152, 8, 128),
    (788, 2048, 2048, 1, 256), (788, 2048, 2048, 2, 128), (564, 2048, 1024, 1, 256), (532, 1024, 1152, 2, 256), (330, 1152, 640, 1, 256), (788, 2048, 2048, 0, 0), (256, 2048, 2560, 0, 0), (768, 1152, 3456, 0, 0), (300, 2048, 512, 8, 128), (100, 1152, 2048, 4, 128),
]


@pytest.mark.parametrize("tokens,K,N,split,bn", GEMM_CASES)
def test_gemm_bias_bf16(tokens, K, N, split, bn):
    import vla_ops as gpu_ops
    d = dev()
    x, w, b = rnd((tokens, K), 1.0, 12, d), rnd((K, N), 0.05, 13, d), rnd((N,), 0.5, 14, d).float()
    out = gpu_ops.gemm(x, w, bias=b, split=split, bn=bn)
    assert_close(out, x.float() @ w.float() + b, what="gemm+bias")


# two 128-feature tiles of one weight per CTA (pair=1): bf16 / residual / QKV epilogues, with and without K split,
# token tiles with a ragged edge, an odd number of feature tiles (the second tile of the last CTA is empty)
@pytest.mark.parametrize("tokens,K,N,split,bn", [(788, 2048, 2048, 1, 256), (788, 4096, 2048, 4, 256), (300, 1152, 1152, 2, 128),
                                                 (256, 1152, 4304, 1, 256), (600, 2048, 384, 1, 128), (51, 1024, 1024, 4, 64)])
def test_gemm_pair_bias_bf16(tokens, K, N, split, bn):
    import vla_ops as gpu_ops
    d = dev()
    x, w, b = rnd((tokens, K), 1.0, 42, d), rnd((K, N), 0.05, 43, d), rnd((N,), 0.5, 44, d).float()
    out = gpu_ops.gemm(x, w, bias=b, split=split, bn=bn, pair=1)
    assert_close(out, x.float() @ w.float() + b, what="paired gemm+bias")


@pytest.mark.parametrize("tokens,K,N,split,gated", [(788, 16384, 2048, 4, False), (788, 2048, 2048, 1, True), (1576, 4304, 1152, 1, False)])
def test_gemm_pair_residual(tokens, K, N, split, gated):
    import vla_ops as gpu_ops
    d = dev()
    x, w = rnd((tokens, K), 1.0, 45, d), rnd((K, N), 0.02, 46, d)
    res = rnd((tokens, N), 1.0, 47, d).float()
    gate = rnd((N,), 1.0, 48, d).float() if gated else None
    bias = rnd((N,), 0.5, 49, d).float()
    out = gpu_ops.gemm(x, w, bias=bias, epi=1, res=res, gate=gate, split=split, bn=256, pair=1)
    y = x.float() @ w.float()
    assert_close(out, res + bias + (y * gate if gated else y), rel=1e-4, what="paired residual")


# tcgen05 CTA pairs (pair=2): two CTAs on neighbouring feature tiles share the activation tile, each loading half of it.
# Ragged token tiles (788 = 4 x 224 with a 116-token tail), an odd number of feature tiles (the last pair's second CTA
# has no features), every K split, and every epilogue the forward uses with them.
@pytest.mark.parametrize("tokens,K,N,split,bn", [(788, 2048, 2048, 1, 256), (788, 4096, 2048, 2, 256), (768, 4352, 1152, 4, 256),
                                                 (300, 1152, 1152, 2, 128), (256, 1152, 4304, 1, 256), (600, 2048, 384, 1, 128),
                                                 (768, 1152, 3456, 1, 256), (130, 2048, 1024, 4, 128), (256, 16384, 2048, 4, 128)])
def test_gemm_cta_pair_bias_bf16(tokens, K, N, split, bn):
    import vla_ops as gpu_ops
    d = dev()
    x, w, b = rnd((tokens, K), 1.0, 72, d), rnd((K, N), 0.05, 73, d), rnd((N,), 0.5, 74, d).float()
    out = gpu_ops.gemm(x, w, bias=b, split=split, bn=bn, pair=2)
    assert_close(out, x.float() @ w.float() + b, what="CTA-pair gemm+bias")


@pytest.mark.parametrize("tokens,K,N,split,gated", [(788, 16384, 2048, 2, False), (788, 2048, 2048, 1, True), (1576, 4304, 1152, 1, False),
                                                    (768, 4304, 1152, 4, False)])
def test_gemm_cta_pair_residual(tokens, K, N, split, gated):
    import vla_ops as gpu_ops
    d = dev()
    x, w = rnd((tokens, K), 1.0, 75, d), rnd((K, N), 0.02, 76, d)
    res = rnd((tokens, N), 1.0, 77, d).float()
    gate = rnd((N,), 1.0, 78, d).float() if gated else None
    bias = rnd((N,), 0.5, 79, d).float()
    out = gpu_ops.gemm(x, w, bias=bias, epi=1, res=res, gate=gate, split=split, bn=256, pair=2)
    y = x.float() @ w.float()
    assert_close(out, res + bias + (y * gate if gated else y), rel=1e-4, what="CTA-pair residual")


@pytest.mark.parametrize("tokens,K,N", [(788, 2048, 1024), (256, 2048, 512), (564, 2048, 16384)])
def test_gemm_cta_pair_geglu(tokens, K, N):
    import vla_ops as gpu_ops
    d = dev()
    x, wg, wu = rnd((tokens, K), 1.0, 80, d), rnd((K, N), 0.03, 81, d), rnd((K, N), 0.03, 82, d)
    ref = O.gelu_tanh(x.float() @ wg.float()) * (x.float() @ wu.float())
    assert_close(gpu_ops.gemm(x, wg, w2=wu, act=3, split=1, bn=256, pair=2), ref, what="CTA-pair geglu")


@pytest.mark.parametrize("tokens,split,bn", [(788, 1, 256), (256, 2, 128), (564, 1, 256)])
def test_gemm_cta_pair_qkv_rope(tokens, split, bn):
    import vla_ops as gpu_ops
    d = dev()
    x, w = rnd((tokens, 2048), 1.0, 83, d), rnd((2048, 2560), 0.03, 84, d)
    q, kc, vc, vt = gpu_ops.gemm(x, w, epi=2, split=split, bn=bn, pair=2,
                                 qkv=dict(kv_rows=tokens, pos_off=0, rows_per_obs=tokens, kv_obs_stride=tokens, kv_row_off=0))
    y = x.float() @ w.float()
    cos, sin = O.rope_table(torch.arange(tokens, device=d))
    qr = O.apply_rope(y[:, :2048].reshape(tokens, 8, 256).transpose(0, 1), cos, sin).transpose(0, 1).reshape(tokens, 2048)
    assert_close(q, qr, what="Q")
    assert_close(kc, O.apply_rope(y[:, 2048:2304], cos, sin), what="K")
    assert_close(vc, y[:, 2304:], what="V")
    assert_close(vt[:, :tokens].t(), y[:, 2304:], what="V transposed")


@pytest.mark.parametrize("act", [1, 2])
def test_gemm_activation(act):
    import vla_ops as gpu_ops
    d = dev()
    x, w, b = rnd((256, 1152), 1.0, 15, d), rnd((1152, 4304), 0.03, 16, d), rnd((4304,), 0.5, 17, d).float()
    y = x.float() @ w.float() + b
    ref = O.gelu_tanh(y) if act == 1 else torch.nn.functional.silu(y)
    assert_close(gpu_ops.gemm(x, w, bias=b, act=act), ref, what="gemm+act")


@pytest.mark.parametrize("tokens,K,N,split,bn", [(51, 1024, 4096, 4, 64), (256, 2048, 1024, 1, 256), (788, 2048, 512, 1, 256),
                                                 (130, 2048, 1024, 2, 128), (40, 1024, 1024, 8, 64), (256, 2048, 1024, 2, 256)])
def test_gemm_geglu(tokens, K, N, split, bn):
    import vla_ops as gpu_ops
    d = dev()
    x, wg, wu = rnd((tokens, K), 1.0, 18, d), rnd((K, N), 0.03, 19, d), rnd((K, N), 0.03, 20, d)
    ref = O.gelu_tanh(x.float() @ wg.float()) * (x.float() @ wu.float())
    assert_close(gpu_ops.gemm(x, wg, w2=wu, act=3, split=split, bn=bn), ref, what="geglu")


@pytest.mark.parametrize("tokens,K,N,split,gated", [(51, 4096, 1024, 8, False), (50, 2048, 1024, 8, True), (788, 16384, 2048, 1, False),
                                                    (256, 16384, 256, 8, False), (50, 1024, 32, 4, False)])
def test_gemm_residual(tokens, K, N, split, gated):
    import vla_ops as gpu_ops
    d = dev()
    x, w = rnd((tokens, K), 1.0, 21, d), rnd((K, N), 0.02, 22, d)
    res = rnd((tokens, N), 2.0, 23, d).float()
    gate = rnd((N,), 1.0, 24, d).float() if gated else None
    bias = rnd((N,), 0.5, 25, d).float()
    out = gpu_ops.gemm(x, w, bias=bias, epi=1, res=res, gate=gate, split=split)
    y = x.float() @ w.float()
    ref = res + bias + (y * gate if gated else y)
    assert_close(out, ref, rel=1e-4, what="residual")


def test_gemm_patch_embed_position_rows():
    import vla_ops as gpu_ops
    d = dev()
    x, w = rnd((512, 640), 0.6, 26, d), rnd((640, 1152), 0.02, 27, d)
    pos = rnd((256, 1152), 0.02, 28, d).float()
    out = gpu_ops.gemm(x, w, epi=1, res=pos, res_mod=256)
    assert_close(out, x.float() @ w.float() + pos.repeat(2, 1), rel=1e-4, what="patch embed")


@pytest.mark.parametrize("tokens,K,pos_off,split", [(51, 1024, 788, 4), (788, 2048, 0, 1), (256, 2048, 0, 4), (300, 1024, 100, 1), (200, 1024, 64, 1)])
def test_gemm_qkv_rope(tokens, K, pos_off, split):
    import vla_ops as gpu_ops
    d = dev()
    x, w = rnd((tokens, K), 1.0, 29, d), rnd((K, 2560), 0.03, 30, d)
    row_off = pos_off
    q, kc, vc, vt = gpu_ops.gemm(x, w, epi=2, split=split,
                             qkv=dict(kv_rows=row_off + tokens, pos_off=pos_off, rows_per_obs=tokens,
                                      kv_obs_stride=row_off + tokens, kv_row_off=row_off))
    y = x.float() @ w.float()
    cos, sin = O.rope_table(torch.arange(tokens, device=d) + pos_off)
    qr = O.apply_rope(y[:, :2048].reshape(tokens, 8, 256).transpose(0, 1), cos, sin).transpose(0, 1).reshape(tokens, 2048)
    kr = O.apply_rope(y[:, 2048:2304], cos, sin)
    assert_close(q, qr, what="Q")
    assert_close(kc[row_off:], kr, what="K")
    assert_close(vc[row_off:], y[:, 2304:], what="V")
    assert_close(vt[:, row_off:row_off + tokens].t(), y[:, 2304:], what="V transposed")
    assert kc[:row_off].abs().max().item() == 0 if row_off else True


@pytest.mark.parametrize("views", [1, 3, 5])
def test_vit_attention_tc(views):
    """SigLIP attention on tcgen05 against plain softmax attention per view and head (pi0_infer.py:588-596)."""
    import vla_ops as gpu_ops
    d = dev()
    qkv = rnd((views * 256, 3456), 1.0, 60 + views, d)
    out = gpu_ops.vit_attention_tc(qkv, scale=72 ** -0.5)
    x = qkv.float().reshape(views, 256, 3, 16, 72)
    q, k, v = (x[:, :, i].permute(0, 2, 1, 3) for i in range(3))          # [views, 16, 256, 72]
    p = torch.softmax(q @ k.transpose(-1, -2) * 72 ** -0.5, dim=-1)
    ref = (p @ v).permute(0, 2, 1, 3).reshape(views * 256, 1152)
    assert_close(out, ref, what="siglip attention")
