"""Python callers of the single-operator C-ABI entry points (vla_op_*): kernel-level parity tests and
micro-benchmarks call the kernels through these."""
import ctypes as C

import torch

import _capi


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def gemm(x, w, *, w2=None, bias=None, epi=0, act=0, res=None, gate=None, res_mod=0, split=0, bn=0, pair=0, tok_tile=0, iters=0,
         qkv=None):
    """x bf16 [tokens,K], w bf16 [K,N] (checkpoint layout). Returns the epilogue's output tensor(s)."""
    lib = _capi.lib()
    tokens, K = x.shape
    N = w.shape[1]
    d = _capi.GemmDesc()
    d.x, d.tokens, d.K, d.w, d.w2, d.N = _p(x), tokens, K, _p(w), _p(w2), N
    d.bias, d.epi, d.act = _p(bias), epi, act
    d.split, d.bn, d.iters, d.pair, d.tok_tile = split, bn, iters, pair, tok_tile
    ms = C.c_float(0)
    d.ms_per_iter = C.pointer(ms)
    out = None
    if epi == 0:
        out = torch.full((tokens, N), float("nan"), dtype=torch.bfloat16, device=x.device)
        d.out_bf16, d.ld_out = _p(out), N
    elif epi == 1:
        out = res.clone() if (res is not None and res_mod == 0) else torch.zeros(tokens, N, device=x.device)
        d.out_f32 = _p(out)
        d.res = _p(out) if (res is not None and res_mod == 0) else _p(res)
        d.gate, d.res_mod = _p(gate), res_mod
    else:
        q = torch.zeros(tokens, 2048, dtype=torch.bfloat16, device=x.device)
        rows = qkv["kv_rows"]
        kc = torch.zeros(rows, 256, dtype=torch.bfloat16, device=x.device)
        vc = torch.zeros(rows, 256, dtype=torch.bfloat16, device=x.device)
        vt_ld = (rows + 7) // 8 * 8
        vt = torch.zeros(256, vt_ld, dtype=torch.bfloat16, device=x.device)
        d.q, d.kcache, d.vcache, d.vt, d.vt_ld = _p(q), _p(kc), _p(vc), _p(vt), vt_ld
        d.pos_off, d.rows_per_obs = qkv["pos_off"], qkv["rows_per_obs"]
        d.kv_obs_stride, d.kv_row_off = qkv["kv_obs_stride"], qkv["kv_row_off"]
        out = (q, kc, vc, vt)
    rc = lib.vla_op_gemm(C.byref(d), None)
    _capi.check(rc)
    torch.cuda.synchronize()
    return (out, ms.value) if iters else out


def attention(q, k, v, *, ldq, ldk, ldv, ldo, o, groups_outer=1, groups_inner=1, strides=(0,) * 8, n_q, n_keys, head_dim,
              prefix_alloc=None, valid_prefix=None, restrict_rows=0, scale, ksplit=0, iters=0):
    lib = _capi.lib()
    d = _capi.AttnDesc()
    d.q, d.k, d.v, d.o = _p(q), _p(k), _p(v), _p(o)
    d.ldq, d.ldk, d.ldv, d.ldo = ldq, ldk, ldv, ldo
    d.groups_outer, d.groups_inner = groups_outer, groups_inner
    d.q_go, d.q_gi, d.k_go, d.k_gi, d.v_go, d.v_gi, d.o_go, d.o_gi = strides
    d.n_q, d.n_keys, d.head_dim = n_q, n_keys, head_dim
    d.prefix_alloc = n_keys if prefix_alloc is None else prefix_alloc
    d.valid_prefix = d.prefix_alloc if valid_prefix is None else valid_prefix
    d.restrict_rows, d.scale, d.ksplit, d.iters = restrict_rows, scale, ksplit, iters
    ms = C.c_float(0)
    d.ms_per_iter = C.pointer(ms)
    _capi.check(lib.vla_op_attention(C.byref(d), None))
    torch.cuda.synchronize()
    return ms.value


def attention_tc(q, k, v, *, n_keys=None, prefix_alloc=None, valid_prefix=None, restrict_rows=0, scale, ksplit=0, iters=0):
    """tcgen05 attention: q [n_q,256], k/v [k_rows,256] bf16 (v is transposed here into the layout the kernel reads)."""
    lib = _capi.lib()
    n_q, k_rows = q.shape[0], k.shape[0]
    n_keys = k_rows if n_keys is None else n_keys
    vt_ld = (k_rows + 7) // 8 * 8
    vt = torch.zeros(256, vt_ld, dtype=torch.bfloat16, device=q.device)
    vt[:, :k_rows] = v.t()
    o = torch.zeros(n_q, 256, dtype=torch.bfloat16, device=q.device)
    d = _capi.AttnTcDesc()
    d.q, d.k, d.vt, d.o = _p(q), _p(k), _p(vt), _p(o)
    d.n_q, d.n_keys, d.k_rows, d.vt_ld = n_q, n_keys, k_rows, vt_ld
    d.prefix_alloc = n_keys if prefix_alloc is None else prefix_alloc
    d.valid_prefix = d.prefix_alloc if valid_prefix is None else valid_prefix
    d.restrict_rows, d.scale, d.ksplit, d.iters = restrict_rows, scale, ksplit, iters
    ms = C.c_float(0)
    d.ms_per_iter = C.pointer(ms)
    _capi.check(lib.vla_op_attention_tc(C.byref(d), None))
    torch.cuda.synchronize()
    return (o, ms.value) if iters else o


def norm(x, mode, w=None, b=None):
    lib = _capi.lib()
    rows, D = x.shape
    y = torch.empty(rows, D, dtype=torch.bfloat16, device=x.device)
    _capi.check(lib.vla_op_norm(_p(x), _p(y), rows, D, mode, _p(w), _p(b), None))
    return y


def vit_attention_tc(qkv, *, scale, iters=0):
    """SigLIP attention on tcgen05: qkv bf16 [views*256, 3456] -> bf16 [views*256, 1152]."""
    lib = _capi.lib()
    views = qkv.shape[0] // 256
    out = torch.full((views * 256, 1152), float("nan"), dtype=torch.bfloat16, device=qkv.device)
    ms = C.c_float(0)
    stream = torch.cuda.current_stream(qkv.device).cuda_stream
    _capi.check(lib.vla_op_vit_attention_tc(_p(qkv), _p(out), views, float(scale), iters, C.byref(ms), C.c_void_p(stream)))
    return (out, ms.value) if iters else out
