"""ctypes binding of libvla_b200.so (C ABI in include/vla_b200.h).  No CPU fallback: importing works
anywhere, but every call needs the compiled library and a B200."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvla_b200.so")

VLA_PI0, VLA_PI05 = 0, 1
VLA_BF16, VLA_F32 = 0, 1
ERRORS = {1: "CUDA", 2: "KEY", 3: "SHAPE", 4: "STATE", 5: "LIMIT", 6: "DEVICE"}


class VlaConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("model", "num_views", "chunk_size", "prompt_len", "batch", "device",
                                       "n_vit_layers", "n_layers", "n_steps", "flags")]


class GemmDesc(C.Structure):
    _fields_ = [("x", C.c_void_p), ("tokens", C.c_int), ("K", C.c_int),
                ("w", C.c_void_p), ("w2", C.c_void_p), ("N", C.c_int),
                ("bias", C.c_void_p), ("epi", C.c_int), ("act", C.c_int),
                ("out_bf16", C.c_void_p), ("ld_out", C.c_int),
                ("out_f32", C.c_void_p), ("res", C.c_void_p), ("gate", C.c_void_p), ("res_mod", C.c_int),
                ("q", C.c_void_p), ("kcache", C.c_void_p), ("vcache", C.c_void_p), ("vt", C.c_void_p), ("vt_ld", C.c_int),
                ("pos_off", C.c_int), ("rows_per_obs", C.c_int), ("kv_obs_stride", C.c_int), ("kv_row_off", C.c_int),
                ("split", C.c_int), ("bn", C.c_int), ("iters", C.c_int), ("ms_per_iter", C.POINTER(C.c_float)),
                ("pair", C.c_int), ("tok_tile", C.c_int)]


class AttnDesc(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("ldq", C.c_int), ("ldk", C.c_int), ("ldv", C.c_int), ("ldo", C.c_int),
                ("groups_outer", C.c_int), ("groups_inner", C.c_int),
                ("q_go", C.c_longlong), ("q_gi", C.c_longlong), ("k_go", C.c_longlong), ("k_gi", C.c_longlong),
                ("v_go", C.c_longlong), ("v_gi", C.c_longlong), ("o_go", C.c_longlong), ("o_gi", C.c_longlong),
                ("n_q", C.c_int), ("n_keys", C.c_int), ("head_dim", C.c_int),
                ("prefix_alloc", C.c_int), ("valid_prefix", C.c_int), ("restrict_rows", C.c_int),
                ("scale", C.c_float), ("ksplit", C.c_int), ("iters", C.c_int), ("ms_per_iter", C.POINTER(C.c_float))]


class AttnTcDesc(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("vt", C.c_void_p), ("o", C.c_void_p),
                ("n_q", C.c_int), ("n_keys", C.c_int), ("k_rows", C.c_int), ("vt_ld", C.c_int),
                ("prefix_alloc", C.c_int), ("valid_prefix", C.c_int), ("restrict_rows", C.c_int),
                ("scale", C.c_float), ("ksplit", C.c_int), ("iters", C.c_int), ("ms_per_iter", C.POINTER(C.c_float))]


class GemmNoAllocDesc(C.Structure):
    _fields_ = [("x", C.c_void_p), ("tokens", C.c_int), ("K", C.c_int),
                ("w_nk", C.c_void_p), ("N", C.c_int), ("n_pad", C.c_int), ("k_pad", C.c_int),
                ("bias", C.c_void_p), ("out_bf16", C.c_void_p), ("split", C.c_int)]


EXPORTS = {
    "vla_create": (C.c_int, [C.POINTER(VlaConfig), C.POINTER(C.c_void_p)]),
    "vla_load_weight": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.POINTER(C.c_int64), C.c_int, C.c_int]),
    "vla_finalize": (C.c_int, [C.c_void_p]),
    "vla_set_prompt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "vla_buffer": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "vla_forward": (C.c_int, [C.c_void_p, C.c_void_p]),
    "vla_forward_stages": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "vla_link_trunk_create": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_void_p)]),
    "vla_link_tower_create": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "vla_link_open": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "vla_link_tower_connect": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "vla_link_trunk_connect": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "vla_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "vla_status_word": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "vla_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_size_t)]),
    "vla_set_prompt_ids": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "vla_op_vit_attention_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_int, C.POINTER(C.c_float), C.c_void_p]),
    "vla_preprocess_image": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "vla_preprocess_state": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                       C.c_int, C.c_int, C.POINTER(C.c_double), C.c_void_p]),
    "vla_postprocess_actions": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_int, C.c_int,
                                          C.POINTER(C.c_double), C.c_int, C.c_int, C.POINTER(C.c_double), C.c_void_p]),
    "vla_time_stages": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "vla_stage_kernels": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "vla_destroy": (C.c_int, [C.c_void_p]),
    "vla_last_error": (C.c_char_p, [C.c_void_p]),
    "vla_op_gemm": (C.c_int, [C.POINTER(GemmDesc), C.c_void_p]),
    "vla_op_gemm_noalloc": (C.c_int, [C.POINTER(GemmNoAllocDesc), C.c_void_p]),
    "vla_op_gemm_noalloc_status": (C.c_int, [C.POINTER(C.c_int)]),
    "vla_clear_status": (C.c_int, [C.c_void_p]),
    "vla_expert_timeline": (C.c_int, [C.c_void_p, C.POINTER(C.c_ulonglong), C.c_int, C.POINTER(C.c_int)]),
    "vla_op_attention": (C.c_int, [C.POINTER(AttnDesc), C.c_void_p]),
    "vla_op_attention_tc": (C.c_int, [C.POINTER(AttnTcDesc), C.c_void_p]),
    "vla_op_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def lib():
    """Load the shared library (raises if it has not been built: there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("libvla_b200.so is not built; run `python realtime-vla_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class VlaError(RuntimeError):
    pass


def check(rc, handle=None):
    if rc == 0:
        return
    msg = lib().vla_last_error(handle)
    msg = msg.decode() if msg else ""
    text = "libvla_b200 error %s: %s" % (ERRORS.get(rc, rc), msg)
    if rc == 2:
        raise KeyError(text)          # the reference raises KeyError for an unknown checkpoint key
    raise VlaError(text)
