"""Shared host logic of Pi0Inference / Pi05Inference: owns one library handle, wraps the library's I/O
buffers as torch tensors without copying, and mirrors the checkpoint-loading semantics of the reference
constructors (pi0_infer.py:1337-1338, pi05_infer.py:666-668)."""
import ctypes as C

import numpy as np

import torch

import _capi


class _DevMem:
    """Exposes a raw device allocation to torch through the CUDA array interface (as int16 words)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<i2", "data": (int(ptr), False),
                                         "version": 2}


def vision_encoder_shapes(nl=27, nle=18):
    return {
        "vision_patch_embedding_w": (14, 14, 3, 1152),
        "vision_patch_embedding_b": (1152,),
        "vision_position_embedding": (256, 1152),
        "vision_attn_qkv_w": (nl, 1152, 3 * 1152),
        "vision_attn_qkv_b": (nl, 3 * 1152),
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
        "encoder_multi_modal_projector_w": (1152, 2048),
        "encoder_multi_modal_projector_b": (2048,),
        "encoder_attn_qkv_w": (nle, 2048, 2560),
        "encoder_attn_o_w": (nle, 2048, 2048),
        "encoder_ffn_gate_w": (nle, 2048, 16384),
        "encoder_ffn_up_w": (nle, 2048, 16384),
        "encoder_ffn_down_w": (nle, 16384, 2048),
    }


class Engine:
    def __init__(self, model, num_views, chunk_size, prompt_len, shapes, batch=1, device=None,
                 n_vit_layers=0, n_layers=0, n_steps=0, flags=0):
        if not torch.cuda.is_available():
            raise RuntimeError("realtime-vla_b200 needs a CUDA device (B200); there is no CPU path")
        self.lib = _capi.lib()
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        cfg = _capi.VlaConfig(model=model, num_views=num_views, chunk_size=chunk_size, prompt_len=prompt_len,
                              batch=batch, device=self.device.index, n_vit_layers=n_vit_layers,
                              n_layers=n_layers, n_steps=n_steps, flags=flags)
        h = C.c_void_p()
        _capi.check(self.lib.vla_create(C.byref(cfg), C.byref(h)))
        self.handle = h
        self.shapes = shapes
        self.batch = batch
        self.chunk_size = chunk_size

    def close(self):
        if getattr(self, "handle", None):
            self.lib.vla_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load(self, key, value):
        """self.weights[key].copy_(value) of the reference: unknown key -> KeyError, wrong shape -> RuntimeError."""
        if key not in self.shapes:
            raise KeyError(key)
        t = value if isinstance(value, torch.Tensor) else torch.as_tensor(value)
        want = tuple(self.shapes[key])
        if tuple(t.shape) != want:
            raise RuntimeError("checkpoint tensor '%s' has shape %s, expected %s" % (key, tuple(t.shape), want))
        t = t.detach()
        if t.dtype == torch.float32:
            dt = _capi.VLA_F32
        else:
            t = t.to(torch.bfloat16)
            dt = _capi.VLA_BF16
        t = t.contiguous()
        shape = (C.c_int64 * max(t.dim(), 1))(*t.shape)
        _capi.check(self.lib.vla_load_weight(self.handle, key.encode(), C.c_void_p(t.data_ptr()), shape, t.dim(), dt),
                    self.handle)

    def finalize(self):
        with torch.cuda.device(self.device):
            _capi.check(self.lib.vla_finalize(self.handle), self.handle)

    def buffer(self, name, shape, dtype=torch.bfloat16):
        ptr, nbytes = C.c_void_p(), C.c_size_t()
        _capi.check(self.lib.vla_buffer(self.handle, name.encode(), C.byref(ptr), C.byref(nbytes)), self.handle)
        raw = torch.as_tensor(_DevMem(ptr.value, nbytes.value), device=self.device)
        if dtype == torch.float32:
            return raw.view(torch.float32).view(shape)
        return raw.view(dtype).view(shape)

    def set_prompt(self, embeds):
        """Prompt rows as embeddings; enqueued on the current stream, like the forward that follows."""
        embeds = embeds.detach().to(device=self.device, dtype=torch.bfloat16).contiguous()
        stream = torch.cuda.current_stream(self.device)
        _capi.check(self.lib.vla_set_prompt(self.handle, C.c_void_p(embeds.data_ptr()), embeds.shape[0],
                                            C.c_void_p(stream.cuda_stream)), self.handle)
        embeds.record_stream(stream)   # the copy may still be reading the rows when this tensor is released

    def set_prompt_ids(self, ids):
        """Prompt as token ids (int, host or device): embedded on the device from 'embedding_weight', inside the graph."""
        ids = torch.as_tensor(ids).detach().to(torch.int32).contiguous()
        stream = torch.cuda.current_stream(self.device)
        _capi.check(self.lib.vla_set_prompt_ids(self.handle, C.c_void_p(ids.data_ptr()), int(ids.numel()),
                                                C.c_void_p(stream.cuda_stream)), self.handle)
        if ids.is_cuda:
            ids.record_stream(stream)

    # ---- the steps either side of the forward (the reference's evaluation script does them with PIL / numpy) ----
    def preprocess_image(self, view, frame, obs=0):
        """uint8 (H, W, 3) RGB frame (numpy array or tensor, host or device) -> resized, padded, normalised view."""
        t = frame if isinstance(frame, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(frame))
        if t.dtype != torch.uint8 or t.dim() != 3 or t.shape[2] != 3:
            raise RuntimeError("camera frame must be uint8 (H, W, 3), got %s %s" % (t.dtype, tuple(t.shape)))
        t = t.contiguous()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _capi.check(self.lib.vla_preprocess_image(self.handle, obs, view, C.c_void_p(t.data_ptr()), t.shape[0], t.shape[1],
                                                  C.c_void_p(stream)), self.handle)
        if not t.is_cuda:
            torch.cuda.current_stream(self.device).synchronize()   # the host frame may be released after the call

    @staticmethod
    def _f64(x, n=None):
        a = np.ascontiguousarray(np.asarray(x, dtype=np.float64).reshape(-1))
        return a, a.ctypes.data_as(C.POINTER(C.c_double))

    def preprocess_state(self, state, a, b, mode, obs=0, want_values=False):
        """mode 0: (state - mean) / (std + 1e-6); mode 1: (state - q01) / (q99 - q01 + 1e-6) * 2 - 1; float64."""
        s, ps = self._f64(state)
        n = s.shape[0]
        (av, pa), (bv, pb) = self._f64(np.asarray(a)[:n]), self._f64(np.asarray(b)[:n])
        if av.shape[0] != n or bv.shape[0] != n:
            raise RuntimeError("statistics shorter than the state")
        out = np.empty(n, np.float64) if want_values else None
        po = out.ctypes.data_as(C.POINTER(C.c_double)) if want_values else None
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _capi.check(self.lib.vla_preprocess_state(self.handle, obs, ps, pa, pb, n, mode, po, C.c_void_p(stream)), self.handle)
        return out

    def postprocess_actions(self, a, b, mode, state_raw, action_dim, obs=0):
        """-> float64 (chunk, action_dim): un-normalised actions, delta -> absolute except the gripper dimensions."""
        (av, pa), (bv, pb) = self._f64(a), self._f64(b)
        sv, ps = self._f64(state_raw)
        out = np.empty((self.chunk_size, action_dim), np.float64)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _capi.check(self.lib.vla_postprocess_actions(self.handle, obs, pa, pb, min(av.shape[0], bv.shape[0]), mode, ps, sv.shape[0],
                                                     action_dim, out.ctypes.data_as(C.POINTER(C.c_double)), C.c_void_p(stream)),
                    self.handle)
        return out

    def forward(self):
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _capi.check(self.lib.vla_forward(self.handle, C.c_void_p(stream)), self.handle)

    def forward_stages(self, mask):
        """Subset of the forward: 1 = vision towers + projector, 2 = prompt + prefix prefill, 4 = action expert."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _capi.check(self.lib.vla_forward_stages(self.handle, int(mask), C.c_void_p(stream)), self.handle)

    # ---- multi-view latency mode: mailboxes of the in-graph NVLink exchange (see include/vla_b200.h) ----
    def link_create(self, n_views=0):
        """Mailbox of a trunk (n_views > 0) or of a tower (0) -> (64-byte IPC handle, pointer valid in this process)."""
        buf, ptr = C.create_string_buffer(64), C.c_void_p()
        if n_views > 0:
            rc = self.lib.vla_link_trunk_create(self.handle, int(n_views), buf, C.byref(ptr))
        else:
            rc = self.lib.vla_link_tower_create(self.handle, buf, C.byref(ptr))
        _capi.check(rc, self.handle)
        return buf.raw, ptr.value

    def link_open(self, ipc_handle):
        """Pointer to another process's mailbox (closed when this engine is destroyed)."""
        ptr = C.c_void_p()
        _capi.check(self.lib.vla_link_open(self.handle, C.create_string_buffer(ipc_handle, 64), C.byref(ptr)), self.handle)
        return ptr.value

    def link_tower_connect(self, trunk_mailbox, view, n_views):
        _capi.check(self.lib.vla_link_tower_connect(self.handle, C.c_void_p(trunk_mailbox), int(view), int(n_views)), self.handle)

    def link_trunk_connect(self, view, tower_mailbox):
        _capi.check(self.lib.vla_link_trunk_connect(self.handle, int(view), C.c_void_p(tower_mailbox)), self.handle)

    def forward_host(self, images, state, noise, out):
        """Host-memory entry: contiguous bf16 CPU tensors in, actions written to `out` (bf16 CPU)."""
        _capi.check(self.lib.vla_forward_host(self.handle, C.c_void_p(images.data_ptr()),
                                              C.c_void_p(state.data_ptr()) if state is not None else None,
                                              C.c_void_p(noise.data_ptr()), C.c_void_p(out.data_ptr())), self.handle)

    def status_word(self):
        w = C.c_int()
        _capi.check(self.lib.vla_status_word(self.handle, C.byref(w)), self.handle)
        return w.value

    def clear_status(self):
        _capi.check(self.lib.vla_clear_status(self.handle), self.handle)

    def expert_timeline(self):
        """(arrive_ns, release_ns) of CTA 0 at every grid barrier of the persistent action-expert kernel."""
        buf = (C.c_ulonglong * 4096)()
        n = C.c_int()
        _capi.check(self.lib.vla_expert_timeline(self.handle, buf, 4096, C.byref(n)), self.handle)
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(n.value // 2)]

    def stats(self):
        n, b = C.c_int(), C.c_size_t()
        _capi.check(self.lib.vla_stats(self.handle, C.byref(n), C.byref(b)), self.handle)
        return n.value, b.value

    def stage_kernels(self):
        """Kernel launches of one forward per stage: [vision, prefix, expert]."""
        n = (C.c_int * 3)()
        _capi.check(self.lib.vla_stage_kernels(self.handle, n), self.handle)
        return list(n)

    def time_stages(self):
        ms = (C.c_float * 3)()
        _capi.check(self.lib.vla_time_stages(self.handle, ms), self.handle)
        return list(ms)
