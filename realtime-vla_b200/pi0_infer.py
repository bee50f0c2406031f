"""Drop-in for the reference's pi0_infer.py: same class name, constructor and forward signature, same
converted-checkpoint dict (pi0_infer.py:1238-1361 of the reference), running on hand-written sm_100a
kernels in libvla_b200.so instead of Triton.

    from pi0_infer import Pi0Inference
    infer = Pi0Inference(checkpoint, num_views=2, chunk_size=50)
    actions = infer.forward(images, state, noise)      # bf16 (chunk, 32) CUDA tensor
"""
import torch

import _capi
from _engine import Engine, vision_encoder_shapes


def pi0_shapes(prompt_len, nlv=27, nl=18):
    s = vision_encoder_shapes(nlv, nl)
    s.update({
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
        "language_embeds": (prompt_len, 2048),
    })
    return s


class Pi0Inference:
    """Pi0Inference(checkpoint, num_views, chunk_size).forward(images, state, noise).

    checkpoint: dict of the converted-checkpoint keys; any subset, 'language_embeds' (prompt_len, 2048)
    required (its row count is the prompt length, 0 rows allowed); unknown key -> KeyError; values may live
    on any device in any float dtype.  forward() copies its arguments into static buffers, replays one CUDA
    graph on the current stream without synchronising, and returns the internal bf16 (chunk, 32) buffer
    (overwritten by the next call), exactly as the reference does.

    Extra keyword arguments (not in the reference): batch (independent observations per forward; inputs
    then carry a leading batch dimension), device, and reduced layer/step counts used by the tests.
    """

    def __init__(self, checkpoint, num_views, chunk_size, *, batch=1, device=None, n_vit_layers=0, n_layers=0,
                 n_steps=0, flags=0):
        self.num_views = num_views
        self.chunk_size = chunk_size
        encoded_prompt = checkpoint["language_embeds"]
        self.prompt_len = len(encoded_prompt)
        shapes = pi0_shapes(self.prompt_len, n_vit_layers or 27, n_layers or 18)
        self._engine = Engine(_capi.VLA_PI0, num_views, chunk_size, self.prompt_len, shapes, batch=batch,
                              device=device, n_vit_layers=n_vit_layers, n_layers=n_layers, n_steps=n_steps,
                              flags=flags)
        for k, v in checkpoint.items():
            self._engine.load(k, v)
        self._engine.finalize()
        lead = (batch,) if batch > 1 else ()
        self.buffers = {
            "observation_images_normalized": self._engine.buffer("observation_images_normalized",
                                                                 lead + (num_views, 224, 224, 3)),
            "observation_state_normalized": self._engine.buffer("observation_state_normalized", lead + (32,)),
            "diffusion_noise": self._engine.buffer("diffusion_noise", lead + (chunk_size, 32)),
        }

    def forward(self, observation_images_normalized, observation_state_normalized, diffusion_noise):
        self.buffers["observation_images_normalized"].copy_(observation_images_normalized)
        self.buffers["observation_state_normalized"].copy_(observation_state_normalized)
        self.buffers["diffusion_noise"].copy_(diffusion_noise)
        self._engine.forward()
        return self.buffers["diffusion_noise"]

    def forward_host(self, images, state, noise):
        """Same computation for callers holding host memory: bf16 CPU tensors in, bf16 CPU actions out,
        host<->device copies and the synchronisation inside the library call."""
        out = torch.empty_like(noise)
        self._engine.forward_host(images.contiguous(), state.contiguous(), noise.contiguous(), out)
        return out
