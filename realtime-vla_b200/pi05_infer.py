"""Drop-in for the reference's pi05_infer.py (pi05_infer.py:530-826 of the reference): same class name,
constructor and forward signature, same converted-checkpoint dict, on the kernels of libvla_b200.so.

    from pi05_infer import Pi05Inference
    infer = Pi05Inference(checkpoint, num_views=2, chunk_size=50, discrete_state_input=False)
    actions = infer.forward(images, noise)
"""
import numpy as np
import torch

import _capi
from _engine import Engine, vision_encoder_shapes


def pi05_shapes(lang_rows, nlv=27, nl=18):
    s = vision_encoder_shapes(nlv, nl)
    s.update({
        "decoder_time_embeds": (10, 1024),
        "decoder_time_mlp_in_w": (1024, 1024),
        "decoder_time_mlp_in_b": (1024,),
        "decoder_time_mlp_out_w": (1024, 1024),
        "decoder_time_mlp_out_b": (1024,),
        "decoder_action_in_proj_w": (32, 1024),
        "decoder_action_in_proj_b": (1024,),
        "decoder_pre_attn_norm_mod_w": (nl, 1024, 3 * 1024),
        "decoder_pre_attn_norm_mod_b": (nl, 3 * 1024),
        "decoder_pre_ffn_norm_mod_w": (nl, 1024, 3 * 1024),
        "decoder_pre_ffn_norm_mod_b": (nl, 3 * 1024),
        "decoder_attn_qkv_w": (nl, 1024, 2560),
        "decoder_attn_o_w": (nl, 2048, 1024),
        "decoder_ffn_gate_w": (nl, 1024, 4096),
        "decoder_ffn_up_w": (nl, 1024, 4096),
        "decoder_ffn_down_w": (nl, 4096, 1024),
        "decoder_action_out_proj_w": (1024, 32),
        "decoder_action_out_proj_b": (32,),
        "decoder_final_norm_mod_w": (1024, 3 * 1024),
        "decoder_final_norm_mod_b": (3 * 1024,),
        "language_embeds": (lang_rows, 2048),
    })
    return s


class Pi05Inference:
    """Pi05Inference(checkpoint, num_views, chunk_size, tokenizer_path=None, max_tokenize_len=200,
    discrete_state_input=True, max_prompt_text=None, state_dim_for_max_prompt=None)
    .forward(images, noise, task_prompt=None, state_tokens=None)

    With discrete_state_input=False the prompt is checkpoint['language_embeds'] and no tokenizer is touched.
    With discrete_state_input=True the prompt text "Task: ..., State: ...;\\nAction: " is tokenised on the
    host and only the token ids go to the library: checkpoint['embedding_weight'] lives on the device and the
    embedding (table[ids] * sqrt(2048), bf16) runs inside the captured graph.  The prompt window is
    max_prompt_len tokens and shorter prompts are masked by their valid length.  Callers that tokenise
    themselves pass forward(..., token_ids=ids) and may leave tokenizer_path=None.

    batch (not in the reference): independent observations per forward, inputs then carry a leading batch
    dimension; all observations of one call share the prompt.
    """

    def __init__(self, checkpoint, num_views, chunk_size, tokenizer_path=None, max_tokenize_len=200,
                 discrete_state_input=True, max_prompt_text=None, state_dim_for_max_prompt=None, *,
                 batch=1, device=None, n_vit_layers=0, n_layers=0, n_steps=0, flags=0, max_prompt_len=None):
        self.discrete_state_input = discrete_state_input
        self.tokenizer_path = tokenizer_path
        self.checkpoint = checkpoint
        self.num_views = num_views
        self.chunk_size = chunk_size
        self.max_tokenize_len = int(max_tokenize_len)
        self.tokenizer = None
        if discrete_state_input and tokenizer_path is not None:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
        if discrete_state_input:
            if self.tokenizer is not None and max_prompt_text is not None and state_dim_for_max_prompt is not None:
                self.max_prompt_len = self.estimate_max_prompt_len(self.tokenizer, max_prompt_text,
                                                                   int(state_dim_for_max_prompt),
                                                                   self.max_tokenize_len, 255)
            else:
                self.max_prompt_len = self.max_tokenize_len
        else:
            self.max_prompt_len = len(checkpoint["language_embeds"])
        if max_prompt_len is not None:        # explicit prompt window (not in the reference; used by the tests)
            self.max_prompt_len = int(max_prompt_len)
        lang_rows = len(checkpoint["language_embeds"])
        shapes = pi05_shapes(lang_rows, n_vit_layers or 27, n_layers or 18)
        if discrete_state_input:
            if "embedding_weight" not in checkpoint:
                raise KeyError("checkpoint must contain 'embedding_weight' when discrete_state_input=True")
            shapes["embedding_weight"] = tuple(checkpoint["embedding_weight"].shape)
        self._engine = Engine(_capi.VLA_PI05, num_views, chunk_size, self.max_prompt_len, shapes, batch=batch, device=device,
                              n_vit_layers=n_vit_layers, n_layers=n_layers, n_steps=n_steps, flags=flags)
        for k, v in checkpoint.items():
            if k == "embedding_weight" and not discrete_state_input:
                continue            # the reference skips the table in this mode (pi05_infer.py:666-668)
            self._engine.load(k, torch.from_numpy(v) if isinstance(v, np.ndarray) else v)
        self._prompt_embed_scale = float(2048 ** 0.5) if discrete_state_input else None
        self._language_embeds = checkpoint["language_embeds"]
        self.encoder_seq_len = num_views * 256 + self.max_prompt_len
        self._engine.finalize()
        lead = (batch,) if batch > 1 else ()
        self.buffers = {
            "observation_images_normalized": self._engine.buffer("observation_images_normalized",
                                                                 lead + (num_views, 224, 224, 3)),
            "diffusion_noise": self._engine.buffer("diffusion_noise", lead + (chunk_size, 32)),
        }

    def estimate_max_prompt_len(self, tokenizer, task_prompt, state_dim, max_tokenize_len=200, state_token_value=255):
        task_prompt = task_prompt.strip().replace("_", " ")
        state_str = " ".join([str(int(state_token_value))] * int(state_dim))
        full_prompt = f"Task: {task_prompt}, State: {state_str};\nAction: "
        ids = tokenizer(full_prompt, return_tensors="pt", truncation=True, max_length=int(max_tokenize_len),
                        padding=False)["input_ids"][0]
        return int(ids.shape[0])

    def build_prompt_ids(self, task_prompt, state_tokens):
        """Token ids of the reference's prompt text (pi05_infer.py:769-783); the embedding happens on the device."""
        if self.tokenizer is None:
            raise RuntimeError("no tokenizer (tokenizer_path=None): pass token_ids to forward()")
        task_prompt = task_prompt.strip().replace("_", " ")
        state_str = " ".join(map(str, state_tokens.tolist()))
        full_prompt = f"Task: {task_prompt}, State: {state_str};\nAction: "
        return self.tokenizer(full_prompt, return_tensors="pt", truncation=True, max_length=self.max_tokenize_len,
                              padding=False)["input_ids"][0]

    def build_prompt_embeds(self, task_prompt, state_tokens):
        """Same result as the reference's method (embeddings, length), computed on the host from the checkpoint
        table; forward() does not use it."""
        ids = self.build_prompt_ids(task_prompt, state_tokens)
        table = self.checkpoint["embedding_weight"]
        table = torch.from_numpy(table) if isinstance(table, np.ndarray) else table
        embeds = table[ids.to(table.device)].to(torch.bfloat16) * self._prompt_embed_scale
        return embeds, int(embeds.shape[0])

    def forward(self, observation_images_normalized, diffusion_noise, task_prompt=None, state_tokens=None,
                prompt_embeds=None, token_ids=None):
        if prompt_embeds is not None:          # pre-embedded prompt (not in the reference)
            self._engine.set_prompt(prompt_embeds)
        elif token_ids is not None:            # pre-tokenised prompt (not in the reference)
            self._engine.set_prompt_ids(token_ids)
        elif self.discrete_state_input:
            self._engine.set_prompt_ids(self.build_prompt_ids(task_prompt, state_tokens))
        self.buffers["observation_images_normalized"].copy_(observation_images_normalized)
        self.buffers["diffusion_noise"].copy_(diffusion_noise)
        self._engine.forward()
        return self.buffers["diffusion_noise"]

    def forward_host(self, images, noise):
        out = torch.empty_like(noise)
        self._engine.forward_host(images.contiguous(), None, noise.contiguous(), out)
        return out
