"""Batched forwards (independent observations per call, the throughput mode) against the per-observation oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import synth, vla_oracle as O   # noqa: E402


def test_pi0_batch_matches_single_observation_oracle():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pi0_infer import Pi0Inference
    torch.backends.cuda.matmul.allow_tf32 = False
    d = torch.device("cuda")
    B, nv = 3, 2
    ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(7, 0), n_vit_layers=2, n_layers=3)
    ins = [synth.make_inputs(nv, 50, s) for s in range(B)]
    images = torch.stack([i[0] for i in ins])
    state = torch.stack([i[1] for i in ins])
    noise = torch.stack([i[2] for i in ins])
    infer = Pi0Inference(ck, nv, 50, batch=B, n_vit_layers=2, n_layers=3, n_steps=2)
    out = infer.forward(images, state, noise).clone()
    torch.cuda.synchronize()
    assert tuple(out.shape) == (B, 50, 32)
    assert infer._engine.status_word() == 0
    w = {k: v.to(d).float() for k, v in ck.items()}
    for b in range(B):
        vx = O.vision_encoder(w, images[b].to(d).float(), n_layers=2)
        enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
        K, V = O.prefix_encoder(w, enc, n_layers=3)
        want = O.pi0_decoder(w, K, V, state[b].to(d).float(), noise[b].to(d).float(), n_layers=3, n_steps=2)
        err = (out[b].float() - want).abs()
        print("observation %d: max-abs %.3e mean-abs %.3e" % (b, err.max().item(), err.mean().item()))
        assert err.max().item() <= 2e-2 and err.mean().item() <= 3e-3


def test_pi05_batch_shared_prompt():
    """Pi05 in throughput mode: several observations per call, one prompt for all of them (shorter than the prompt
    window, so the valid-length mask and the suffix RoPE start are exercised for every group)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pi05_infer import Pi05Inference
    d = torch.device("cuda")
    B, nv, n_prompt, window = 4, 1, 9, 14
    ck = synth.make_checkpoint("pi05", seed=1, prompt_ids=synth.prompt_ids(n_prompt, 2), n_vit_layers=2, n_layers=3)
    ins = [synth.make_inputs(nv, 50, 10 + s) for s in range(B)]
    images = torch.stack([i[0] for i in ins])
    noise = torch.stack([i[2] for i in ins])
    infer = Pi05Inference(ck, nv, 50, discrete_state_input=False, batch=B, n_vit_layers=2, n_layers=3, n_steps=2,
                          max_prompt_len=window)
    out = infer.forward(images, noise).clone()
    torch.cuda.synchronize()
    assert tuple(out.shape) == (B, 50, 32)
    assert infer._engine.status_word() == 0
    w = {k: v.to(d).float() for k, v in ck.items()}
    pad = torch.zeros(window - n_prompt, 2048, device=d)
    for b in range(B):
        vx = O.vision_encoder(w, images[b].to(d).float(), n_layers=2)
        enc = torch.cat([O.project_vision(w, vx), w["language_embeds"], pad], 0)
        K, V = O.prefix_encoder(w, enc, valid_len=256 * nv + n_prompt, n_layers=3)
        want = O.pi05_decoder(w, K, V, noise[b].to(d).float(), 256 * nv + n_prompt, n_layers=3, n_steps=2)
        err = (out[b].float() - want).abs()
        print("observation %d: max-abs %.3e mean-abs %.3e" % (b, err.max().item(), err.mean().item()))
        assert err.max().item() <= 2e-2 and err.mean().item() <= 3e-3


def test_throughput_configuration_full_depth():
    """Throughput mode at its real shape: 32 observations per forward, 2 views, 20 prompt tokens, chunk 50, full
    depth and 10 Euler steps (17 024 prefix tokens per call).  This is the only shape that drives the paired-tile
    multi-wave GEMMs, the grouped tcgen05 attention over 32 groups and the batched SigLIP attention at depth.
    Observations 0, 13 and 31 are checked against the per-observation oracle."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pi0_infer import Pi0Inference
    torch.backends.cuda.matmul.allow_tf32 = False
    d = torch.device("cuda")
    B, nv = 32, 2
    ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(20, 0))
    ins = [synth.make_inputs(nv, 50, 100 + s) for s in range(B)]
    images = torch.stack([i[0] for i in ins])
    state = torch.stack([i[1] for i in ins])
    noise = torch.stack([i[2] for i in ins])
    infer = Pi0Inference(ck, nv, 50, batch=B)
    out = infer.forward(images, state, noise).clone()
    torch.cuda.synchronize()
    assert tuple(out.shape) == (B, 50, 32)
    assert infer._engine.status_word() == 0
    assert torch.isfinite(out.float()).all()
    del infer
    w = {k: v.to(d).float() for k, v in ck.items()}
    for b in (0, 13, 31):
        vx = O.vision_encoder(w, images[b].to(d).float())
        enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
        K, V = O.prefix_encoder(w, enc)
        want = O.pi0_decoder(w, K, V, state[b].to(d).float(), noise[b].to(d).float())
        err = (out[b].float() - want).abs()
        print("observation %d: max-abs %.3e mean-abs %.3e" % (b, err.max().item(), err.mean().item()))
        assert err.max().item() <= 2e-2 and err.mean().item() <= 3e-3
