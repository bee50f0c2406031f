"""The persistent action-expert kernel (one cooperative launch for the whole Euler loop) against the fp32 oracle and
against the per-operator launches it replaces (`flags` bit 4), plus the library behaviour around it: repeatability,
the barrier timeline, prompt updates ordered on the caller's stream, and handles on two devices in one process."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import synth, vla_oracle as O   # noqa: E402

MAX_ABS, MEAN_ABS = 2e-2, 3e-3
PER_OPERATOR = 16


def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda")


def pi0_oracle(ck, images, state, noise, d, nlv, nl, ns):
    w = {k: v.to(d).float() for k, v in ck.items()}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=nlv)
    enc = torch.cat([O.project_vision(w, vx), w["language_embeds"].reshape(-1, 2048)], 0)
    K, V = O.prefix_encoder(w, enc, n_layers=nl)
    return O.pi0_decoder(w, K, V, state.to(d).float(), noise.to(d).float(), n_layers=nl, n_steps=ns)


@pytest.mark.parametrize("chunk,n_prompt", [(50, 20), (55, 0), (7, 3)])
def test_persistent_and_per_operator_paths_agree(chunk, n_prompt):
    """Full expert depth and all 10 Euler steps (2 ViT layers keep the run short): both implementations of the expert
    stage meet the path's tolerance against the oracle, and they agree with each other to bf16 rounding."""
    from pi0_infer import Pi0Inference
    d = dev()
    ck = synth.make_checkpoint("pi0", seed=2, prompt_ids=synth.prompt_ids(n_prompt, 1), n_vit_layers=2)
    images, state, noise = synth.make_inputs(1, chunk, 3)
    want = pi0_oracle(ck, images, state, noise, d, 2, 18, 10)
    outs = []
    for flags in (0, PER_OPERATOR):
        infer = Pi0Inference(ck, 1, chunk, n_vit_layers=2, flags=flags)
        out = infer.forward(images, state, noise).float().clone()
        torch.cuda.synchronize()
        assert infer._engine.status_word() == 0
        n_expert = infer._engine.stage_kernels()[2]
        assert (n_expert == 1) == (flags == 0), "expert stage launches: %d" % n_expert
        err = (out - want).abs()
        print("flags %d: %d expert launches, max-abs %.3e mean-abs %.3e" % (flags, n_expert, err.max().item(), err.mean().item()))
        assert err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS
        outs.append(out)
        del infer
    assert (outs[0] - outs[1]).abs().max().item() <= MAX_ABS


def test_repeatable_and_timeline():
    """Two forwards on the same inputs are bit-identical (the only cross-CTA reduction of the kernel uses integer
    atomics), and the barrier timeline has one (arrival, release) pair per phase, in order."""
    from pi05_infer import Pi05Inference
    d = dev()
    nl, ns = 3, 4
    ck = synth.make_checkpoint("pi05", seed=1, prompt_ids=synth.prompt_ids(9, 2), n_vit_layers=1, n_layers=nl)
    images, _, noise = synth.make_inputs(2, 50, 5)
    infer = Pi05Inference(ck, 2, 50, discrete_state_input=False, n_vit_layers=1, n_layers=nl, n_steps=ns)
    a = infer.forward(images, noise).clone()
    b = infer.forward(images, noise).clone()
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    tl = infer._engine.expert_timeline()
    assert len(tl) == ns * (1 + 6 * nl + 1)
    flat = [t for pair in tl for t in pair]
    assert all(x > 0 for x in flat) and flat == sorted(flat)
    assert infer._engine.status_word() == 0
    # the first forward against the oracle
    w = {k: v.to(d).float() for k, v in ck.items()}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=1)
    enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
    K, V = O.prefix_encoder(w, enc, valid_len=512 + 9, n_layers=nl)
    want = O.pi05_decoder(w, K, V, noise.to(d).float(), 512 + 9, n_layers=nl, n_steps=ns)
    err = (a.float() - want).abs()
    assert err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS


def test_prompt_updates_are_ordered_on_the_callers_stream():
    """Two forwards back to back on a non-default stream with prompts of different lengths: the second prompt's rows,
    valid length and RoPE start are enqueued behind the first forward, so each result matches its own oracle."""
    from pi05_infer import Pi05Inference
    d = dev()
    nl, ns, window = 2, 2, 12
    ck = synth.make_checkpoint("pi05", seed=4, prompt_ids=synth.prompt_ids(window, 3), n_vit_layers=1, n_layers=nl)
    images, _, noise = synth.make_inputs(1, 50, 7)
    infer = Pi05Inference(ck, 1, 50, discrete_state_input=False, n_vit_layers=1, n_layers=nl, n_steps=ns, max_prompt_len=window)
    prompts = [synth.prompt_embeds(synth.prompt_ids(n, 10 + n)).to(d) for n in (11, 4)]
    stream = torch.cuda.Stream()
    outs = []
    with torch.cuda.stream(stream):
        for pe in prompts:
            outs.append(infer.forward(images, noise, prompt_embeds=pe).clone())
    stream.synchronize()
    assert infer._engine.status_word() == 0
    w = {k: v.to(d).float() for k, v in ck.items()}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=1)
    for pe, out in zip(prompts, outs):
        n = pe.shape[0]
        pad = torch.zeros(window - n, 2048, device=d)
        enc = torch.cat([O.project_vision(w, vx), pe.float(), pad], 0)
        K, V = O.prefix_encoder(w, enc, valid_len=256 + n, n_layers=nl)
        want = O.pi05_decoder(w, K, V, noise.to(d).float(), 256 + n, n_layers=nl, n_steps=ns)
        err = (out.float() - want).abs()
        print("prompt of %d rows: max-abs %.3e mean-abs %.3e" % (n, err.max().item(), err.mean().item()))
        assert err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS


def test_handles_on_two_devices():
    """One process, one handle per GPU: kernel attributes and the static scratch of the allocation-free GEMM are kept
    per device, so the second device must work like the first."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from pi0_infer import Pi0Inference
    torch.backends.cuda.matmul.allow_tf32 = False
    ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(4, 0), n_vit_layers=1, n_layers=2)
    images, state, noise = synth.make_inputs(1, 50, 0)
    want = pi0_oracle(ck, images, state, noise, torch.device("cuda", 0), 1, 2, 2)
    infers = [Pi0Inference(ck, 1, 50, device=i, n_vit_layers=1, n_layers=2, n_steps=2) for i in (0, 1)]
    for i, infer in enumerate(infers):
        with torch.cuda.device(i):
            out = infer.forward(images, state, noise).float().clone()
            torch.cuda.synchronize(i)
        assert infer._engine.status_word() == 0
        err = (out.to("cuda:0") - want).abs()
        assert err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS
