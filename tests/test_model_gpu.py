"""Whole-path parity on a B200: Pi0Inference / Pi05Inference (CUDA, through the C ABI) against the fp32 oracle
on the same seeded synthetic checkpoint and inputs.  Tolerance of the path for bf16 arithmetic: actions within
max-abs 2e-2 and mean-abs 3e-3 of the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import synth, vla_oracle as O   # noqa: E402

MAX_ABS, MEAN_ABS = 2e-2, 3e-3


def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    return torch.device("cuda")


def report(name, got, want):
    err = (got.float() - want.float()).abs()
    print("%s: max-abs %.4e mean-abs %.4e (|want| mean %.3f max %.3f)" %
          (name, err.max().item(), err.mean().item(), want.abs().mean().item(), want.abs().max().item()))
    return err.max().item(), err.mean().item()


def check_actions(got, want):
    assert torch.isfinite(got.float()).all()
    mx, mean = report("actions", got, want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS


def sliced(ck, nlv, nl):
    """First nlv / nl layers of a full-depth checkpoint."""
    out = {}
    for k, v in ck.items():
        if k.startswith("vision_") and v.dim() >= 2 and v.shape[0] == 27 and "patch" not in k and "position" not in k:
            out[k] = v[:nlv]
        elif (k.startswith("encoder_") or k.startswith("decoder_")) and v.dim() >= 2 and v.shape[0] == 18:
            out[k] = v[:nl]
        else:
            out[k] = v
    return out


@pytest.fixture(scope="module")
def small_pi0():
    ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(5, 0), n_vit_layers=2, n_layers=3)
    return ck


def test_pi0_small_intermediates(small_pi0):
    from pi0_infer import Pi0Inference
    d = dev()
    ck = small_pi0
    images, state, noise = synth.make_inputs(1, 50, 0)
    infer = Pi0Inference(ck, 1, 50, n_vit_layers=2, n_layers=3, n_steps=2)
    out = infer.forward(images, state, noise).clone()
    torch.cuda.synchronize()
    assert infer._engine.status_word() == 0
    w = {k: v.to(d).float() for k, v in ck.items()}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
    enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
    K, V = O.prefix_encoder(w, enc, n_layers=3)
    want = O.pi0_decoder(w, K, V, state.to(d).float(), noise.to(d).float(), n_layers=3, n_steps=2)
    P, S = 256 + 5, 51
    e = infer._engine
    mx, _ = report("vision_x", e.buffer("vision_x", (256, 1152), torch.float32), vx)
    assert mx < 3e-2 * vx.abs().max().item()
    mx, _ = report("K cache", e.buffer("encoder_K", (3, P + S, 256))[:, :P], K)
    assert mx < 3e-2 * K.abs().max().item()
    mx, _ = report("V cache", e.buffer("encoder_V", (3, P + S, 256))[:, :P], V)
    assert mx < 3e-2 * V.abs().max().item()
    check_actions(out, want)


@pytest.mark.parametrize("model,nv,chunk,n_prompt", [("pi0", 2, 10, 0), ("pi0", 1, 100, 3), ("pi0", 3, 63, 17), ("pi0", 1, 1, 2),
                                                    ("pi05", 2, 16, 7), ("pi05", 1, 120, 1), ("pi05", 3, 64, 30)])
def test_other_shapes(model, nv, chunk, n_prompt):
    """Chunk sizes other than 50 (suffix token counts on both sides of the 64- and 128-token tiles), every number
    of views, short and empty prompts: reduced-depth models against the oracle."""
    d = dev()
    ck = synth.make_checkpoint(model, seed=3, prompt_ids=synth.prompt_ids(n_prompt, 4), n_vit_layers=1, n_layers=2)
    images, state, noise = synth.make_inputs(nv, chunk, 2)
    w = {k: v.to(d).float() for k, v in ck.items()}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=1)
    enc = torch.cat([O.project_vision(w, vx), w["language_embeds"].reshape(-1, 2048)], 0)
    P = nv * 256 + n_prompt
    if model == "pi0":
        from pi0_infer import Pi0Inference
        infer = Pi0Inference(ck, nv, chunk, n_vit_layers=1, n_layers=2, n_steps=3)
        out = infer.forward(images, state, noise).clone()
        K, V = O.prefix_encoder(w, enc, n_layers=2)
        want = O.pi0_decoder(w, K, V, state.to(d).float(), noise.to(d).float(), n_layers=2, n_steps=3)
    else:
        from pi05_infer import Pi05Inference
        infer = Pi05Inference(ck, nv, chunk, discrete_state_input=False, n_vit_layers=1, n_layers=2, n_steps=3)
        out = infer.forward(images, noise).clone()
        K, V = O.prefix_encoder(w, enc, valid_len=P, n_layers=2)
        want = O.pi05_decoder(w, K, V, noise.to(d).float(), P, n_layers=2, n_steps=3)
    torch.cuda.synchronize()
    assert infer._engine.status_word() == 0
    assert out.shape == (chunk, 32)
    check_actions(out, want)


@pytest.mark.parametrize("model", ["pi0", "pi05"])
def test_outlier_channels(model):
    """Residual streams of trained transformers carry a few channels that are orders of magnitude larger than the
    rest.  The folded norms keep an un-normalised bf16 copy of the stream, so check that such channels (output
    features of the residual projections scaled x40, everywhere in the ViT, the prefix and the expert) do not
    cost accuracy: same tolerance as for the plain synthetic weights, relative to the size of the actions."""
    d = dev()
    ck = synth.make_checkpoint(model, seed=5, prompt_ids=synth.prompt_ids(6, 5), n_vit_layers=2, n_layers=3)
    g = torch.Generator().manual_seed(99)
    for k in ("vision_attn_o_w", "vision_ffn_down_w", "encoder_attn_o_w", "encoder_ffn_down_w", "decoder_attn_o_w", "decoder_ffn_down_w"):
        w = ck[k].float()
        cols = torch.randperm(w.shape[-1], generator=g)[:6]
        w[..., cols] *= 40.0
        ck[k] = w.to(torch.bfloat16)
    images, state, noise = synth.make_inputs(2, 50, 6)
    if model == "pi0":
        from pi0_infer import Pi0Inference
        infer = Pi0Inference(ck, 2, 50, n_vit_layers=2, n_layers=3, n_steps=3)
        out = infer.forward(images, state, noise).clone()
        w = {k: v.to(d).float() for k, v in ck.items()}
        vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
        enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
        K, V = O.prefix_encoder(w, enc, n_layers=3)
        want = O.pi0_decoder(w, K, V, state.to(d).float(), noise.to(d).float(), n_layers=3, n_steps=3)
    else:
        from pi05_infer import Pi05Inference
        infer = Pi05Inference(ck, 2, 50, discrete_state_input=False, n_vit_layers=2, n_layers=3, n_steps=3)
        out = infer.forward(images, noise).clone()
        w = {k: v.to(d).float() for k, v in ck.items()}
        vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
        enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
        K, V = O.prefix_encoder(w, enc, valid_len=512 + 6, n_layers=3)
        want = O.pi05_decoder(w, K, V, noise.to(d).float(), 512 + 6, n_layers=3, n_steps=3)
    torch.cuda.synchronize()
    assert infer._engine.status_word() == 0
    stream_max = infer._engine.buffer("decoder_x", (50 + (model == "pi0"), 1024), torch.float32).abs().max().item()
    print("largest residual-stream value in the expert: %.1f" % stream_max)
    check_actions(out, want)


def test_pi0_api_semantics(small_pi0):
    from pi0_infer import Pi0Inference
    dev()
    ck = dict(small_pi0)
    images, state, noise = synth.make_inputs(1, 50, 0)
    infer = Pi0Inference(ck, 1, 50, n_vit_layers=2, n_layers=3, n_steps=2)
    a = infer.forward(images, state, noise)
    first = a.clone()
    # returns the internal buffer (same object every call), inputs of any float dtype / device are accepted
    b = infer.forward(images.float().cuda(), state.float(), noise.double())
    assert b is a and b.dtype == torch.bfloat16 and tuple(b.shape) == (50, 32)
    assert torch.equal(first, b.clone())            # deterministic: fixed-order split-K reductions
    host = infer.forward_host(images, state, noise)
    assert torch.equal(host, first.cpu())
    with pytest.raises(RuntimeError):
        infer.forward(images[:, :100], state, noise)
    bad = dict(ck)
    bad["no_such_weight"] = torch.zeros(3)
    with pytest.raises(KeyError):
        Pi0Inference(bad, 1, 50, n_vit_layers=2, n_layers=3, n_steps=2)
    with pytest.raises(KeyError):
        Pi0Inference({k: v for k, v in ck.items() if k != "language_embeds"}, 1, 50)
    bad = dict(ck)
    bad["vision_final_norm_w"] = torch.zeros(7)
    with pytest.raises(RuntimeError):
        Pi0Inference(bad, 1, 50, n_vit_layers=2, n_layers=3, n_steps=2)
    # subset of keys is accepted (the reference's benchmark passes only language_embeds)
    Pi0Inference({"language_embeds": ck["language_embeds"]}, 1, 50, n_vit_layers=1, n_layers=2, n_steps=1)
    # more keys than the path supports
    with pytest.raises(RuntimeError):
        Pi0Inference({"language_embeds": torch.zeros(300, 2048)}, 3, 50, n_vit_layers=1, n_layers=2, n_steps=1)


def test_pi05_small_valid_len():
    from pi05_infer import Pi05Inference
    d = dev()
    ids = synth.prompt_ids(9, 3)
    ck = synth.make_checkpoint("pi05", seed=1, prompt_ids=ids, n_vit_layers=2, n_layers=3)
    images, _, noise = synth.make_inputs(1, 50, 1)
    # prompt window of 16 tokens, 9 of them valid: exercises the prefix-length masks and RoPE start
    infer = Pi05Inference(ck, 1, 50, discrete_state_input=False, n_vit_layers=2, n_layers=3, n_steps=2, max_prompt_len=16)
    out = infer.forward(images, noise).clone()
    torch.cuda.synchronize()
    assert infer._engine.status_word() == 0
    w = {k: v.to(d).float() for k, v in ck.items()}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
    pad = torch.zeros(16 - 9, 2048, device=d)
    enc = torch.cat([O.project_vision(w, vx), w["language_embeds"], pad], 0)
    K, V = O.prefix_encoder(w, enc, valid_len=256 + 9, n_layers=3)
    want = O.pi05_decoder(w, K, V, noise.to(d).float(), 256 + 9, n_layers=3, n_steps=2)
    check_actions(out, want)
    # a different (shorter) prompt per call, as with the tokenizer path
    short = w["language_embeds"][:4]
    out2 = infer.forward(images, noise, prompt_embeds=short.to(torch.bfloat16)).clone()
    enc = torch.cat([O.project_vision(w, vx), short, torch.zeros(12, 2048, device=d)], 0)
    K, V = O.prefix_encoder(w, enc, valid_len=256 + 4, n_layers=3)
    want2 = O.pi05_decoder(w, K, V, noise.to(d).float(), 256 + 4, n_layers=3, n_steps=2)
    check_actions(out2, want2)


def test_pi05_prompt_from_token_ids():
    """discrete_state_input=True with pre-tokenised ids: the library embeds them on the device inside the graph
    (pi05_infer.py:769-785, 811-822).  The gathered prompt rows must be bit-exact, the actions within tolerance."""
    from pi05_infer import Pi05Inference
    d = dev()
    ck = synth.make_checkpoint("pi05", seed=1, prompt_ids=synth.prompt_ids(0, 3), n_vit_layers=2, n_layers=3)
    g = torch.Generator().manual_seed(77)
    vocab = 1000
    ck["embedding_weight"] = (torch.randn(vocab, 2048, generator=g) * 0.02).to(torch.bfloat16)
    images, _, noise = synth.make_inputs(1, 50, 1)
    infer = Pi05Inference(ck, 1, 50, tokenizer_path=None, discrete_state_input=True, n_vit_layers=2, n_layers=3, n_steps=2,
                          max_prompt_len=16)
    w = {k: v.to(d).float() for k, v in ck.items() if k != "embedding_weight"}
    vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
    lang = infer._engine.buffer("language_embeds", (16, 2048))      # the bf16 prompt rows the gather writes
    for n_ids, seed in ((11, 5), (16, 6), (3, 7)):      # a different prompt length per call
        ids = torch.randint(0, vocab, (n_ids,), generator=torch.Generator().manual_seed(seed))
        out = infer.forward(images, noise, token_ids=ids if seed != 6 else ids.to(d)).clone()   # host and device ids
        torch.cuda.synchronize()
        assert infer._engine.status_word() == 0
        prompt = O.pi05_prompt_from_ids(ck["embedding_weight"], ids).to(d)
        assert torch.equal(lang[:n_ids].float(), prompt), "gathered prompt rows differ"
        assert not lang[n_ids:].any(), "rows beyond the prompt must be zero"
        enc = torch.cat([O.project_vision(w, vx), prompt, torch.zeros(16 - n_ids, 2048, device=d)], 0)
        K, V = O.prefix_encoder(w, enc, valid_len=256 + n_ids, n_layers=3)
        want = O.pi05_decoder(w, K, V, noise.to(d).float(), 256 + n_ids, n_layers=3, n_steps=2)
        check_actions(out, want)
    # embeddings still work on the same object, and ids again after them
    short = O.pi05_prompt_from_ids(ck["embedding_weight"], torch.arange(4)).to(torch.bfloat16)
    out_e = infer.forward(images, noise, prompt_embeds=short).clone()
    out_i = infer.forward(images, noise, token_ids=torch.arange(4)).clone()
    torch.cuda.synchronize()
    assert torch.equal(out_e, out_i)
    # an id outside the table is clamped and reported through the status word, not a fault
    infer.forward(images, noise, token_ids=torch.tensor([1, vocab + 5, 2]))
    torch.cuda.synchronize()
    assert infer._engine.status_word() != 0
    with pytest.raises(RuntimeError):
        infer.forward(images, noise, token_ids=torch.arange(17))      # longer than the prompt window
    with pytest.raises(RuntimeError):
        infer.forward(images, noise, task_prompt="pick", state_tokens=None)   # no tokenizer was given


@pytest.mark.parametrize("cfg", [1, 2, 3])
def test_full_configs(cfg):
    """Benchmark configurations 1-3 at full depth (27 / 18 layers, 10 steps)."""
    d = dev()
    c = synth.config(cfg)
    ck = c["checkpoint"]
    images, state, noise = c["inputs"]
    if c["model"] == "pi0":
        from pi0_infer import Pi0Inference
        infer = Pi0Inference(ck, c["num_views"], 50)
        out = infer.forward(images, state, noise).clone()
        want = O.pi0_forward(ck, images, state, noise, device=d)
    else:
        from pi05_infer import Pi05Inference
        infer = Pi05Inference(ck, c["num_views"], 50, discrete_state_input=False)
        out = infer.forward(images, noise).clone()
        want = O.pi05_forward(ck, images, noise, device=d)
    torch.cuda.synchronize()
    assert infer._engine.status_word() == 0
    check_actions(out, want)
    del infer
    torch.cuda.empty_cache()
