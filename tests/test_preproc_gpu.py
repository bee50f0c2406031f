"""GPU: the device pre/post-processing (vla_preprocess_image / _state, vla_postprocess_actions, RobotIO) against
the oracle restatement and the fixtures produced by the reference's own code.  Everything here is bit-exact."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "realtime-vla_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)
from oracle import preproc_oracle as P  # noqa: E402
from oracle import synth  # noqa: E402
from tests.test_preproc_oracle import FRAMES, GOLD, stats  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pi0():
    from pi0_infer import Pi0Inference
    ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(4, 0), n_vit_layers=1, n_layers=2)
    return Pi0Inference(ck, 3, 50, n_vit_layers=1, n_layers=2, n_steps=2), ck


def want_view(resized_u8):
    return torch.from_numpy(P.normalize_image(resized_u8)).to(torch.bfloat16)


@pytest.mark.parametrize("h,w,seed", FRAMES)
def test_image_matches_reference_fixture(pi0, h, w, seed):
    infer, _ = pi0
    frame = P.synthetic_frame(h, w, seed)
    infer._engine.preprocess_image(1, frame)
    torch.cuda.synchronize()
    got = infer.buffers["observation_images_normalized"][1].cpu()
    assert torch.equal(got, want_view(GOLD["resized_%dx%d_%d" % (h, w, seed)]))


@pytest.mark.parametrize("h,w", [(720, 1280), (224, 300), (224, 224), (1080, 1920), (50, 37), (225, 224), (17, 400), (480, 640)])
def test_image_matches_oracle(pi0, h, w):
    infer, _ = pi0
    frame = P.synthetic_frame(h, w, 3 * h + w)
    # host numpy frame into view 0, the same frame as a device tensor into view 2
    infer._engine.preprocess_image(0, frame)
    infer._engine.preprocess_image(2, torch.from_numpy(frame).cuda())
    torch.cuda.synchronize()
    want = want_view(P.resize_with_pad(frame))
    buf = infer.buffers["observation_images_normalized"].cpu()
    assert torch.equal(buf[0], want) and torch.equal(buf[2], want)


def test_image_argument_errors(pi0):
    infer, _ = pi0
    with pytest.raises(RuntimeError):
        infer._engine.preprocess_image(3, P.synthetic_frame(100, 100, 1))          # only 3 views
    with pytest.raises(RuntimeError):
        infer._engine.preprocess_image(0, np.zeros((100, 100), np.uint8))           # not (H, W, 3)
    with pytest.raises(RuntimeError):
        infer._engine.preprocess_image(0, np.zeros((1, 2000, 3), np.uint8))         # resizes to zero rows


def test_state_pi0(pi0):
    infer, _ = pi0
    ns = {"state": stats(11, 14)}
    state = (np.random.RandomState(21).randn(14) * 2).astype(np.float32)
    vals = infer._engine.preprocess_state(state, ns["state"]["mean"], ns["state"]["std"], 0, want_values=True)
    want = P.normalize_state(state, ns, "pi0", 14)
    assert np.array_equal(vals, want) and np.array_equal(vals, GOLD["state_norm_pi0"])
    buf = infer.buffers["observation_state_normalized"].cpu()
    want32 = torch.zeros(32)
    want32[:14] = torch.from_numpy(want.astype(np.float32))
    assert torch.equal(buf, want32.to(torch.bfloat16))


def test_state_pi05_formula(pi0):
    infer, _ = pi0
    ns = {"state": stats(11, 14)}
    state = (np.random.RandomState(21).randn(14) * 2).astype(np.float32)
    vals = infer._engine.preprocess_state(state, ns["state"]["q01"], ns["state"]["q99"], 1, want_values=True)
    assert np.array_equal(vals, GOLD["state_norm_pi05"])
    assert np.array_equal(np.digitize(vals, bins=np.linspace(-1, 1, 257)[:-1]) - 1, GOLD["state_digitized"])


@pytest.mark.parametrize("mode,action_dim", [(0, 7), (0, 14), (1, 14), (1, 10), (0, 32)])
def test_postprocess_actions(pi0, mode, action_dim):
    infer, _ = pi0
    model = "pi05" if mode else "pi0"
    st = {"actions": stats(12, 32 if action_dim > 14 else 14)}
    r = np.random.RandomState(31)
    actions = torch.from_numpy(r.randn(50, 32).astype(np.float32)).to(torch.bfloat16)
    state = r.randn(32 if action_dim > 14 else 14).astype(np.float32)
    infer.buffers["diffusion_noise"].copy_(actions)
    a, b = (st["actions"]["q01"], st["actions"]["q99"]) if mode else (st["actions"]["mean"], st["actions"]["std"])
    got = infer._engine.postprocess_actions(a, b, mode, state, action_dim)
    want = P.postprocess_actions(actions.float().numpy(), st, model, state, action_dim)
    assert got.shape == want.shape and np.array_equal(got, want)


def test_robot_loop_step(pi0):
    """Raw frames + raw state + noise -> robot actions through RobotIO equals the host pre/post-processing of the
    oracle around the same forward."""
    from robot_io import RobotIO
    infer, ck = pi0
    ns = {"state": stats(11, 14), "actions": stats(12, 14)}
    io = RobotIO(infer, ns, action_dim=14)
    frames = [P.synthetic_frame(480, 640, 1), P.synthetic_frame(360, 640, 2), P.synthetic_frame(300, 200, 3)]
    state = (np.random.RandomState(4).randn(14)).astype(np.float32)
    noise = synth.make_inputs(3, 50, 0)[2]
    got = io.step(frames, state, noise)
    # the same step with the oracle's host pre/post-processing around the plain forward
    imgs = torch.stack([torch.from_numpy(P.normalize_image(P.resize_with_pad(f))) for f in frames])
    s32 = torch.zeros(32)
    s32[:14] = torch.from_numpy(P.normalize_state(state, ns, "pi0", 14).astype(np.float32))
    act = infer.forward(imgs, s32, noise).float().cpu().numpy()
    want = P.postprocess_actions(act, ns, "pi0", state, 14)
    assert np.array_equal(got, want)
