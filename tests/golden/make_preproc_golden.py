"""Generates tests/golden/preproc_golden.npz by executing the reference's OWN pre/post-processing methods.

The reference's test.py cannot be imported here (it imports openpi and jax at module level), so the methods
of PiModelEvaluator that make up the image / state / action transforms (test.py:82-151) are taken out of its
syntax tree and compiled into a stub class; nothing of them is copied into this repository.  Inputs are the
deterministic frames and statistics of oracle/preproc_oracle.py, so the test can rebuild them.

Run in the build container (needs the reference checkout, PIL, einops):
    python tests/golden/make_preproc_golden.py /path/to/reference
"""
import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import preproc_oracle as P  # noqa: E402

METHODS = ["_parse_image", "_pad_to_dim", "_resize_with_pad", "_normalize_image", "_normalize_state", "_digitize_state",
           "_unnormalize_actions"]
FRAMES = [(480, 640, 1), (360, 640, 2), (300, 200, 3), (100, 80, 6), (233, 224, 7)]


def reference_class(ref_root):
    src = open(os.path.join(ref_root, "test.py")).read()
    tree = ast.parse(src)
    cls = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "PiModelEvaluator")
    keep = [n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name in METHODS]
    assert len(keep) == len(METHODS), "the reference's test.py no longer has the expected methods"
    stub = ast.ClassDef(name="Ref", bases=[], keywords=[], body=keep, decorator_list=[], type_params=[])
    mod = ast.Module(body=[stub], type_ignores=[])
    ast.fix_missing_locations(mod)
    import einops
    from PIL import Image
    ns = {"np": np, "Image": Image, "einops": einops}
    exec(compile(mod, "reference test.py (methods only)", "exec"), ns)
    return ns["Ref"]


def stats(seed, dim):
    r = np.random.RandomState(seed)
    mean, std = r.randn(dim), np.abs(r.randn(dim)) + 0.1
    q01 = r.randn(dim) - 2.0
    return {"mean": mean.tolist(), "std": std.tolist(), "q01": q01.tolist(), "q99": (q01 + np.abs(r.randn(dim)) * 3 + 0.5).tolist()}


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_preproc_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    Ref = reference_class(ref_root)
    out = {}
    for model in ("pi0", "pi05"):
        ev = Ref()
        ev.model_version = model
        ev._digitize_bins = np.linspace(-1, 1, 256 + 1)[:-1]      # test.py:40
        ev._state_q01 = ev._state_q99 = ev._actions_q01 = ev._actions_q99 = None
        if model == "pi0":
            for (h, w, seed) in FRAMES:
                frame = P.synthetic_frame(h, w, seed)
                img = ev._resize_with_pad(ev._parse_image(frame), 224, 224)
                out["resized_%dx%d_%d" % (h, w, seed)] = img
            out["normalized_crop"] = ev._normalize_image(img)[100:108, 100:116]
        ns = {"state": stats(11, 14), "actions": stats(12, 14)}
        r = np.random.RandomState(21)
        state = r.randn(14).astype(np.float32) * 2
        actions = r.randn(50, 32).astype(np.float32)
        sn = ev._normalize_state(ev._pad_to_dim(state, 14), ns, 14)
        out["state_norm_" + model] = sn
        if model == "pi05":
            out["state_digitized"] = ev._digitize_state(sn)
        out["actions_unnorm_" + model] = ev._unnormalize_actions(actions, {"actions": stats(12, 32)}, 32)
    np.savez_compressed(os.path.join(HERE, "preproc_golden.npz"), **out)
    for k, v in out.items():
        print(k, v.shape, v.dtype)


if __name__ == "__main__":
    main()
