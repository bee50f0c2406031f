"""The steps either side of the forward in a robot loop, on the device: camera frames -> model input, robot
state -> model input, action chunk -> robot command.  The reference does them on the host in its evaluation
script (PiModelEvaluator._apply_input_transforms / infer, test.py:153-204); these wrappers keep its data
conventions (norm_stats dict with 'state' / 'actions' holding mean/std for Pi0 and q01/q99 for Pi05, three
camera views, 256-bin state tokens for Pi05) and give bit-identical numbers.

    io = RobotIO(infer, norm_stats, action_dim=7)            # infer: Pi0Inference or Pi05Inference
    actions = io.step(frames, state, noise)                   # Pi0
    actions = io.step(frames, state, noise, task_prompt="pick up the cube")   # Pi05 with a tokenizer
"""
import numpy as np
import torch


class RobotIO:
    def __init__(self, infer, norm_stats, action_dim=7):
        self.infer = infer
        self.engine = infer._engine
        self.stats = norm_stats
        self.action_dim = int(action_dim)
        self.pi05 = type(infer).__name__ == "Pi05Inference"
        self.digitize_bins = np.linspace(-1, 1, 256 + 1)[:-1]          # test.py:40

    def _pair(self, which):
        s = self.stats[which]
        return (s["q01"], s["q99"], 1) if self.pi05 else (s["mean"], s["std"], 0)

    def set_frames(self, frames):
        """frames: one uint8 (H, W, 3) RGB array or tensor per camera view (test.py:157-162)."""
        if len(frames) != self.infer.num_views:
            raise RuntimeError("expected %d camera frames, got %d" % (self.infer.num_views, len(frames)))
        for v, f in enumerate(frames):
            self.engine.preprocess_image(v, f)

    def normalize_state(self, state):
        """Pi0: fills the state input buffer and returns None.  Pi05: returns the 256-bin state tokens
        (test.py:118-137) for the prompt."""
        a, b, mode = self._pair("state")
        vals = self.engine.preprocess_state(state, a, b, mode, want_values=self.pi05)
        if self.pi05:
            return np.digitize(vals, bins=self.digitize_bins) - 1
        return None

    def step(self, frames, state, noise, task_prompt=None, token_ids=None):
        """One control step: raw frames + raw state + noise -> float64 (chunk, action_dim) robot actions."""
        state = np.asarray(state)
        self.set_frames(frames)
        tokens = self.normalize_state(state)
        images = self.infer.buffers["observation_images_normalized"]       # already filled in place
        if self.pi05:
            if token_ids is not None:
                self.infer.forward(images, noise, token_ids=token_ids)
            else:
                self.infer.forward(images, noise, task_prompt, tokens)
        else:
            self.infer.forward(images, self.infer.buffers["observation_state_normalized"], noise)
        a, b, mode = self._pair("actions")
        return self.engine.postprocess_actions(a, b, mode, state, self.action_dim)
