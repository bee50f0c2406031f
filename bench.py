"""Benchmark of the Pi0 single-observation forward (the reference's headline: median forward latency,
benchmark.py:17-33 of the reference; plus observations/s for the data-parallel scaling run).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|cfg2|cfg3]

One "step" = one forward of one observation.  The default workload is Pi0, 3 views, 20 prompt tokens, chunk 50,
10 Euler steps, full depth, seeded random bf16 weights and inputs (no checkpoint or camera data exists offline).
N > 1 runs one independent replica per GPU (the path has no cross-observation exchange: weak scaling, no collective
on the data path).

Prints one JSON line.  `value` is observations/s over all ranks, timed on the device over exactly K graph
replays with the inputs resident in HBM; the weights streamed by every forward (5.2 GB) exceed L2 by 40x,
so no L2 flush is needed between iterations.  `e2e` is the same through the host-memory entry point of the
C ABI (pinned host buffers in, actions out, copies and synchronisation inside the timed region).
`roofline` describes the stage that owns most of the forward, the action expert (one persistent kernel launch per
forward, HBM-bound weight streaming); `roofline_prefix` the largest tensor-bound kernel (prefix GeGLU GEMM).
`reference_triton` is the reference's own Triton forward, timed on the same GPU by its own benchmark script from an
unmodified copy under baseline/_ref (in a subprocess, before the timed region); `throughput_cfg5` is the throughput
configuration (32 observations per forward and GPU) measured in the same run.
`--impl reference` times the fp32 CPU oracle (the reference has no CPU path of its own) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "realtime-vla_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

WORKLOADS = {
    "cfg1": dict(model="pi0", num_views=1, prompt_len=0, chunk=50, seed=0),
    "cfg2": dict(model="pi0", num_views=3, prompt_len=20, chunk=50, seed=0),
    "cfg3": dict(model="pi05", num_views=2, prompt_len=52, chunk=50, seed=1),
    # Pi05 at the shape the reference's benchmark.py was timed on this GPU type (3 views, 20 prompt tokens)
    "pi05_3v": dict(model="pi05", num_views=3, prompt_len=20, chunk=50, seed=1),
    # action expert alone over a prefilled K/V cache (the weight-streaming stage): stage mask 4 of the forward
    "cfg4": dict(model="pi0", num_views=3, prompt_len=20, chunk=50, seed=0, stages=4),
    # throughput mode for Pi05: 32 observations per forward sharing one prompt
    "pi05_b32": dict(model="pi05", num_views=2, prompt_len=52, chunk=50, seed=1, batch=32),
    # throughput mode: 32 independent observations per forward on each GPU
    "cfg5": dict(model="pi0", num_views=2, prompt_len=20, chunk=50, seed=0, batch=32),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture): the prefix GeGLU GEMM at
# 788 tokens, and the persistent action-expert kernel (captured at reduced depth, scaled to 18 layers x 10 steps by
# the layer-steps processed: its traffic is the weight stream, which grows in proportion).
NCU_TRAFFIC_GEGLU = {"cfg2": 144519168}
NCU_TRAFFIC_EXPERT = {"any": int(354.1e6 * 18)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


DEPTH = {"vit": 27, "layers": 18, "steps": 10}      # reduced only by the profiling options --vit-layers / --layers / --euler-steps


def depth_kw():
    """Keyword arguments of the inference classes for a reduced depth (nothing when the depth is the model's)."""
    kw = {}
    if DEPTH["vit"] != 27:
        kw["n_vit_layers"] = DEPTH["vit"]
    if DEPTH["layers"] != 18:
        kw["n_layers"] = DEPTH["layers"]
    if DEPTH["steps"] != 10:
        kw["n_steps"] = DEPTH["steps"]
    return kw


def fast_checkpoint(model, prompt_len, seed, device):
    """Random bf16 checkpoint of the full-depth shapes, drawn on `device` (timing only: values follow the
    same N(0, 0.02) / unit-LayerNorm recipe as the parity tests but from the device generator)."""
    from oracle import synth
    shapes = {}
    shapes.update(synth.vision_shapes(DEPTH["vit"]))
    shapes.update(synth.encoder_shapes(DEPTH["layers"]))
    shapes.update(synth.pi0_decoder_shapes(DEPTH["layers"]) if model == "pi0" else synth.pi05_decoder_shapes(DEPTH["layers"]))
    g = torch.Generator(device=device).manual_seed(seed)
    ck = {}
    for k, shp in shapes.items():
        if k.endswith("_norm_w"):
            ck[k] = torch.ones(shp, dtype=torch.bfloat16, device=device)
        elif k.endswith("_norm_b"):
            ck[k] = torch.zeros(shp, dtype=torch.bfloat16, device=device)
        elif k == "decoder_time_embeds":
            from oracle.vla_oracle import sincos_time_table
            ck[k] = sincos_time_table(10).to(device)
        else:
            std = 0.002 if k.startswith("decoder_action_fused_out_proj") else 0.02
            ck[k] = (torch.randn(shp, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)
    ck["language_embeds"] = (torch.randn(prompt_len, 2048, generator=g, device=device) * 0.02 * 2048 ** 0.5).to(torch.bfloat16)
    return ck


def inputs(wl, device):
    g = torch.Generator(device=device).manual_seed(1234)
    lead = (wl["batch"],) if wl.get("batch", 1) > 1 else ()
    images = (torch.rand(*lead, wl["num_views"], 224, 224, 3, generator=g, device=device) * 2 - 1).to(torch.bfloat16)
    state = torch.randn(*lead, 32, generator=g, device=device).to(torch.bfloat16)
    noise = torch.randn(*lead, wl["chunk"], 32, generator=g, device=device).to(torch.bfloat16)
    return images, state, noise


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                mx = float(f[2])
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}
        return out


def max_over_ranks(dist, device, values):
    """Element-wise maximum of per-rank timings over all ranks (the step time of a multi-GPU job is set by
    its slowest rank); works with NCCL on GPU and gloo on CPU."""
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def percentile(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


def dominant_kernel_roofline(wl, device):
    """Times the dominant kernel of the workload alone (CUDA events around back-to-back launches on one stream)
    and returns the roofline object.  For every Pi0/Pi05 configuration that kernel is the prefix GeGLU GEMM:
    hidden[P,16384] = gelu(x Wg) * (x Wu), 4*P*2048*16384 FLOPs per launch (two P x 2048 x 16384 products), tensor-bound when P >= 512 and
    co-limited by the 134 MB weight stream at P = 256."""
    import vla_ops as gpu_ops
    P = (wl["num_views"] * 256 + wl["prompt_len"]) * wl.get("batch", 1)      # prefix tokens per forward
    g = torch.Generator(device=device).manual_seed(7)
    x = torch.randn(P, 2048, generator=g, device=device).to(torch.bfloat16)
    wg = (torch.randn(2048, 16384, generator=g, device=device) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(2048, 16384, generator=g, device=device) * 0.02).to(torch.bfloat16)
    _, ms = gpu_ops.gemm(x, wg, w2=wu, act=3, iters=20)
    flops = 4.0 * P * 2048 * 16384
    pk, which = peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    return {"kernel": "gemm_sm100_kernel<256,dual> prefix GeGLU P=%d" % P, "bound": "tensor", "achieved": round(achieved, 1),
            "peak": pk["bf16_tflops"], "peak_source": which + " burst", "unit": "TFLOP/s",
            "frac": round(achieved / pk["bf16_tflops"], 4), "ms_per_launch": round(ms, 4),
            "traffic": None}


def expert_down_roofline(wl, device):
    """Action-expert down projection x[S,1024] += hidden[S,4096] @ Wd: 8.4 MB of weights per launch, split over a
    cluster of 8 along K; HBM-bound (the weights are read exactly once per launch)."""
    import vla_ops
    S = wl["chunk"] + (1 if wl["model"] == "pi0" else 0)
    g = torch.Generator(device=device).manual_seed(7)
    x = torch.randn(S, 4096, generator=g, device=device).to(torch.bfloat16)
    w = (torch.randn(4096, 1024, generator=g, device=device) * 0.02).to(torch.bfloat16)
    res = torch.randn(S, 1024, generator=g, device=device)
    _, ms = vla_ops.gemm(x, w, epi=1, res=res, iters=50)
    nbytes = 4096 * 1024 * 2 + S * 4096 * 2 + 2 * S * 1024 * 4
    pk, which = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"kernel": "gemm_sm100_kernel<64,single,split 8> expert down projection S=%d" % S, "bound": "hbm", "achieved": round(gbs, 1),
            "peak": pk["hbm_gbs"], "peak_source": which, "unit": "GB/s", "frac": round(gbs / pk["hbm_gbs"], 4),
            "ms_per_launch": round(ms, 5), "bytes_per_launch": nbytes,
            "note": "back-to-back launches of one shape: the 8.4 MB of weights stay in L2, so this is the launch-latency floor, not a DRAM figure"}


def expert_attention_timing(wl, device):
    """Suffix attention of one action-expert layer: 8 S query rows over P + S keys, head dim 256, Pi0 mask."""
    import vla_ops
    P = wl["num_views"] * 256 + wl["prompt_len"]
    S = wl["chunk"] + (1 if wl["model"] == "pi0" else 0)
    g = torch.Generator(device=device).manual_seed(7)
    q = torch.randn(S * 8, 256, generator=g, device=device).to(torch.bfloat16)
    k = torch.randn(P + S, 256, generator=g, device=device).to(torch.bfloat16)
    v = torch.randn(P + S, 256, generator=g, device=device).to(torch.bfloat16)
    _, ms = vla_ops.attention_tc(q, k, v, prefix_alloc=P, valid_prefix=P, restrict_rows=8, scale=1 / 16, iters=50)
    flops = 4.0 * S * 8 * (P + S) * 256
    return {"kernel": "attention_tc_kernel suffix attention rows=%d keys=%d" % (S * 8, P + S), "bound": "latency",
            "achieved": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_launch": round(ms, 5)}


def siglip_attention_timing(wl, device):
    """SigLIP attention of one ViT layer: num_views x 16 heads x (256 x 256) at head dim 72 on the tcgen05 kernel."""
    import vla_ops
    nv = wl["num_views"]
    g = torch.Generator(device=device).manual_seed(9)
    qkv = torch.randn(nv * 256, 3456, generator=g, device=device).to(torch.bfloat16)
    _, ms = vla_ops.vit_attention_tc(qkv, scale=72 ** -0.5, iters=50)
    flops = 4.0 * nv * 16 * 256 * 256 * 72
    return {"kernel": "vit_attention_tc_kernel views=%d heads=16 tokens=256 head_dim=72" % nv, "bound": "latency",
            "achieved": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_launch": round(ms, 5)}


def preprocess_timing(wl, device):
    """Camera frames -> model input on the device (vla_preprocess_image: Pillow-exact bilinear resize, pad,
    normalise, bf16) for 640 x 480 frames, one per view: device time with the frames resident, end-to-end time from
    pinned host frames, and the same work on the host cores (the oracle's numpy restatement, and Pillow itself,
    which is what the reference's evaluation script calls)."""
    from pi0_infer import Pi0Inference
    from oracle import preproc_oracle as P
    import numpy as np
    nv = wl["num_views"]
    infer = Pi0Inference({"language_embeds": torch.zeros(0, 2048)}, nv, wl["chunk"], n_vit_layers=1, n_layers=1, n_steps=1)
    frames = [P.synthetic_frame(480, 640, 10 + v) for v in range(nv)]
    dev_frames = [torch.from_numpy(f).to(device) for f in frames]
    pin_frames = [torch.from_numpy(f).pin_memory() for f in frames]
    eng = infer._engine

    def run(fs):
        for v, f in enumerate(fs):
            eng.preprocess_image(v, f)
    for _ in range(5):
        run(dev_frames)
    torch.cuda.synchronize()
    iters = 200
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run(dev_frames)
    e1.record()
    torch.cuda.synchronize()
    dev_ms = e0.elapsed_time(e1) / iters
    t0 = time.perf_counter()
    for _ in range(iters):
        run(pin_frames)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / iters
    t0 = time.perf_counter()
    for f in frames:
        P.normalize_image(P.resize_with_pad(f))
    port_ms = (time.perf_counter() - t0) * 1e3
    pil_ms = None
    try:
        from PIL import Image
        t0 = time.perf_counter()
        for _ in range(20):
            for f in frames:
                small = Image.fromarray(f).resize((224, 168), resample=Image.BILINEAR)
                canvas = Image.new(small.mode, (224, 224), 0)
                canvas.paste(small, (0, 28))
                (np.array(canvas).astype(np.float32) / 255.0 * 2.0 - 1.0)
        pil_ms = (time.perf_counter() - t0) * 1e3 / 20
    except ImportError:
        pass
    # algorithmic bytes per frame: read the frame, write + read the horizontally resampled picture, write the bf16 view
    per_frame = 480 * 640 * 3 + 2 * 480 * 224 * 3 + 224 * 224 * 3 * 2
    pk, which = peaks()
    gbs = nv * per_frame / (dev_ms * 1e-3) / 1e9
    return {"kernel": "pp_resize_h_kernel + pp_resize_v_pad_norm_kernel, %d frames of 480x640" % nv, "bound": "hbm",
            "achieved": round(gbs, 2), "peak": pk["hbm_gbs"], "peak_source": which, "unit": "GB/s", "frac": round(gbs / pk["hbm_gbs"], 5),
            "ms_per_step": round(dev_ms, 5), "e2e_ms_per_step": round(e2e_ms, 5), "h2d_bytes_per_step": nv * 480 * 640 * 3,
            "cpu_baseline": {"port_ms_per_step": round(port_ms, 3), "pillow_ms_per_step": None if pil_ms is None else round(pil_ms, 3),
                             "cores": 1, "sample": "the same %d frames once (numpy restatement) / 20 times (Pillow)" % nv},
            "note": "%d launches of ~1 MB each: bound by launch and memory latency, not by bandwidth" % (2 * nv)}


def decoder_stream(wl, decoder_ms):
    """Action-expert weight streaming: algorithmic bytes of the 10 Euler steps (18 layers x 34.603 MB of weights
    + 2.23 MB of in/out projections + the K/V cache rows read by the suffix attention, per step) over the
    measured decoder stage time, against the HBM copy peak."""
    P = wl["num_views"] * 256 + wl["prompt_len"]
    S = wl["chunk"] + (1 if wl["model"] == "pi0" else 0)
    per_step = 18 * (34.603e6 + 1024.0 * (P + S)) + 2.23e6
    gbs = 10 * per_step / (decoder_ms * 1e-3) / 1e9
    pk, which = peaks()
    return {"bytes_per_forward": int(10 * per_step), "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "peak_source": which,
            "unit": "GB/s", "frac": round(gbs / pk["hbm_gbs"], 4), "bound": "hbm"}


def expert_stage_roofline(wl, infer, noise, reps=20):
    """The action-expert stage (one persistent kernel launch per forward; per-operator launches for batched handles):
    average duration over `reps` launches, CUDA events on the launching stream, K/V cache filled by a full forward
    before; algorithmic bytes = weights + K/V rows streamed by the 10 Euler steps, against the measured HBM copy peak."""
    noise_buf = infer.buffers["diffusion_noise"]
    torch.cuda.synchronize()
    for _ in range(3):
        noise_buf.copy_(noise)
        infer._engine.forward_stages(4)
    total = 0.0
    for _ in range(reps):
        noise_buf.copy_(noise)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        infer._engine.forward_stages(4)
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    ms = total / reps
    r = decoder_stream(wl, ms)
    n_launch = infer._engine.stage_kernels()[2]
    r.update(kernel="expert_persistent_kernel: action-expert stage, 10 Euler steps, %d launch%s per forward" % (n_launch, "" if n_launch == 1 else "es"),
             ms_per_launch=round(ms, 4), bytes_per_launch=r.pop("bytes_per_forward"), traffic=NCU_TRAFFIC_EXPERT.get("any"),
             peak_source=r["peak_source"] + " copy bandwidth (kernel timed inside a long step)")
    return r


def reference_triton(wl, gpu_index, timeout_s=900):
    """The reference's own Triton forward on this GPU: its unmodified benchmark script (median of 100 wall-clock
    forward + synchronize after 3 warm-ups) from the copy under baseline/_ref, in a subprocess, same model / views /
    prompt length / chunk.  Returns {"p50_ms", "runs", "clocks"} or {"unavailable": why}."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "benchmark.py")):
        return {"unavailable": "no copy of the reference under baseline/_ref on this machine"}
    if wl.get("batch", 1) > 1 or wl.get("stages"):
        return {"unavailable": "the reference has no batch dimension and no stage subset"}
    cmd = [sys.executable, "benchmark.py", "--model_version", wl["model"], "--num_views", str(wl["num_views"]),
           "--chunk_size", str(wl["chunk"]), "--prompt_len", str(wl["prompt_len"])]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", str(gpu_index)))
    sampler = ClockSampler(gpu_index)
    sampler.start()
    t0 = time.time()
    try:
        res = subprocess.run(cmd, cwd=ref_dir, env=env, capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        sampler.stop()
        return {"unavailable": "the reference's benchmark script did not finish within %d s" % timeout_s}
    clocks = sampler.stop()
    import re
    m = re.search(r"runs (\d+) median time per inference: ([0-9.]+) ms", res.stdout)
    if res.returncode != 0 or not m:
        tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or [""]
        return {"unavailable": "the reference's benchmark script failed (did not compile or run): %s" % tail[0][:200]}
    return {"p50_ms": float(m.group(2)), "runs": int(m.group(1)), "clocks": clocks, "wall_s": round(time.time() - t0, 1),
            "method": "reference benchmark.py: median of wall-clock forward + synchronize, 3 warm-ups, CUDA-graph replay"}


def throughput_cfg5(device, local, flags, dist, world, steps=8):
    """Throughput configuration in the same run: Pi0, 2 views, 20 prompt tokens, 32 observations per forward on each
    GPU (device-resident inputs, CUDA events, max over ranks)."""
    from pi0_infer import Pi0Inference
    wl = dict(WORKLOADS["cfg5"])
    ck = fast_checkpoint("pi0", wl["prompt_len"], wl["seed"], device)
    infer = Pi0Inference(ck, wl["num_views"], wl["chunk"], device=local, flags=flags, batch=wl["batch"])
    del ck
    images, state, noise = inputs(wl, device)
    for _ in range(3):
        infer.forward(images, state, noise)
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        infer.forward(images, state, noise)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = max_over_ranks(dist, device, [e0.elapsed_time(e1)])[0]
    ok = infer._engine.status_word() == 0
    del infer
    torch.cuda.empty_cache()
    return {"value": round(wl["batch"] * world * steps / (ms * 1e-3), 2), "unit": "obs/s", "n_gpus": world, "batch_per_gpu": wl["batch"],
            "steps": steps, "ms_per_step": round(ms / steps, 3), "status_clean": ok,
            "config": {k: wl[k] for k in ("model", "num_views", "prompt_len", "chunk")}, "clocks": clocks}


def use_all_host_threads():
    """The CPU legs use every core this process may run on: torchrun exports OMP_NUM_THREADS=1 to its workers,
    which would otherwise leave the oracle on one thread."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def oracle_forward_fn(wl, ck):
    from oracle import vla_oracle as O
    use_all_host_threads()
    w = {k: v.cpu() for k, v in ck.items()}
    images, state, noise = [t.cpu() for t in inputs(wl, "cpu")]
    if wl.get("batch", 1) > 1:      # the oracle has no batch dimension: one observation of the batch per step
        images, state, noise = images[0], state[0], noise[0]
    if wl.get("stages") == 4:       # expert alone: the prefix K/V cache is computed once, outside the timed calls
        wf = O._weights_f32(w, "cpu")
        vx = O.vision_encoder(wf, images.float())
        enc = torch.cat([O.project_vision(wf, vx), wf["language_embeds"].reshape(-1, 2048)], 0)
        K, V = O.prefix_encoder(wf, enc)
        return lambda: O.pi0_decoder(wf, K, V, state.float(), noise.float())
    if wl["model"] == "pi0":
        return lambda: O.pi0_forward(w, images, state, noise)
    return lambda: O.pi05_forward(w, images, noise)


def cpu_baseline(wl, ck, budget_s=25.0):
    """The fp32 oracle on the host cores: one full forward of the same workload (a bounded sample of 1 step)."""
    fn = oracle_forward_fn(wl, ck)
    fn()                                   # warm-up: thread pool, allocator, page faults of the fp32 weight copies
    t0 = time.time()
    fn()
    dt = time.time() - t0
    return {"value": round(1.0 / dt, 5), "unit": "obs/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "1 full forward of the workload after 1 warm-up forward, %.1f s" % dt}


def run_reference(args, wl, rank, world):
    if rank != 0:
        return
    device = "cuda" if torch.cuda.is_available() else "cpu"
    ck = fast_checkpoint(wl["model"], wl["prompt_len"], wl["seed"], device)
    fn = oracle_forward_fn(wl, ck)
    del ck
    warm = args.warmup
    for _ in range(warm):
        fn()
    times, t_start = [], time.time()
    for _ in range(args.steps):
        t0 = time.time()
        fn()
        times.append(time.time() - t0)
        if time.time() - t_start > 150:      # keep the whole run within a few minutes
            break
    total = sum(times)
    val = len(times) / total
    line = {"impl": "reference", "metric": "observations_per_s", "value": round(val, 5), "unit": "obs/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": warm, "ms_per_step": round(1e3 * total / len(times), 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, **{k: wl[k] for k in ("model", "num_views", "prompt_len", "chunk")},
                       "euler_steps": 10, "note": "fp32 eager PyTorch oracle on host cores; the reference has no CPU path"},
            "latency_ms": {"p50": round(1e3 * percentile(times, 0.5), 2), "p99": round(1e3 * percentile(times, 0.99), 2)},
            "cpu_baseline": {"value": round(val, 5), "unit": "obs/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": "%d full forwards" % len(times)},
            "e2e": {"value": round(val, 5), "unit": "obs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_latency_mode(args, wl, rank, world, local, device, dist):
    """Multi-view latency mode: rank v < num_views runs the SigLIP tower of view v, the projected tiles reach rank 0
    either inside the captured graphs (peer stores over NVLink, --exchange fused) or through an NCCL gather between
    two graph launches (--exchange nccl); rank 0 runs the prefix prefill and the action expert."""
    import multi_gpu as M
    nv = wl["num_views"]
    if world < nv or wl["model"] != "pi0":
        raise SystemExit("--mode latency needs a Pi0 workload and one rank per view (%d views, %d ranks)" % (nv, world))
    ck = fast_checkpoint("pi0", wl["prompt_len"], wl["seed"], device)
    Tower, Trunk = M.gpu_factories(ck, nv, wl["chunk"], device=local, flags=args.flags)
    runner = (M.FusedLatencyPi0 if args.exchange == "fused" else M.MultiViewLatencyPi0)(nv, Tower, Trunk)
    images, state, noise = inputs(wl, device)
    host_args = [t.cpu().pin_memory() for t in (images, state, noise)]
    step = lambda: runner.forward(images, state, noise)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    lat = []
    for _ in range(args.steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        lat.append(a.elapsed_time(b))
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = runner.forward(*host_args)
        if out is not None:
            out.cpu()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    total_ms, e2e_ms = max_over_ranks(dist, device, [total_ms, e2e_s * 1e3])
    if rank == 0:
        # rank 0 launches its own tower (vision stage of a 1-view engine) and the trunk's prefix + expert stages
        n_trunk = runner.tower.infer._engine.stage_kernels()[0] + sum(runner.trunk.infer._engine.stage_kernels()[1:])
        line = {"metric": "observations_per_s", "value": round(args.steps / (total_ms * 1e-3), 3), "unit": "obs/s",
                "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(total_ms / args.steps, 4),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, **{k: wl[k] for k in ("model", "num_views", "prompt_len", "chunk")},
                           "euler_steps": 10, "batch_per_gpu": 1,
                           "parallelism": "latency mode: %d SigLIP towers on %d GPUs, %s, prefix + expert on rank 0" %
                                          (nv, nv, "tiles pushed over NVLink inside the graphs" if args.exchange == "fused" else "NCCL gather of the projected tiles")},
                "latency_ms": {"p50": round(percentile(lat, 0.5), 4), "p99": round(percentile(lat, 0.99), 4),
                               "note": "rank 0, device events around tower + exchange + prefix + expert"},
                "e2e": {"value": round(args.steps / (e2e_ms * 1e-3), 3), "unit": "obs/s",
                        "h2d_bytes_per_step": sum(x.numel() * 2 for x in host_args), "d2h_bytes_per_step": wl["chunk"] * 32 * 2,
                        "ms_per_step": round(e2e_ms / args.steps, 4)},
                "gpu_launches": n_trunk * args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-triton", action="store_true", help="skip timing the reference's Triton forward (1-GPU runs only)")
    ap.add_argument("--no-cfg5", action="store_true", help="skip the throughput configuration (32 observations per forward and GPU)")
    ap.add_argument("--batch", type=int, default=0, help="override the observations per forward of a workload (throughput mode)")
    ap.add_argument("--mode", default="replicas", choices=["replicas", "latency"],
                    help="replicas: every rank runs whole forwards (default); latency: one observation, one SigLIP tower "
                         "per rank + gather (needs at least num_views ranks)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="latency mode: image tokens pushed over NVLink inside the graphs, or an NCCL gather between two graph launches")
    ap.add_argument("--flags", type=int, default=0, help="vla_config.flags: 1 = no programmatic dependent launch, 2 = no CUDA graph")
    ap.add_argument("--microbench", nargs="?", const="geglu", default=None, choices=["geglu", "expert_down", "expert_attention", "siglip_attention", "preprocess"],
                    help="time one kernel alone and print its roofline object: geglu = the dominant kernel of the workload "
                         "(prefix GeGLU GEMM); expert_down = action-expert down projection (51 x 4096 -> 1024, HBM-bound weight "
                         "stream); expert_attention = suffix attention of the action expert on the tcgen05 kernel; siglip_attention = "
                         "attention of one SigLIP layer on the tcgen05 kernel; preprocess = camera "
                         "frames -> model input (resize, pad, normalise) on the device against the host code")
    ap.add_argument("--vit-layers", type=int, default=27, help="profiling only: SigLIP layers (a reduced-depth model keeps an ncu capture small)")
    ap.add_argument("--layers", type=int, default=18, help="profiling only: prefix / expert layers")
    ap.add_argument("--euler-steps", type=int, default=10, help="profiling only: Euler steps")
    ap.add_argument("--profile-forward", action="store_true",
                    help="run two forwards and bracket the second with cudaProfilerStart/Stop (for ncu "
                         "--profile-from-start off); prints no benchmark line")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        wl["batch"] = args.batch
    DEPTH.update(vit=args.vit_layers, layers=args.layers, steps=args.euler_steps)
    if depth_kw() and not args.profile_forward:
        raise SystemExit("a reduced depth is for --profile-forward only: a benchmark line is always the full model")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, wl, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if args.microbench:
        fn = {"geglu": dominant_kernel_roofline, "expert_down": expert_down_roofline, "expert_attention": expert_attention_timing,
              "siglip_attention": siglip_attention_timing, "preprocess": preprocess_timing}
        print(json.dumps(fn[args.microbench](wl, device)), flush=True)
        return
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    if args.mode == "latency":
        if dist is None:
            raise SystemExit("--mode latency needs torchrun with at least num_views ranks")
        run_latency_mode(args, wl, rank, world, local, device, dist)
        return

    ref_triton = None
    if world == 1 and not args.no_reference_triton and not args.profile_forward:
        ref_triton = reference_triton(wl, local)       # before this process holds GPU memory, outside every timed region

    if wl["model"] == "pi0":
        from pi0_infer import Pi0Inference
        ck = fast_checkpoint("pi0", wl["prompt_len"], wl["seed"], device)
        infer = Pi0Inference(ck, wl["num_views"], wl["chunk"], device=local, flags=args.flags, batch=wl.get("batch", 1), **depth_kw())
        images, state, noise = inputs(wl, device)
        step = lambda: infer.forward(images, state, noise)
        host_args = [t.cpu().pin_memory() for t in (images, state, noise)]
        host_step = lambda: infer.forward_host(*host_args)
        if wl.get("stages"):
            # stage subset (the expert alone): one full forward fills the K/V cache, then every step copies the
            # noise in and replays only that stage; the host-memory figure keeps the same subset
            step()
            noise_buf, mask, host_noise = infer.buffers["diffusion_noise"], wl["stages"], host_args[2]

            def step():
                noise_buf.copy_(noise)
                infer._engine.forward_stages(mask)

            def host_step():
                noise_buf.copy_(host_noise, non_blocking=True)
                infer._engine.forward_stages(mask)
                return noise_buf.cpu()
            host_args = [host_noise]
    else:
        from pi05_infer import Pi05Inference
        ck = fast_checkpoint("pi05", wl["prompt_len"], wl["seed"], device)
        infer = Pi05Inference(ck, wl["num_views"], wl["chunk"], discrete_state_input=False, device=local, flags=args.flags,
                              batch=wl.get("batch", 1), **depth_kw())
        images, state, noise = inputs(wl, device)
        step = lambda: infer.forward(images, noise)
        host_args = [t.cpu().pin_memory() for t in (images, noise)]
        host_step = lambda: infer.forward_host(*host_args)
    n_kernels, dev_bytes = infer._engine.stats()
    if wl.get("stages"):
        n_kernels = sum(n for i, n in enumerate(infer._engine.stage_kernels()) if wl["stages"] >> i & 1)
    if args.profile_forward:
        step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print("profiled one forward of %s: %d kernel launches" % (args.workload, n_kernels))
        return

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- timed region: exactly K steps, device time -------------------------------------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    # ---- per-step latency (device events around each forward, host sync between) -----------------------
    lat = []
    for _ in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        lat.append(a.elapsed_time(b))
    # ---- end to end through the host-memory entry point ---------------------------------------------------
    for _ in range(3):
        host_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        host_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    assert infer._engine.status_word() == 0, "device status word raised"

    total_ms, e2e_ms = max_over_ranks(dist, device, [total_ms, e2e_s * 1e3])
    stage_ms = infer._engine.time_stages()
    obs = wl.get("batch", 1)          # observations per step and GPU
    expert_roof = expert_stage_roofline(wl, infer, noise) if obs == 1 else None
    single = obs == 1 and not wl.get("stages")
    if not single or args.no_cfg5:
        cfg5 = None
    else:
        if rank != 0:
            del infer
            torch.cuda.empty_cache()
        cfg5 = throughput_cfg5(device, local, args.flags, dist, world)

    if rank == 0:
        h2d = sum(x.numel() * 2 for x in host_args)
        d2h = obs * wl["chunk"] * 32 * 2
        line = {"metric": "observations_per_s", "value": round(obs * world * args.steps / (total_ms * 1e-3), 3), "unit": "obs/s",
                "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(total_ms / args.steps, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, **{k: wl[k] for k in ("model", "num_views", "prompt_len", "chunk")},
                           "euler_steps": 10, "batch_per_gpu": obs, "parallelism": "replicas x%d" % world,
                           "l2": "5.2 GB of weights streamed per step, 40x the 126 MB L2; no flush needed"},
                "latency_ms": {"p50": round(percentile(lat, 0.5), 4), "p99": round(percentile(lat, 0.99), 4)},
                "stage_ms": {"vision": round(stage_ms[0], 4), "prefix": round(stage_ms[1], 4), "decoder": round(stage_ms[2], 4),
                             "note": "eager launches with events between stages, outside the graph"},
                "e2e": {"value": round(obs * world * args.steps / (e2e_ms * 1e-3), 3), "unit": "obs/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms / args.steps, 4)},
                "decoder_stream": decoder_stream(wl, stage_ms[2]) if obs == 1 else None,
                "gpu_launches": n_kernels * args.steps, "kernels_per_step": n_kernels, "device_bytes": dev_bytes,
                "clocks": clocks}
        del infer
        torch.cuda.empty_cache()
        if wl.get("stages") == 4:
            line["config"]["stages"] = "action expert only (stage mask 4), K/V cache prefilled by one forward"
        if expert_roof is not None:
            # the expert stage owns most of a single-observation forward: it is the dominant "kernel" of the workload
            line["roofline"] = expert_roof
            line["roofline"]["share_of_forward"] = round(stage_ms[2] / max(sum(stage_ms), 1e-9), 3)
            line["decoder_stream"] = None
            if not wl.get("stages"):
                line["roofline_prefix"] = dominant_kernel_roofline(wl, device)
                line["roofline_prefix"]["traffic"] = NCU_TRAFFIC_GEGLU.get(args.workload)
        else:
            line["roofline"] = dominant_kernel_roofline(wl, device)
            line["roofline"]["traffic"] = NCU_TRAFFIC_GEGLU.get(args.workload)
        if ref_triton is not None:
            line["reference_triton"] = ref_triton
            if "p50_ms" in ref_triton:
                line["speedup_vs_triton"] = round(ref_triton["p50_ms"] / percentile(lat, 0.5), 3)
        if cfg5 is not None:
            line["throughput_cfg5"] = cfg5
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl, ck)
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
