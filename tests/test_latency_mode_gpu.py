"""Multi-view latency mode on 2 GPUs (one SigLIP tower per GPU, NCCL gather of the projected tiles) against
the fp32 oracle of the whole forward (and, for information, the single-GPU forward of the same engine).
Skipped with fewer than 2 GPUs."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "realtime-vla_b200")):
        sys.path.insert(0, p)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import synth
        import multi_gpu as M
        from pi0_infer import Pi0Inference
        nv = 2
        ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(6, 0), n_vit_layers=2, n_layers=3)
        images, state, noise = synth.make_inputs(nv, 50, 0)
        kw = dict(device=rank, n_vit_layers=2, n_layers=3, n_steps=2)
        Tower, Trunk = M.gpu_factories(ck, nv, 50, **kw)
        runner = M.MultiViewLatencyPi0(nv, Tower, Trunk)
        out = runner.forward(images.cuda(), state, noise)
        torch.cuda.synchronize()
        if rank == 0:
            from oracle import vla_oracle as O
            torch.backends.cuda.matmul.allow_tf32 = False
            d = torch.device("cuda", rank)
            w = {k: v.to(d).float() for k, v in ck.items()}
            vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
            enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
            K, V = O.prefix_encoder(w, enc, n_layers=3)
            want = O.pi0_decoder(w, K, V, state.to(d).float(), noise.to(d).float(), n_layers=3, n_steps=2)
            err = (out.float() - want).abs()
            ret["max_abs"], ret["mean_abs"] = err.max().item(), err.mean().item()
            single = Pi0Inference(ck, nv, 50, **kw)
            same = single.forward(images, state, noise).clone()
            torch.cuda.synchronize()
            ret["vs_single_gpu"] = (out.float() - same.float()).abs().max().item()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_towers_match_oracle():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, 29655, ret), nprocs=2, join=True)
    print("latency mode vs oracle: max-abs %.3e mean-abs %.3e; vs single-GPU engine: %.3e" %
          (ret["max_abs"], ret["mean_abs"], ret["vs_single_gpu"]))
    # tolerance of the path for bf16 arithmetic
    assert ret["max_abs"] <= 2e-2 and ret["mean_abs"] <= 3e-3


def _fused_worker(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "realtime-vla_b200")):
        sys.path.insert(0, p)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import synth
        import multi_gpu as M
        from pi0_infer import Pi0Inference
        nv, n_forwards = 2, 5
        ck = synth.make_checkpoint("pi0", seed=0, prompt_ids=synth.prompt_ids(6, 0), n_vit_layers=2, n_layers=3)
        kw = dict(device=rank, n_vit_layers=2, n_layers=3, n_steps=2)
        Tower, Trunk = M.gpu_factories(ck, nv, 50, **kw)
        runner = M.FusedLatencyPi0(nv, Tower, Trunk)
        inputs = [synth.make_inputs(nv, 50, 20 + i) for i in range(n_forwards)]
        outs = []
        # no synchronisation between the forwards: the tower of rank 1 runs ahead of the trunk as far as the two
        # staging slots allow, then waits in its push kernel for the trunk's acknowledgement
        for images, state, noise in inputs:
            out = runner.forward(images.cuda(), state, noise)
            if rank == 0:
                outs.append(out.clone())
        torch.cuda.synchronize()
        status = runner.tower.engine.status_word()
        if rank == 0:
            status |= runner.trunk.engine.status_word()
            from oracle import vla_oracle as O
            torch.backends.cuda.matmul.allow_tf32 = False
            d = torch.device("cuda", rank)
            single = Pi0Inference(ck, nv, 50, **kw)
            worst = 0.0
            for (images, state, noise), out in zip(inputs, outs):
                same = single.forward(images, state, noise).clone()
                torch.cuda.synchronize()
                worst = max(worst, (out.float() - same.float()).abs().max().item())
            ret["vs_single_gpu"] = worst
            images, state, noise = inputs[-1]
            w = {k: v.to(d).float() for k, v in ck.items()}
            vx = O.vision_encoder(w, images.to(d).float(), n_layers=2)
            enc = torch.cat([O.project_vision(w, vx), w["language_embeds"]], 0)
            K, V = O.prefix_encoder(w, enc, n_layers=3)
            want = O.pi0_decoder(w, K, V, state.to(d).float(), noise.to(d).float(), n_layers=3, n_steps=2)
            err = (outs[-1].float() - want).abs()
            ret["max_abs"], ret["mean_abs"] = err.max().item(), err.mean().item()
        ret["status_%d" % rank] = status
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_fused_exchange_matches_single_gpu_and_oracle():
    """The in-graph NVLink exchange (peer stores + flags, link.cuh): five forwards back to back with different inputs
    are each bit-identical to the single-GPU engine (the tiles are copied, not recomputed), the last one is within the
    path's tolerance of the oracle, and no bounded wait ran out."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_fused_worker, args=(2, 29657, ret), nprocs=2, join=True)
    print("fused latency mode vs oracle: max-abs %.3e mean-abs %.3e; vs single-GPU engine: %.3e" %
          (ret["max_abs"], ret["mean_abs"], ret["vs_single_gpu"]))
    assert ret["status_0"] == 0 and ret["status_1"] == 0
    assert ret["vs_single_gpu"] == 0.0
    assert ret["max_abs"] <= 2e-2 and ret["mean_abs"] <= 3e-3
