"""World-size-2 and -3 gloo runs (CPU) of the multi-GPU host logic: which rank owns which view, where the
gathered tiles land, and the max-over-ranks timing reduction of the benchmark."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, num_views, ret):
    sys.path.insert(0, os.path.join(ROOT, "realtime-vla_b200"))
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import multi_gpu as M

        class FakeTower:
            def __init__(self, r):
                self.tile = torch.zeros(256, 2048)

            def set_image(self, img):
                self.img = img

            def run(self):   # "projection": every token = mean of the view's image, plus the view id
                self.tile.fill_(float(self.img.float().mean()))

        class FakeTrunk:
            def __init__(self):
                self.encoder_x = torch.full((num_views * 256 + 5, 2048), -1.0)

            def set_inputs(self, state, noise):
                self.noise = noise

            def run(self):
                return self.encoder_x[:, 0].clone()

        runner = M.MultiViewLatencyPi0(num_views, FakeTower, FakeTrunk)
        images = torch.stack([torch.full((224, 224, 3), float(10 + v)) for v in range(num_views)])
        out = runner.forward(images, torch.zeros(32), torch.zeros(50, 32))
        if rank == 0:
            want = torch.cat([torch.full((256,), float(10 + v)) for v in range(num_views)] + [torch.full((5,), -1.0)])
            ret["ok"] = bool(torch.equal(out, want))
        else:
            assert out is None
        # benchmark reduction: max over ranks of the per-rank timings
        import bench
        t = bench.max_over_ranks(dist, torch.device("cpu"), [10.0 + rank, 5.0 - rank])
        if rank == 0:
            ret["max"] = t
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,num_views", [(2, 2), (3, 2), (3, 3)])
def test_latency_mode_gather_layout(world, num_views):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29600 + world * 10 + num_views
    mp.spawn(_worker, args=(world, port, num_views, ret), nprocs=world, join=True)
    assert ret["ok"]
    assert ret["max"] == [10.0 + world - 1, 5.0]


def test_view_assignment():
    sys.path.insert(0, os.path.join(ROOT, "realtime-vla_b200"))
    import multi_gpu as M
    assert [M.view_of_rank(r, 3) for r in range(4)] == [0, 1, 2, None]
    assert M.tile_rows(2) == slice(512, 768)
