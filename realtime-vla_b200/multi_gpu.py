"""Multi-GPU modes of the Pi0 forward on one node, one process per GPU (torch.distributed).

Latency mode (multi-view), two variants: MultiViewLatencyPi0 gathers the tiles with NCCL between two graph launches,
FusedLatencyPi0 moves them inside the graphs with peer stores (link.cuh).  The SigLIP towers of the camera views are independent until the projected image
tokens enter the prefix (vision_encoder of the reference, pi0_infer.py:598-646, is row-wise or per view), so
rank v < num_views runs the tower + projector of view v on its own GPU and the (256, 2048) tiles are gathered
over NVLink into rows 256v.. of the prefix residual stream on rank 0, which then runs the prefix prefill and
the action expert.  The prefix and the expert stay on one GPU: they are a strict chain of 35 + 180 layers.

Throughput mode needs no code here: observations are independent, every rank runs its own Pi0Inference
(optionally batched) and there is no exchange (see bench.py --gpus N).

The engines and the gather are injected so that the rank/row bookkeeping can be tested on CPU with gloo.
"""
import torch
import torch.distributed as dist

VISION, PREFIX, EXPERT = 1, 2, 4


def view_of_rank(rank, num_views):
    """The camera view a rank's tower processes, or None for ranks beyond the number of views."""
    return rank if rank < num_views else None


def tile_rows(view):
    """Rows of the prefix residual stream that receive the projected tokens of `view`."""
    return slice(256 * view, 256 * (view + 1))


class MultiViewLatencyPi0:
    """forward(images (nv,224,224,3), state, noise) -> actions on rank 0 (None elsewhere).

    make_tower(rank) -> object with .set_image(img (224,224,3)), .run() and .tile (256,2048) fp32 tensor;
    make_trunk() (rank 0 only) -> object with .encoder_x (P,2048) fp32 tensor, .set_inputs(state, noise),
    .run() -> actions.  The default factories wrap Pi0Inference engines (see gpu_factories).
    """

    def __init__(self, num_views, make_tower, make_trunk, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world < num_views:
            raise ValueError("latency mode needs one rank per view: %d views, world size %d" % (num_views, self.world))
        self.num_views = num_views
        self.view = view_of_rank(self.rank, num_views)
        self.tower = make_tower(self.rank) if self.view is not None else None
        self.trunk = make_trunk() if self.rank == 0 else None
        like = self.tower.tile if self.tower is not None else None
        # ranks without a view still take part in the gather with a scratch tile
        self._idle_tile = None if like is not None else torch.zeros(256, 2048, dtype=torch.float32, device=self._device())

    def _device(self):
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.get_backend(self.group) == "nccl" else torch.device("cpu")

    def forward(self, images, state, noise):
        if self.tower is not None:
            self.tower.set_image(images[self.view])
            self.tower.run()
            tile = self.tower.tile
        else:
            tile = self._idle_tile
        if self.rank == 0:
            dst = [self.trunk.encoder_x[tile_rows(v)] if v < self.num_views else torch.empty_like(tile)
                   for v in range(self.world)]
            dist.gather(tile, gather_list=dst, dst=0, group=self.group)
            self.trunk.set_inputs(state, noise)
            return self.trunk.run()
        dist.gather(tile, gather_list=None, dst=0, group=self.group)
        return None


class FusedLatencyPi0:
    """Latency mode with the exchange inside the captured graphs: the last kernel of every tower's vision stage stores
    its (256, 2048) tile over NVLink into the trunk GPU and raises a flag, the first kernel of the trunk's prefix stage
    waits for the flags (link.cuh).  No collective and no host synchronisation between the stages; torch.distributed
    only carries the CUDA IPC handles of the mailboxes once, at construction.

    make_tower(rank) / make_trunk() as for MultiViewLatencyPi0, with an `.engine` attribute (the C-ABI engine)."""

    def __init__(self, num_views, make_tower, make_trunk, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world < num_views:
            raise ValueError("latency mode needs one rank per view: %d views, world size %d" % (num_views, self.world))
        self.num_views = num_views
        self.view = view_of_rank(self.rank, num_views)
        self.tower = make_tower(self.rank) if self.view is not None else None
        self.trunk = make_trunk() if self.rank == 0 else None
        # mailboxes: every rank publishes (IPC handle of its tower's mailbox, IPC handle of the trunk's mailbox)
        mine = [None, None]
        local = {}
        if self.tower is not None:
            mine[0], local["tower"] = self.tower.engine.link_create(0)
        if self.trunk is not None:
            mine[1], local["trunk"] = self.trunk.engine.link_create(num_views)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        trunk_handle = everyone[0][1]
        if self.tower is not None:
            # a process cannot open its own IPC handle: rank 0's tower takes the trunk's pointer directly
            box = local["trunk"] if self.rank == 0 else self.tower.engine.link_open(trunk_handle)
            self.tower.engine.link_tower_connect(box, self.view, num_views)
        if self.trunk is not None:
            for v in range(num_views):
                box = local["tower"] if v == 0 else self.trunk.engine.link_open(everyone[v][0])
                self.trunk.engine.link_trunk_connect(v, box)
        dist.barrier(group=group)   # every mailbox is connected before the first forward

    def forward(self, images, state, noise):
        if self.tower is not None:
            self.tower.set_image(images[self.view])
            self.tower.run()
        if self.trunk is not None:
            self.trunk.set_inputs(state, noise)
            return self.trunk.run()
        return None


def gpu_factories(checkpoint, num_views, chunk_size, **kw):
    """Tower / trunk factories over Pi0Inference engines: the tower is a 1-view engine running only the vision
    stage; the trunk is the full engine running the prefix and expert stages."""
    from pi0_infer import Pi0Inference

    class Tower:
        def __init__(self, rank):
            vision = {k: v for k, v in checkpoint.items() if k.startswith("vision_") or k.startswith("encoder_multi_modal")}
            vision["language_embeds"] = checkpoint["language_embeds"][:0]
            self.infer = Pi0Inference(vision, 1, chunk_size, **kw)
            self.engine = self.infer._engine
            self.tile = self.infer._engine.buffer("encoder_x", (256, 2048), torch.float32)

        def set_image(self, img):
            self.infer.buffers["observation_images_normalized"].copy_(img.reshape(1, 224, 224, 3))

        def run(self):
            self.infer._engine.forward_stages(VISION)

    class Trunk:
        def __init__(self):
            self.infer = Pi0Inference(checkpoint, num_views, chunk_size, **kw)
            self.engine = self.infer._engine
            P = num_views * 256 + len(checkpoint["language_embeds"])
            self.encoder_x = self.infer._engine.buffer("encoder_x", (P, 2048), torch.float32)

        def set_inputs(self, state, noise):
            self.infer.buffers["observation_state_normalized"].copy_(state)
            self.infer.buffers["diffusion_noise"].copy_(noise)

        def run(self):
            self.infer._engine.forward_stages(PREFIX | EXPERT)
            return self.infer.buffers["diffusion_noise"]

    return Tower, Trunk
