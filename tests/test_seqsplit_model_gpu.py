"""Whole-model sequence parallelism on real GPUs (needs at least two; skipped otherwise): the logits of the
row-split forward over NCCL equal the single-GPU forward."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, size, ret):
    import vig_b200
    from vig_b200 import seqsplit
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        shape = oracle.ViGShape(192, 3, 2, 1.0, 1.0, True, True, num_classes=16)
        model = vig_b200.ViG.from_shape(shape)
        model.load_state_dict(oracle.make_state_dict(shape, seed=4))
        model = model.cuda().bfloat16().eval()
        images = oracle.make_images(2, size, seed=6).cuda().bfloat16()
        with torch.no_grad():
            split = seqsplit.vig_forward_sequence_parallel(model, images)
            whole = model(images)
        ret[rank] = (split.float().cpu(), whole.float().cpu())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("size", [224, 512])
def test_row_split_forward_matches_single_gpu(size):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), size, ret), nprocs=world, join=True)
    ref = oracle.vig_forward(oracle.make_state_dict(oracle.ViGShape(192, 3, 2, 1.0, 1.0, True, True, num_classes=16), seed=4),
                             oracle.make_images(2, size, seed=6), oracle.ViGShape(192, 3, 2, 1.0, 1.0, True, True, num_classes=16))
    for r in range(world):
        split, whole = ret[r]
        scale = whole.abs().max()
        e_split, e_ref = float((split - whole).abs().max() / scale), float((split - ref).abs().max() / ref.abs().max())
        print(f"rank {r}: split vs single GPU {e_split:.2e}, split vs fp32 oracle {e_ref:.2e}")
        assert e_split < 1e-2          # same arithmetic up to bf16 rounding of boundary data
        assert e_ref < 2e-2            # and within the bf16 bar of the fp32 oracle
