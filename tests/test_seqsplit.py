"""Sequence-split bi-GLA: the fold of per-slice summaries reproduces the unsplit scan.
CPU: real ranks over gloo with the oracle standing in for the CUDA operator (host logic + collective).
GPU: the slices of P emulated ranks run one after the other on one device through the C ABI."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from conftest import rel_err
from vig_b200 import seqsplit


def _oracle_summary(q, k, v, gf, gb, **kw):
    _, s_f, s_b = oracle.naive_bi_gla(q, k, v, gf, gb, return_states=True)
    return seqsplit.pack_summary(s_f, gf.float().sum(2), s_b, gb.float().sum(2))


def _oracle_scan(q, k, v, gf, gb, init_f, init_b, **kw):
    return oracle.naive_bi_gla(q, k, v, gf, gb, init_fwd=init_f, init_bwd=init_b, out_scale=kw.get("out_scale", 1.0))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, L, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ins = oracle.make_bigla_inputs(1, 2, L, 32, 64, seed=12)
        per = L // world
        sl = [t[:, :, rank * per:(rank + 1) * per if rank < world - 1 else L] for t in ins]
        o = seqsplit.bi_gla_sequence_parallel(*sl, summary_fn=_oracle_summary, scan_fn=_oracle_scan, out_scale=0.5)
        ret[rank] = o
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_split_over_gloo_matches_unsplit_oracle(world):
    L = 101
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), L, ret), nprocs=world, join=True)
    ref = oracle.naive_bi_gla(*oracle.make_bigla_inputs(1, 2, L, 32, 64, seed=12), out_scale=0.5)
    got = torch.cat([ret[r] for r in range(world)], dim=2)
    assert rel_err(got, ref) < 1e-5


def test_fold_with_outer_initial_states():
    ins = oracle.make_bigla_inputs(1, 1, 60, 32, 64, seed=3)
    g = torch.Generator().manual_seed(1)
    i_f, i_b = torch.randn(1, 1, 32, 64, generator=g), torch.randn(1, 1, 32, 64, generator=g)
    ref = oracle.naive_bi_gla(*ins, init_fwd=i_f, init_bwd=i_b)
    cuts = [0, 13, 40, 60]
    slices = [[t[:, :, a:b] for t in ins] for a, b in zip(cuts[:-1], cuts[1:])]
    summaries = [_oracle_summary(*s) for s in slices]
    outs = []
    for r, s in enumerate(slices):
        s_f, s_b = seqsplit.fold(summaries, r, 32, 64, init_fwd=i_f, init_bwd=i_b)
        outs.append(_oracle_scan(*s, s_f, s_b))
    assert rel_err(torch.cat(outs, 2), ref) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,P,L", [(torch.float32, 4, 1000), (torch.bfloat16, 4, 4096), (torch.bfloat16, 8, 16384)])
def test_sequence_split_on_gpu_matches_unsplit(dtype, P, L):
    import vig_b200
    B, H, dk, dv = 1, 2, 64, 64
    ins = [t.to("cuda", dtype) for t in oracle.make_bigla_inputs(B, H, L, dk, dv, seed=8)]
    whole = vig_b200.bi_gla(*ins, out_scale=0.5)
    per = (L + P - 1) // P
    slices = [[t[:, :, r * per:min(L, (r + 1) * per)] for t in ins] for r in range(P)]
    summaries = [seqsplit.cuda_summary(*s) for s in slices]          # what each rank would all-gather
    outs = []
    for r, s in enumerate(slices):
        s_f, s_b = seqsplit.fold(summaries, r, dk, dv)
        outs.append(seqsplit.cuda_scan(*s, s_f, s_b, out_scale=0.5))
    got = torch.cat(outs, 2)
    tol = 1e-4 if dtype == torch.float32 else 1e-3 * 8          # split == unsplit up to bf16 rounding of boundary states
    assert rel_err(got.float(), whole.float()) < tol
    if L <= 4096:
        ref = oracle.naive_bi_gla(*[t.float().cpu() for t in ins], out_scale=0.5)
        assert rel_err(got.float(), ref) < (1e-4 if dtype == torch.float32 else 2e-2)


def _halo_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w, C = 5, 8
        x = torch.arange(2 * 3 * w * C, dtype=torch.float32).reshape(2, 3 * w, C) + 1000 * rank     # my 3 rows of the grid
        top, bottom = seqsplit.exchange_halo_rows(x, w, None, rank, world)
        ret[rank] = (top, bottom, x[:, :w].clone(), x[:, -w:].clone())
    finally:
        dist.destroy_process_group()


def test_halo_rows_come_from_the_two_neighbours_only():
    world = 3
    ret = mp.Manager().dict()
    mp.spawn(_halo_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        top, bottom, first, last = ret[r]
        assert (top is None) == (r == 0) and (bottom is None) == (r == world - 1)      # image border: zero padding
        if r > 0:
            assert torch.equal(top, ret[r - 1][3])            # the last row of the rank above
        if r < world - 1:
            assert torch.equal(bottom, ret[r + 1][2])         # the first row of the rank below


@pytest.mark.parametrize("size,world", [(224, 2), (224, 3), (320, 4), (128, 8)])
def test_stem_split_by_image_rows_matches_whole_stem(size, world):
    """The row split of the stem that ``vig_forward_sequence_parallel`` performs (own image rows plus the patch row above,
    first patch row of the result dropped) reproduces the stem of the whole image: written with the oracle's stem on CPU."""
    shape = oracle.ViGShape(192, 3, 1, 1.0, 1.0, True, True, num_classes=16)
    sd = {k: v.float() for k, v in oracle.make_state_dict(shape, seed=3).items()}
    images = oracle.make_images(2, size, seed=size)
    whole, (h, w) = oracle.patch_embed_v2(sd, images)
    whole = whole.view(2, h, w, -1)
    patch = 16
    for rank in range(world):
        r0, r1 = seqsplit.row_range(h, rank, world)
        top = 1 if r0 > 0 else 0
        sub = images[:, :, patch * (r0 - top):patch * r1]
        tokens, (hs, ws) = oracle.patch_embed_v2(sd, sub)
        assert (hs, ws) == (r1 - r0 + top, w)
        part = tokens.view(2, hs, w, -1)[:, top:]
        assert rel_err(part, whole[:, r0:r1]) < 1e-5
