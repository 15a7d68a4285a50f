"""Sequence-split bi-GLA across ranks: for very long sequences (L >= 16384) each rank owns a contiguous
slice of the tokens and only per-head boundary states cross the interconnect.

The scan is associative: a slice acts on an entering state S as ``S -> diag(exp(D)) S + U`` where ``U`` is the
slice's end state from a zero start and ``D`` its summed log-gates (per key channel).  So

    1. every rank computes (U_f, D_f, U_b, D_b) of its slice           -- ``local_summary`` (no output pass)
    2. one all-gather of ``[B, H, 2, dk*dv + dk]`` fp32 per rank         -- ``exchange`` (NCCL on GPUs, gloo in tests)
    3. every rank folds its predecessors (forward) / successors (backward) into its entering states -- ``fold``
    4. and runs the full operator on its slice with those initial states.

The reference has no sequence parallelism (its hooks for it are the ``initial_state`` / ``output_final_state``
arguments of ``fused_chunk_gla``, ``fla/ops/gla/chunk_fuse.py:554-572``); the collective is issued by the host
through ``torch.distributed`` and lands in local memory before any kernel reads it.

``fold`` is plain tensor arithmetic and runs on any device; the per-slice work is injected (``summary_fn`` /
``scan_fn``) so the same driver is exercised on CPU ranks with a stand-in for the CUDA operator.
"""
import torch
import torch.distributed as dist


def pack_summary(u_f, d_f, u_b, d_b):
    """[B,H,dk,dv] x2 and [B,H,dk] x2  ->  one [B,H,2,dk*dv+dk] fp32 message."""
    B, H, dk, dv = u_f.shape
    f = torch.cat([u_f.reshape(B, H, dk * dv), d_f], dim=-1)
    b = torch.cat([u_b.reshape(B, H, dk * dv), d_b], dim=-1)
    return torch.stack([f, b], dim=2).float().contiguous()


def unpack_summary(msg, dk, dv):
    u = msg[..., :dk * dv].reshape(*msg.shape[:-1], dk, dv)
    d = msg[..., dk * dv:]
    return u[:, :, 0], d[:, :, 0], u[:, :, 1], d[:, :, 1]


def fold(summaries, rank, dk, dv, init_fwd=None, init_bwd=None):
    """Entering states of slice ``rank`` from the gathered summaries (list over ranks, slice order = rank order).

    forward:  S = init_fwd; for r < rank:            S = exp(D_f[r]) * S + U_f[r]
    backward: S = init_bwd; for r > rank, descending: S = exp(D_b[r]) * S + U_b[r]
    """
    u_f0, _, _, _ = unpack_summary(summaries[0], dk, dv)
    s_f = torch.zeros_like(u_f0) if init_fwd is None else init_fwd.float().clone()
    s_b = torch.zeros_like(u_f0) if init_bwd is None else init_bwd.float().clone()
    for r in range(rank):
        u, d, _, _ = unpack_summary(summaries[r], dk, dv)
        s_f = s_f * d.exp().unsqueeze(-1) + u
    for r in range(len(summaries) - 1, rank, -1):
        _, _, u, d = unpack_summary(summaries[r], dk, dv)
        s_b = s_b * d.exp().unsqueeze(-1) + u
    return s_f.contiguous(), s_b.contiguous()


def exchange(msg, group=None):
    """All-gather of the per-rank summaries; returns the list over ranks."""
    world = dist.get_world_size(group)
    out = [torch.empty_like(msg) for _ in range(world)]
    dist.all_gather(out, msg, group=group)
    return out


def cuda_summary(q, k, v, g_fwd, g_bwd, **kw):
    """Slice summary with the CUDA operator (states only: no output pass, q is not read)."""
    from . import ops
    _, ex = ops.bi_gla(q, k, v, g_fwd, g_bwd, output_final_state=True, output_logdecay=True, want_output=False,
                       gate_logit_normalizer=kw.get("gate_logit_normalizer", 0.0), clamp_min=kw.get("clamp_min"))
    return pack_summary(ex["final_fwd"], ex["logdecay_fwd"], ex["final_bwd"], ex["logdecay_bwd"])


def cuda_scan(q, k, v, g_fwd, g_bwd, init_fwd, init_bwd, **kw):
    from . import ops
    return ops.bi_gla(q, k, v, g_fwd, g_bwd, init_state_fwd=init_fwd, init_state_bwd=init_bwd, **kw)


def bi_gla_sequence_parallel(q, k, v, g_fwd, g_bwd, group=None, summary_fn=cuda_summary, scan_fn=cuda_scan, **kw):
    """bi-GLA of this rank's token slice ([B,H,L_local,d] tensors); ranks hold consecutive slices in rank order.
    ``kw`` (scale, out_scale, gate_logit_normalizer, clamp_min, out) is passed to the operator."""
    rank = dist.get_rank(group)
    dk, dv = k.shape[-1], v.shape[-1]
    skw = {n: kw[n] for n in ("gate_logit_normalizer", "clamp_min") if n in kw}
    msg = summary_fn(q, k, v, g_fwd, g_bwd, **skw)
    summaries = exchange(msg, group)
    s_f, s_b = fold(summaries, rank, dk, dv)
    return scan_fn(q, k, v, g_fwd, g_bwd, s_f, s_b, **kw)


# ---------------------------------------------------------------------------------------------------------
# Whole-model sequence parallelism: the token grid is split by image rows.  Everything in a block is token-local
# except (1) the depthwise 3x3 conv, which needs one row of halo from each neighbour, and (2) the scan, which
# needs the boundary states; both are one small all-gather per block.  The final average pool is one all-reduce.

def row_range(h, rank, world):
    """Rows [r0, r1) of an h-row token grid owned by ``rank`` (as even as possible, earlier ranks get the extra)."""
    base, extra = divmod(h, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def _halo_local_fn(group, rank, world):
    """Depthwise conv over this rank's rows with one row of halo gathered from the neighbours."""
    from . import ops

    def local_fn(x, taps, bias, hw, act):
        rows, w = hw
        B, L, C = x.shape
        edges = torch.stack([x[:, :w], x[:, L - w:]], dim=0).contiguous()          # my first and last row
        gathered = [torch.empty_like(edges) for _ in range(world)]
        dist.all_gather(gathered, edges, group=group)
        top = gathered[rank - 1][1] if rank > 0 else torch.zeros_like(edges[0])        # zero rows = the conv's padding
        bot = gathered[rank + 1][0] if rank + 1 < world else torch.zeros_like(edges[0])
        padded = torch.cat([top, x, bot], dim=1)
        y = ops.dwconv3x3(padded, taps, bias, (rows + 2, w), act)
        return y[:, w:L + w].contiguous()
    return local_fn


def vig_forward_sequence_parallel(model, images, group=None):
    """Logits of ``model`` (a ``vig_b200.ViG`` in eval mode) with the token sequence of every image split across
    the ranks of ``group`` by rows of the patch grid.  Every rank passes the same ``images`` and gets the same
    logits.  The stem is computed redundantly on every rank (about 4 % of the model's work)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    tokens, (h, w) = model.patch_embed(images)
    if h < world:
        raise ValueError("more ranks than rows in the patch grid")
    B, _, C = tokens.shape
    x = tokens + model._pos((h, w))
    r0, r1 = row_range(h, rank, world)
    x = x.view(B, h, w, C)[:, r0:r1].reshape(B, (r1 - r0) * w, C).contiguous()
    hooks = dict(patch_resolution=(r1 - r0, w), local_fn=_halo_local_fn(group, rank, world),
                 scan_fn=lambda q, k, v, gf, gb, **kw: bi_gla_sequence_parallel(q, k, v, gf, gb, group=group, **kw))
    hidden, residual = x, None
    for blk in model.blocks:
        hidden, residual = blk.forward_deferred(hidden, residual, **hooks)
    x = model.norm(hidden, residual)
    pooled = x.float().sum(dim=1)
    dist.all_reduce(pooled, group=group)
    return model.head((pooled / (h * w)).to(x.dtype))
