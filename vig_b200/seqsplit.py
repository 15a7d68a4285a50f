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
