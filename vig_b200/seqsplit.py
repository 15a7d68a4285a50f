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
    """Entering states of slice ``rank`` from the gathered summaries (list over ranks, or one stacked
    ``[world, B, H, 2, dk*dv+dk]`` tensor; slice order = rank order).

    forward:  S = init_fwd; for r < rank:            S = exp(D_f[r]) * S + U_f[r]
    backward: S = init_bwd; for r > rank, descending: S = exp(D_b[r]) * S + U_b[r]

    Unrolled, S = sum_r w_r * U_r with w_r = exp(sum of the log-decays of the slices between r and this one).  With
    P = cumulative sum of D over the rank axis (one call for both directions), the slices between r and ``rank`` sum to
    ``P[rank-1] - P[r]`` (forward, r < rank) and ``P[r-1] - P[rank]`` (backward, r > rank): one cumulative sum, and per
    direction a subtraction, an exponential and a weighted sum -- a dozen launches whatever the world size (the host's
    launch time is what bounds the split forward at 8 ranks).
    """
    msgs = summaries if torch.is_tensor(summaries) else torch.stack(list(summaries))
    world = msgs.shape[0]
    u = msgs[..., :dk * dv].unflatten(-1, (dk, dv))                    # [world, B, H, 2, dk, dv]
    d = msgs[..., dk * dv:]                                            # [world, B, H, 2, dk]
    prefix = torch.cumsum(d, 0)                                        # inclusive, both directions at once

    def zero_state():
        return torch.zeros_like(u[0, :, :, 0])

    if rank > 0:
        # forward: slices r = 0 .. rank-1, each decayed by the slices r+1 .. rank-1
        w = (prefix[rank - 1, :, :, 0].unsqueeze(0) - prefix[:rank, :, :, 0]).exp()
        s_f = (u[:rank, :, :, 0] * w.unsqueeze(-1)).sum(0)
        if init_fwd is not None:
            s_f = s_f + init_fwd.float() * prefix[rank - 1, :, :, 0].exp().unsqueeze(-1)
    else:
        s_f = zero_state() if init_fwd is None else init_fwd.float().clone()
    if rank + 1 < world:
        # backward: slices r = rank+1 .. world-1, each decayed by the slices rank+1 .. r-1
        w = (prefix[rank:world - 1, :, :, 1] - prefix[rank, :, :, 1].unsqueeze(0)).exp()
        s_b = (u[rank + 1:, :, :, 1] * w.unsqueeze(-1)).sum(0)
        if init_bwd is not None:
            s_b = s_b + init_bwd.float() * (prefix[world - 1, :, :, 1] - prefix[rank, :, :, 1]).exp().unsqueeze(-1)
    else:
        s_b = zero_state() if init_bwd is None else init_bwd.float().clone()
    return s_f.contiguous(), s_b.contiguous()


def exchange(msg, group=None):
    """All-gather of the per-rank summaries into one ``[world, ...]`` tensor (one collective, one output buffer)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(msg.shape), dtype=msg.dtype, device=msg.device)
    if msg.is_cuda:
        dist.all_gather_into_tensor(out, msg.contiguous(), group=group)
    else:                                                   # gloo (CPU ranks in the tests) has only the list form
        dist.all_gather(list(out.unbind(0)), msg.contiguous(), group=group)
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


def exchange_halo_rows(x, w, group, rank, world):
    """Send my first image row up and my last row down, receive the neighbours' rows next to mine: two point-to-point
    transfers per neighbour, nothing from the ranks further away.  Returns ``(top, bottom)``, ``None`` at the image border."""
    B, L, C = x.shape
    first, last = x[:, :w].contiguous(), x[:, L - w:].contiguous()
    top = torch.empty_like(first) if rank > 0 else None
    bottom = torch.empty_like(first) if rank + 1 < world else None
    peer = lambda r: dist.get_global_rank(group, r) if group is not None else r
    ops_ = []
    if rank > 0:
        ops_ += [dist.P2POp(dist.isend, first, peer(rank - 1), group), dist.P2POp(dist.irecv, top, peer(rank - 1), group)]
    if rank + 1 < world:
        ops_ += [dist.P2POp(dist.isend, last, peer(rank + 1), group), dist.P2POp(dist.irecv, bottom, peer(rank + 1), group)]
    for req in dist.batch_isend_irecv(ops_) if ops_ else []:
        req.wait()
    return top, bottom


def _halo_local_fn(group, rank, world):
    """Depthwise conv over this rank's rows with one row of halo from each neighbour, read in place by the kernel."""
    from . import ops

    def local_fn(x, taps, bias, hw, act):
        rows, w = hw
        top, bottom = exchange_halo_rows(x, w, group, rank, world)
        if x.dtype == torch.float32:                         # the halo form of the kernel is 16-bit only: pad and slice
            B, L, C = x.shape
            z = torch.zeros_like(x[:, :w])
            padded = torch.cat([z if top is None else top, x, z if bottom is None else bottom], dim=1)
            return ops.dwconv3x3(padded, taps, bias, (rows + 2, w), act)[:, w:L + w].contiguous()
        return ops.dwconv3x3(x, taps, bias, hw, act, top=top, bottom=bottom)
    return local_fn


def vig_forward_sequence_parallel(model, images, group=None):
    """Logits of ``model`` (a ``vig_b200.ViG`` in eval mode) with the token sequence of every image split across
    the ranks of ``group`` by rows of the patch grid.  Every rank passes the same ``images`` and gets the same
    logits.  The stem is split by image rows like the blocks (one patch row of overlap above each rank's rows)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    patch = 2 * model.patch_embed.stride
    B, _, H_img, W_img = images.shape
    if H_img % patch or W_img % patch:
        raise ValueError("image sides must be multiples of the patch size")
    h, w = H_img // patch, W_img // patch
    if h < world:
        raise ValueError("more ranks than rows in the patch grid")
    r0, r1 = row_range(h, rank, world)
    # The stem is split too: a patch row depends on image rows 16 p - 9 .. 16 p + 15 (conv k9 s8 p1, then conv k3 s2 p1),
    # so a rank runs the stem on its own image rows plus the patch row above and drops that row of the result; nothing
    # below its last row is needed.
    top = 1 if r0 > 0 else 0
    sub = images[:, :, patch * (r0 - top):patch * r1].contiguous()
    tokens, (hs, _) = model.patch_embed(sub)
    C = tokens.shape[-1]
    tokens = tokens.view(B, hs, w, C)[:, top:]
    x = tokens + model._pos((h, w)).view(1, h, w, C)[:, r0:r1]
    x = x.reshape(B, (r1 - r0) * w, C).contiguous()
    hooks = dict(patch_resolution=(r1 - r0, w), local_fn=_halo_local_fn(group, rank, world),
                 scan_fn=lambda q, k, v, gf, gb, **kw: bi_gla_sequence_parallel(q, k, v, gf, gb, group=group, **kw))
    hidden, residual = x, None
    for blk in model.blocks:
        hidden, residual = blk.forward_deferred(hidden, residual, **hooks)
    x = model.norm(hidden, residual)
    pooled = x.float().sum(dim=1)
    dist.all_reduce(pooled, group=group)
    return model.head((pooled / (h * w)).to(x.dtype))


def phase_times(model, images, group=None, steps=3):
    """Milliseconds per forward that this rank spends in the parts the sequence split adds (CUDA events around each call:
    ``summary`` = states-only scan + packing, ``all_gather``, ``fold``, ``halo_exchange``) and in the scan proper and the
    stem, averaged over ``steps`` forwards after one warm-up.  A collective's figure includes the time this rank waits for
    the slowest one."""
    import sys
    mod = sys.modules[__name__]
    events = {}

    def timed(name, fn):
        def inner(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **k)
            e1.record()
            events.setdefault(name, []).append((e0, e1))
            return r
        return inner

    saved = {n: getattr(mod, n) for n in ("exchange", "fold", "exchange_halo_rows", "bi_gla_sequence_parallel")}
    summary_fn, scan_fn = timed("summary", cuda_summary), timed("scan", cuda_scan)
    inner_split = saved["bi_gla_sequence_parallel"]
    stem = model.patch_embed.forward
    try:
        mod.exchange = timed("all_gather", saved["exchange"])
        mod.fold = timed("fold", saved["fold"])
        mod.exchange_halo_rows = timed("halo_exchange", saved["exchange_halo_rows"])
        mod.bi_gla_sequence_parallel = lambda q, k, v, gf, gb, group=None, **kw: inner_split(
            q, k, v, gf, gb, group=group, summary_fn=summary_fn, scan_fn=scan_fn, **kw)
        model.patch_embed.forward = timed("stem", stem)
        with torch.no_grad():
            vig_forward_sequence_parallel(model, images, group)
            torch.cuda.synchronize()
            events.clear()
            for _ in range(steps):
                vig_forward_sequence_parallel(model, images, group)
            torch.cuda.synchronize()
    finally:
        for n, f in saved.items():
            setattr(mod, n, f)
        model.patch_embed.forward = stem
    return {n: sum(a.elapsed_time(b) for a, b in ev) / steps for n, ev in events.items()}
