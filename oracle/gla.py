"""Naive recurrent gated linear attention on CPU, fp32 (or fp64): the operator oracle.

Restates ``flash-linear-attention/fla/ops/gla/naive.py:13-58`` (``naive_recurrent_gla``):
for every token, in scan order, ``h = h * exp(g_t)[..., None] + k_t^T v_t`` and
``o_t = (q_t * scale) . h``; the gate of token t decays the incoming state before
token t's own outer product is added, so a token always sees itself.

The bidirectional operator of ViG is the forward scan with the forward gates plus
the reverse scan with the backward gates, both indexed by the original token
position (``fla/ops/gla/recurrent_fuse.py:77-80`` walks the second half of the gate
tensor from the last token to the first).  The reference's wrappers then halve the
sum (``recurrent_fuse.py:442``) and the eval branch of the model halves it again
(``classification/models/vig.py:443``); here that is the explicit ``out_scale``.
"""
import torch


def naive_gla(q, k, v, g, scale=None, initial_state=None, reverse=False, dtype=torch.float32):
    """One-direction scan.  q,k,g: [B,H,L,dk]; v: [B,H,L,dv].  Returns (o [B,H,L,dv], final_state [B,H,dk,dv])."""
    q, k, v, g = (t.detach().to("cpu", dtype) for t in (q, k, v, g))
    B, H, L, dk = q.shape
    dv = v.shape[-1]
    if scale is None or scale == -1:
        scale = dk ** -0.5
    h = torch.zeros(B, H, dk, dv, dtype=dtype)
    if initial_state is not None:
        h = h + initial_state.detach().to("cpu", dtype)
    o = torch.zeros(B, H, L, dv, dtype=dtype)
    order = range(L - 1, -1, -1) if reverse else range(L)
    for i in order:
        decay = g[:, :, i].exp()
        h = h * decay[..., None] + k[:, :, i, :, None] * v[:, :, i, None, :]
        o[:, :, i] = ((q[:, :, i] * scale)[..., None] * h).sum(-2)
    return o, h


def naive_bi_gla(q, k, v, g_fwd, g_bwd, scale=None, out_scale=1.0, dtype=torch.float32,
                 init_fwd=None, init_bwd=None, return_states=False):
    """Bidirectional operator: out_scale * (forward scan with g_fwd + reverse scan with g_bwd)."""
    o_f, s_f = naive_gla(q, k, v, g_fwd, scale, init_fwd, reverse=False, dtype=dtype)
    o_b, s_b = naive_gla(q, k, v, g_bwd, scale, init_bwd, reverse=True, dtype=dtype)
    o = (o_f + o_b) * out_scale
    return (o, s_f, s_b) if return_states else o


def chunked_bi_gla_f64(q, k, v, g_fwd, g_bwd, scale=None, out_scale=1.0, chunk=64):
    """The chunked algebra the CUDA kernels use, in fp64 with dense per-chunk matrices.

    Not the reference's code path; it is here so the tests can show that the chunked
    form (intra-chunk masked scores with cumulative log-gates, inter-chunk state
    products, per-chunk state updates; ``fla/ops/gla/chunk_fuse.py:76-97,244-254``
    describe the reference's version) equals the naive recurrence.
    """
    f64 = torch.float64
    q, k, v, gf, gb = (t.detach().to("cpu", f64) for t in (q, k, v, g_fwd, g_bwd))
    B, H, L, dk = q.shape
    dv = v.shape[-1]
    if scale is None or scale == -1:
        scale = dk ** -0.5
    o = torch.zeros(B, H, L, dv, dtype=f64)
    starts = list(range(0, L, chunk))
    # forward direction
    S = torch.zeros(B, H, dk, dv, dtype=f64)
    for s in starts:
        e = min(L, s + chunk)
        G = gf[:, :, s:e].cumsum(2)                                  # inclusive prefix
        A = torch.einsum("bhid,bhjd->bhij", q[:, :, s:e] * scale * G.exp(), k[:, :, s:e] * (-G).exp())
        A = A.tril()
        o[:, :, s:e] += A @ v[:, :, s:e] + (q[:, :, s:e] * scale * G.exp()) @ S
        last = G[:, :, -1:]
        S = S * last.transpose(2, 3).exp() + (k[:, :, s:e] * (last - G).exp()).transpose(2, 3) @ v[:, :, s:e]
    # backward direction
    S = torch.zeros(B, H, dk, dv, dtype=f64)
    for s in reversed(starts):
        e = min(L, s + chunk)
        R = gb[:, :, s:e].flip(2).cumsum(2).flip(2)                  # inclusive suffix
        A = torch.einsum("bhid,bhjd->bhij", q[:, :, s:e] * scale * R.exp(), k[:, :, s:e] * (-R).exp())
        A = A.triu()
        o[:, :, s:e] += A @ v[:, :, s:e] + (q[:, :, s:e] * scale * R.exp()) @ S
        first = R[:, :, :1]
        S = S * first.transpose(2, 3).exp() + (k[:, :, s:e] * (first - R).exp()).transpose(2, 3) @ v[:, :, s:e]
    return o * out_scale
