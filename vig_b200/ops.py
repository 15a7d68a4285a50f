"""Operator API with the reference's names and argument conventions, backed by the CUDA library.

``bid_fused_recurrent_gla`` / ``fused_recurrent_gla`` mirror ``fla/ops/gla/recurrent_fuse.py:631-685``,
``fused_chunk_gla`` mirrors ``fla/ops/gla/chunk_fuse.py:554-572`` and ``chunk_gla``
``fla/ops/gla/chunk.py:561-580``; ``bi_gla`` is the explicit form of the merged operator.
Tensors are ``[B, H, L, d]`` views with a contiguous last dimension; no copies are made.
``bi_gla`` and the one-direction entry points are differentiable (``vig_bigla_bwd``); the block's other kernels
are inference-only.
"""
import math

import torch

from . import _lib

_NAN = float("nan")
_ws_cache = {}


def _workspace(nbytes, device):
    """Per-device scratch buffer that only grows (allocated through torch's caching allocator)."""
    if nbytes == 0:
        return None
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    buf = _ws_cache.get(device)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=device)
        _ws_cache[device] = buf
    return buf


def bi_gla(q, k, v, g_fwd, g_bwd, scale=-1, out_scale=1.0, *, out=None, gate_logit_normalizer=0.0, clamp_min=None,
           init_state_fwd=None, init_state_bwd=None, output_final_state=False, output_logdecay=False,
           dir_mask=3, impl=_lib.IMPL_AUTO, want_output=True, status=None):
    """o_t = out_scale * scale * q_t (S^f_t + S^b_t) with separate forward / backward log-gates.

    ``status``: optional int32 CUDA tensor of one element; kernels OR error bits into it (bit 0: a bounded wait
    ran out, bit 1: a chunk's cumulative gate left the range of the tensor-core factorisation).
    Returns ``o`` or ``(o, extras)`` where ``extras`` holds ``final_fwd/final_bwd`` ([B,H,dk,dv] fp32) and
    ``logdecay_fwd/logdecay_bwd`` ([B,H,dk] fp32) when requested.
    """
    _lib.require_cuda(q, k, v, g_fwd, g_bwd)
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g_fwd, g_bwd)):
        if (init_state_fwd is not None or init_state_bwd is not None or output_final_state or output_logdecay
                or out is not None or not want_output):
            raise NotImplementedError("the differentiable form takes no states and allocates its own output")
        return _BiGLAFunction.apply(q, k, v, g_fwd, g_bwd, float(scale if scale is not None else -1), float(out_scale),
                                    float(gate_logit_normalizer), clamp_min, dir_mask, impl)
    B, H, L, dk = k.shape
    dv = v.shape[-1]
    code = _lib.dtype_code(k)
    for t in (q, v, g_fwd, g_bwd):
        if t is not None and t.dtype != k.dtype:
            raise TypeError("q, k, v and the gates must share one dtype")
    dev = k.device
    if want_output:
        if out is None:
            out = torch.empty(B, H, L, dv, dtype=v.dtype, device=dev)
    else:
        out = None
    f32 = dict(dtype=torch.float32, device=dev)
    extras = {}
    if output_final_state:
        if dir_mask & 1:
            extras["final_fwd"] = torch.empty(B, H, dk, dv, **f32)
        if dir_mask & 2:
            extras["final_bwd"] = torch.empty(B, H, dk, dv, **f32)
    if output_logdecay:
        if dir_mask & 1:
            extras["logdecay_fwd"] = torch.empty(B, H, dk, **f32)
        if dir_mask & 2:
            extras["logdecay_bwd"] = torch.empty(B, H, dk, **f32)
    for s in (init_state_fwd, init_state_bwd):
        if s is not None and (s.dtype != torch.float32 or not s.is_contiguous() or s.shape != (B, H, dk, dv)):
            raise ValueError("initial states must be contiguous fp32 [B,H,dk,dv]")
    L_ = _lib.lib()
    nbytes = L_.vig_bigla_workspace_bytes(B, H, L, dk, dv, code, impl)
    ws = _workspace(nbytes, dev)
    st = L_.vig_bigla_fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g_fwd), _lib.ptr(g_bwd), _lib.ptr(out),
        B, H, L, dk, dv, code,
        _lib.strides3(q) if q is not None else None, _lib.strides3(k), _lib.strides3(v),
        _lib.strides3(g_fwd) if g_fwd is not None else None, _lib.strides3(g_bwd) if g_bwd is not None else None,
        _lib.strides3(out) if out is not None else None,
        float(scale if scale is not None else -1), float(out_scale), float(gate_logit_normalizer),
        _NAN if clamp_min is None else float(clamp_min),
        _lib.ptr(init_state_fwd), _lib.ptr(init_state_bwd),
        _lib.ptr(extras.get("final_fwd")), _lib.ptr(extras.get("final_bwd")),
        _lib.ptr(extras.get("logdecay_fwd")), _lib.ptr(extras.get("logdecay_bwd")),
        dir_mask, impl, _lib.ptr(ws), ws.numel() if ws is not None else 0, _lib.ptr(status), _lib.stream_ptr())
    _lib.check(st, "vig_bigla_fwd")
    if extras:
        return out, extras
    return out


def bi_gla_backward(q, k, v, g_fwd, g_bwd, d_out, scale=-1, out_scale=1.0, dir_mask=3):
    """Gradients of ``bi_gla`` with log-space gates: ``(dq, dk, dv, dg_fwd, dg_bwd)`` (``None`` for a direction that
    is masked out).  The kernels deliver ``e = dq*q - dk*k`` per direction; the gate gradients are its cumulative
    sums over the tokens (``fla/ops/gla/chunk_fuse.py:506-516`` does the same in PyTorch)."""
    _lib.require_cuda(q, k, v, d_out)
    B, H, L, dk = k.shape
    dv = v.shape[-1]
    dev = k.device
    dq, dk_, dv_ = (torch.empty(B, H, L, d, dtype=k.dtype, device=dev) for d in (dk, dk, dv))
    e_f = torch.empty(B, H, L, dk, dtype=torch.float32, device=dev) if dir_mask & 1 else None
    e_b = torch.empty(B, H, L, dk, dtype=torch.float32, device=dev) if dir_mask & 2 else None
    L_ = _lib.lib()
    nbytes = L_.vig_bigla_bwd_workspace_bytes(B, H, L, dk, dv)
    ws = _workspace(nbytes, dev)
    s3 = lambda t: None if t is None else _lib.strides3(t)
    st = L_.vig_bigla_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g_fwd), _lib.ptr(g_bwd), _lib.ptr(d_out),
                          _lib.ptr(dq), _lib.ptr(dk_), _lib.ptr(dv_), _lib.ptr(e_f), _lib.ptr(e_b),
                          B, H, L, dk, dv, _lib.dtype_code(k), s3(q), s3(k), s3(v), s3(g_fwd), s3(g_bwd), s3(d_out),
                          float(scale if scale is not None else -1), float(out_scale), dir_mask,
                          _lib.ptr(ws), ws.numel() if ws is not None else 0, _lib.stream_ptr())
    _lib.check(st, "vig_bigla_bwd")
    dg_f = e_f.flip(2).cumsum(2).flip(2) if e_f is not None else None
    dg_b = e_b.cumsum(2) if e_b is not None else None
    return dq, dk_, dv_, dg_f, dg_b


class _BiGLAFunction(torch.autograd.Function):
    """Differentiable ``bi_gla``: forward through ``vig_bigla_fwd``, backward through ``vig_bigla_bwd``.  Raw gate
    logits are turned into log-gates here so that one backward kernel serves both forms."""

    @staticmethod
    def forward(ctx, q, k, v, g_fwd, g_bwd, scale, out_scale, gate_norm, clamp_min, dir_mask, impl):
        def to_log(x):
            if x is None:
                return None, None
            g = torch.nn.functional.logsigmoid(x.float()) / gate_norm if gate_norm > 0 else x.float()
            if clamp_min is not None:
                g = torch.clamp_min(g, clamp_min)
            return g.to(x.dtype), g
        gf, gf32 = to_log(g_fwd)
        gb, gb32 = to_log(g_bwd)
        with torch.no_grad():
            o = bi_gla(q, k, v, gf, gb, scale=scale, out_scale=out_scale, dir_mask=dir_mask, impl=impl)
        ctx.save_for_backward(q, k, v, g_fwd, g_bwd, gf, gb)
        ctx.cfg = (scale, out_scale, gate_norm, clamp_min, dir_mask)
        return o

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, x_f, x_b, gf, gb = ctx.saved_tensors
        scale, out_scale, gate_norm, clamp_min, dir_mask = ctx.cfg
        dq, dk, dv, dg_f, dg_b = bi_gla_backward(q, k, v, gf, gb, d_out.contiguous(), scale, out_scale, dir_mask)

        def through_gate(dg, x, g):
            if dg is None or x is None:
                return None
            if clamp_min is not None:
                dg = dg * (g.float() > clamp_min)
            if gate_norm > 0:                                       # d logsigmoid(x) / dx = sigmoid(-x)
                dg = dg * torch.sigmoid(-x.float()) / gate_norm
            return dg.to(x.dtype)
        return dq, dk, dv, through_gate(dg_f, x_f, gf), through_gate(dg_b, x_b, gb), None, None, None, None, None, None


def bi_gla_noalloc(q, k, v, g_fwd, g_bwd, out, scale=-1, out_scale=1.0, gate_logit_normalizer=0.0, clamp_min=None,
                   impl=_lib.IMPL_AUTO):
    """``bi_gla`` through the entry point that allocates nothing: the caller supplies ``out`` and the scan's
    scratch is a fixed array inside the library (see ``vig_bigla_fwd_noalloc`` in the header for who needs
    this and for its size limit).  Calls on one device must not overlap on the GPU."""
    _lib.require_cuda(q, k, v, g_fwd, g_bwd, out)
    B, H, L, dk = k.shape
    dv = v.shape[-1]
    st = _lib.lib().vig_bigla_fwd_noalloc(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g_fwd), _lib.ptr(g_bwd), _lib.ptr(out), B, H, L, dk, dv,
        _lib.dtype_code(k), _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(g_fwd), _lib.strides3(g_bwd),
        _lib.strides3(out), float(scale if scale is not None else -1), float(out_scale), float(gate_logit_normalizer),
        _NAN if clamp_min is None else float(clamp_min), impl, None, _lib.stream_ptr())
    _lib.check(st, "vig_bigla_fwd_noalloc")
    return out


def bid_fused_recurrent_gla(q, k, v, gk=None, gv=None, scale=-1, initial_state=None, output_final_state=False,
                            causal=True):
    """``fla/ops/gla/recurrent_fuse.py:659-685``: ``gk`` is ``[2B,H,L,dk]`` (forward gates then backward
    gates, both in original token order); returns ``((o_f + o_b) / 2, None)``."""
    if gk is None or gv is not None or initial_state is not None or output_final_state:
        raise NotImplementedError("only the form ViG calls is implemented: gk given, no gv / states")
    B = q.shape[0]
    if gk.shape[0] != 2 * B:
        raise ValueError("gk must stack forward and backward gates along the batch: [2B,H,L,dk]")
    return bi_gla(q, k, v, gk[:B], gk[B:], scale=scale, out_scale=0.5), None


def _one_direction(q, k, v, g, scale, initial_state, output_final_state, reverse):
    mask = 2 if reverse else 1
    kw = dict(init_state_bwd=initial_state) if reverse else dict(init_state_fwd=initial_state)
    if initial_state is not None:
        kw = {n: s.detach().float().contiguous() for n, s in kw.items()}
    res = bi_gla(q, k, v, None if reverse else g, g if reverse else None, scale=scale, dir_mask=mask,
                 output_final_state=output_final_state, **kw)
    if output_final_state:
        o, ex = res
        return o, ex["final_bwd" if reverse else "final_fwd"]
    return res, None


def fused_chunk_gla(q, k, v, g, scale=-1, initial_state=None, output_final_state=False):
    """``fla/ops/gla/chunk_fuse.py:554-572``: causal scan, ``(o, final_state)``; ``final_state`` fp32 or None."""
    return _one_direction(q, k, v, g, scale, initial_state, output_final_state, reverse=False)


def chunk_gla(q, k, v, g, scale=-1, initial_state=None, output_final_state=False):
    """``fla/ops/gla/chunk.py:561-580``: same function as ``fused_chunk_gla``."""
    return _one_direction(q, k, v, g, scale, initial_state, output_final_state, reverse=False)


def fused_recurrent_gla(q, k, v, gk=None, gv=None, scale=-1, initial_state=None, output_final_state=False,
                        causal=True, reverse=False):
    """``fla/ops/gla/recurrent_fuse.py:631-657`` with key-wise gates only."""
    if gk is None or gv is not None:
        raise NotImplementedError("only key-wise gates (gk) are implemented")
    return _one_direction(q, k, v, gk, scale, initial_state, output_final_state, reverse=reverse)


# --------------------------------------------------------------------------------------------------
def dwconv3x3(x, weight_tap_major, bias, hw, act_silu, out=None):
    """Depthwise 3x3 (+SiLU) on ``[B, h*w, C]`` tokens; ``weight_tap_major`` is ``[9, C]``."""
    _lib.require_cuda(x, weight_tap_major)
    B, L, C = x.shape
    h, w = hw
    if h * w != L or not x.is_contiguous():
        raise ValueError("x must be contiguous [B, h*w, C]")
    y = torch.empty_like(x) if out is None else out
    st = _lib.lib().vig_dwconv3x3_fwd(_lib.ptr(x), _lib.ptr(weight_tap_major), _lib.ptr(bias), _lib.ptr(y),
                                      B, h, w, C, int(bool(act_silu)), _lib.dtype_code(x), _lib.stream_ptr())
    _lib.check(st, "vig_dwconv3x3_fwd")
    return y


def _rows(t, what):
    """Row stride of a [B, L, N] tensor whose (b, l) dimensions collapse to one row index."""
    if t.stride(-1) != 1 or t.stride(0) != t.shape[1] * t.stride(1):
        raise ValueError(f"{what} must be a row-major [B, L, N] tensor or a column slice of one")
    return t.stride(1)


def gate_inject(o, local, gate_logits, w_gnorm, w_lnorm, eps, out_act, out=None):
    """``o`` is a ``[B,H,L,dv]`` view (any b/h/l strides); ``local``, ``gate_logits`` are ``[B,L,H*dv]``
    (column slices of a wider projection are fine)."""
    _lib.require_cuda(o, local, gate_logits)
    B, H, L, dv = o.shape
    y = torch.empty(B, L, H * dv, dtype=local.dtype, device=local.device) if out is None else out
    st = _lib.lib().vig_gate_inject_fwd(_lib.ptr(o), _lib.strides3(o), _lib.ptr(local), _lib.ptr(gate_logits),
                                        _lib.ptr(w_gnorm), _lib.ptr(w_lnorm), _lib.ptr(y),
                                        _rows(local, "local"), _rows(gate_logits, "gate_logits"), _rows(y, "out"),
                                        B, H, L, dv, float(eps), int(bool(out_act)), _lib.dtype_code(local), _lib.stream_ptr())
    _lib.check(st, "vig_gate_inject_fwd")
    return y


def add_rmsnorm(x, weight, residual=None, eps=1e-6, prenorm=False):
    """``RMSNorm.forward`` semantics (``fla/modules/rmsnorm.py:491-512``): returns ``y`` or ``(y, x + residual)``."""
    _lib.require_cuda(x, weight)
    N = x.shape[-1]
    if not x.is_contiguous() or (residual is not None and not residual.is_contiguous()):
        raise ValueError("x and residual must be contiguous")
    y = torch.empty_like(x)
    res_out = torch.empty_like(x) if (prenorm and residual is not None) else None
    st = _lib.lib().vig_add_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(res_out),
                                        x.numel() // N, N, float(eps), _lib.dtype_code(x), _lib.stream_ptr())
    _lib.check(st, "vig_add_rmsnorm_fwd")
    if prenorm:
        return y, (res_out if residual is not None else x)
    return y


def layernorm_act(x, weight, bias, eps=1e-5, act_swish=False, pre_bias=None, post_add=None):
    """LayerNorm over the last (contiguous) dimension with affine parameters and optional swish
    (``LayerNorm2d`` of ``classification/models/vig.py:619-624`` on channels-last data).  ``pre_bias`` is an
    optional per-channel vector added to ``x`` first (the bias of the convolution that produced ``x``);
    ``post_add`` an optional ``[P, N]`` tensor added to row ``r`` as ``post_add[r % P]`` (the position embedding)."""
    _lib.require_cuda(x, weight, bias)
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    N = x.shape[-1]
    y = torch.empty_like(x)
    if post_add is not None:
        pa = post_add.reshape(-1, N).to(x.dtype).contiguous()
        st = _lib.lib().vig_layernorm_act_add_fwd(_lib.ptr(x), _lib.ptr(pre_bias), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(pa), pa.shape[0],
                                                  _lib.ptr(y), x.numel() // N, N, float(eps), int(bool(act_swish)), _lib.dtype_code(x),
                                                  _lib.stream_ptr())
        _lib.check(st, "vig_layernorm_act_add_fwd")
        return y
    st = _lib.lib().vig_layernorm_act_fwd(_lib.ptr(x), _lib.ptr(pre_bias), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), x.numel() // N, N,
                                          float(eps), int(bool(act_swish)), _lib.dtype_code(x), _lib.stream_ptr())
    _lib.check(st, "vig_layernorm_act_fwd")
    return y


def linear_add_rmsnorm_supported(x, w):
    """True when ``linear_add_rmsnorm`` can run on these operands (16-bit CUDA tensors, K % 64 == 0, N in {64, 128, 192, 256, 384})."""
    if not (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype and x.stride(-1) == 1):
        return False
    N, K = w.shape
    M = x.numel() // K
    return bool(_lib.lib().vig_linear_add_rmsnorm_supported(M, K, N, _lib.dtype_code(x)))


def linear_add_rmsnorm(x, w, residual, norm_weight, eps=1e-6):
    """``r = x @ w.T + residual`` (``residual`` may be None), ``h = RMSNorm(r) * norm_weight`` in one tensor-core kernel
    (see ``vig_linear_add_rmsnorm_fwd``).  Returns ``(h, r)``; x: [..., K], w: [N, K], residual: [..., N]."""
    _lib.require_cuda(x, w)
    N, K = w.shape
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    res = residual.reshape(M, N).contiguous() if residual is not None else None
    out_r = torch.empty(M, N, dtype=x.dtype, device=x.device)
    out_h = torch.empty(M, N, dtype=x.dtype, device=x.device)
    st = _lib.lib().vig_linear_add_rmsnorm_fwd(_lib.ptr(x2), x2.stride(0), _lib.ptr(w.contiguous()), _lib.ptr(res), _lib.ptr(norm_weight),
                                               _lib.ptr(out_r), _lib.ptr(out_h), M, K, N, float(eps), _lib.dtype_code(x), None,
                                               _lib.stream_ptr())
    _lib.check(st, "vig_linear_add_rmsnorm_fwd")
    return out_h.view(*lead, N), out_r.view(*lead, N)


def stem_unfold(x, s):
    """Space-to-depth with the first stem convolution's padding: ``[B,Cin,H,W] -> [B, H/s+1, W/s+1, s*s*Cin]``
    (see ``vig_stem_unfold_fwd``)."""
    _lib.require_cuda(x)
    B, Cin, H, W = x.shape
    x = x.contiguous()
    cells = torch.empty(B, H // s + 1, W // s + 1, s * s * Cin, dtype=x.dtype, device=x.device)
    st = _lib.lib().vig_stem_unfold_fwd(_lib.ptr(x), _lib.ptr(cells), B, Cin, H, W, s, _lib.dtype_code(x), _lib.stream_ptr())
    _lib.check(st, "vig_stem_unfold_fwd")
    return cells


def swiglu(gate, y):
    """``fla/modules/activations.py:109-113``: ``gate * sigmoid(gate) * y``; inputs may be the two halves of one projection."""
    _lib.require_cuda(gate, y)
    I = gate.shape[-1]
    g2, y2 = gate.reshape(-1, I) if gate.is_contiguous() else gate.flatten(0, -2), y.reshape(-1, I) if y.is_contiguous() else y.flatten(0, -2)
    if g2.stride(1) != 1 or y2.stride(1) != 1 or g2.stride(0) != y2.stride(0):
        raise ValueError("gate and y must be row-major with equal row strides")
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    st = _lib.lib().vig_swiglu_fwd(_lib.ptr(g2), _lib.ptr(y2), _lib.ptr(out), g2.shape[0], I, g2.stride(0), I,
                                   _lib.dtype_code(gate), _lib.stream_ptr())
    _lib.check(st, "vig_swiglu_fwd")
    return out


def linear_swiglu_supported(x, weight, preferred=False):
    """True when ``linear_swiglu`` has a fused kernel for this input (bf16 / fp16, K % 64 == 0, K <= 384, I % 64 == 0);
    with ``preferred`` also that it beats the library GEMM followed by the SwiGLU kernel (K <= 192)."""
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or weight.dtype != x.dtype:
        return False
    K, I = x.shape[-1], weight.shape[0] // 2
    L_ = _lib.lib()
    fn = L_.vig_linear_swiglu_preferred if preferred else L_.vig_linear_swiglu_supported
    return weight.is_contiguous() and bool(fn(x.numel() // K, K, I, _lib.dtype_code(x)))


def linear_swiglu(x, weight):
    """``swiglu(*F.linear(x, weight).chunk(2, -1))`` in one tensor-core kernel (``GLAMLP.forward``, ``vig.py:494-497``):
    ``weight`` is the ``[2I, K]`` gate projection, the result is ``[..., I]``."""
    _lib.require_cuda(x, weight)
    K, I = x.shape[-1], weight.shape[0] // 2
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    out = torch.empty(*x.shape[:-1], I, dtype=x.dtype, device=x.device)
    st = _lib.lib().vig_linear_swiglu_fwd(_lib.ptr(x2), x2.stride(0), _lib.ptr(weight), _lib.ptr(out), I, x2.shape[0], K, I,
                                          _lib.dtype_code(x), None, _lib.stream_ptr())
    _lib.check(st, "vig_linear_swiglu_fwd")
    return out


def swiglu_linear(x, y, weight, bias):
    """``fla/modules/activations.py:150-174``: ``F.linear(swiglu(x, y), weight, bias)``."""
    return torch.nn.functional.linear(swiglu(x, y), weight, bias)
