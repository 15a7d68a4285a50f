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
# (dk, dv) pairs the backward kernels are compiled for (vig_bigla_bwd)
BWD_HEAD_DIMS = {(16, 32), (32, 32), (32, 64), (64, 64), (64, 128)}
_ws_cache = {}
_status_words = {}


class StatusWord:
    """The device-side error word of one GPU.  Every scan and fused-GEMM launch of this module ORs its error bits into
    it (bit 0: a bounded wait inside a kernel ran out, bit 1: a chunk's cumulative log-gate left the range the
    tensor-core factorisation covers, so that chunk's numbers are wrong).  ``check()`` reads it with a synchronising
    copy; ``snapshot()`` / ``poll()`` read it without stalling the stream (an asynchronous copy to pinned memory that
    the next ``poll()`` looks at once it has landed)."""
    BITS = {1: "a bounded wait inside a kernel ran out", 2: "a cumulative log-gate left the tensor-core range (use impl=IMPL_SIMT)"}

    def __init__(self, device):
        self.tensor = torch.zeros(1, dtype=torch.int32, device=device)
        self._host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._event = None

    def _raise(self, value):
        self.tensor.zero_()
        what = "; ".join(msg for bit, msg in self.BITS.items() if value & bit) or "unknown bits"
        raise RuntimeError(f"vig_b200 kernels reported status {value}: {what}")

    def check(self):
        """Blocking read; raises (and clears the word) when a kernel has reported an error."""
        self._event = None
        value = int(self.tensor.item())
        if value:
            self._raise(value)

    def snapshot(self):
        """Queue an asynchronous read on the current stream (skipped while the stream is being captured)."""
        if torch.cuda.is_current_stream_capturing():
            return
        self.poll()
        if self._event is None:
            self._host.copy_(self.tensor, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()

    def poll(self):
        """Look at the last snapshot if its copy has finished; raises like ``check``.  A no-op while the stream is being
        captured into a CUDA graph (an event query is not permitted there and would invalidate the capture)."""
        if torch.cuda.is_current_stream_capturing():
            return
        if self._event is not None and self._event.query():
            self._event = None
            value = int(self._host[0])
            if value:
                self._raise(value)


def status_word(device=None):
    """The ``StatusWord`` of ``device`` (default: the current CUDA device), created on first use."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sw = _status_words.get(device)
    if sw is None:
        sw = _status_words[device] = StatusWord(device)
    return sw


def check_status(device=None):
    """Raise if any kernel launched through this module on ``device`` has reported an error since the last check."""
    status_word(device).check()


def _status_ptr(status, device):
    return _lib.ptr(status_word(device).tensor if status is None else status)


def _same_device(*tensors):
    """All given tensors (``None`` entries skipped) must be CUDA tensors on one device; returns it."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("vig_b200 kernels need CUDA tensors; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors live on different devices ({dev} and {t.device})")
    return dev


def _check_scan_shapes(q, k, v, g_fwd, g_bwd, out=None):
    """Shapes and dtypes the scan kernels index with: q and the gates like k, out like v."""
    if k.dim() != 4 or v.dim() != 4 or v.shape[:3] != k.shape[:3]:
        raise ValueError(f"k and v must be [B,H,L,dk] / [B,H,L,dv]; got {tuple(k.shape)} and {tuple(v.shape)}")
    for name, t in (("q", q), ("g_fwd", g_fwd), ("g_bwd", g_bwd)):
        if t is not None and t.shape != k.shape:
            raise ValueError(f"{name} must have k's shape {tuple(k.shape)}; got {tuple(t.shape)}")
    for name, t in (("q", q), ("v", v), ("g_fwd", g_fwd), ("g_bwd", g_bwd), ("out", out)):
        if t is not None and t.dtype != k.dtype:
            raise TypeError(f"{name} has dtype {t.dtype}, k has {k.dtype}: q, k, v, the gates and out must share one dtype")
    if out is not None and out.shape != v.shape:
        raise ValueError(f"out must have v's shape {tuple(v.shape)}; got {tuple(out.shape)}")


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

    ``status``: int32 CUDA tensor of one element that the kernels OR error bits into (bit 0: a bounded wait ran
    out, bit 1: a chunk's cumulative gate left the range of the tensor-core factorisation); default: the device's
    ``status_word()``, which ``check_status()`` reads.
    Returns ``o`` or ``(o, extras)`` where ``extras`` holds ``final_fwd/final_bwd`` ([B,H,dk,dv] fp32) and
    ``logdecay_fwd/logdecay_bwd`` ([B,H,dk] fp32) when requested.
    """
    dev = _same_device(q, k, v, g_fwd, g_bwd, out, init_state_fwd, init_state_bwd, status)
    _check_scan_shapes(q if want_output else None, k, v, g_fwd, g_bwd, out)
    if want_output and q is None:
        raise ValueError("q is required unless want_output=False")
    B, H, L, dk = k.shape
    dv = v.shape[-1]
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g_fwd, g_bwd)):
        if (init_state_fwd is not None or init_state_bwd is not None or output_final_state or output_logdecay
                or out is not None or not want_output):
            raise NotImplementedError("the differentiable form takes no states and allocates its own output")
        if (dk, dv) not in BWD_HEAD_DIMS:
            raise NotImplementedError(f"the backward kernels cover (dk, dv) in {sorted(BWD_HEAD_DIMS)}; got ({dk}, {dv})")
        return _BiGLAFunction.apply(q, k, v, g_fwd, g_bwd, float(scale if scale is not None else -1), float(out_scale),
                                    float(gate_logit_normalizer), clamp_min, dir_mask, impl)
    code = _lib.dtype_code(k)
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
    with torch.cuda.device(dev):
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
            dir_mask, impl, _lib.ptr(ws), ws.numel() if ws is not None else 0, _status_ptr(status, dev), _lib.stream_ptr())
    _lib.check(st, "vig_bigla_fwd")
    if extras:
        return out, extras
    return out


def bi_gla_backward(q, k, v, g_fwd, g_bwd, d_out, scale=-1, out_scale=1.0, dir_mask=3):
    """Gradients of ``bi_gla`` with log-space gates: ``(dq, dk, dv, dg_fwd, dg_bwd)`` (``None`` for a direction that
    is masked out).  The kernels deliver ``e = dq*q - dk*k`` per direction; the gate gradients are its cumulative
    sums over the tokens (``fla/ops/gla/chunk_fuse.py:506-516`` does the same in PyTorch)."""
    dev = _same_device(q, k, v, g_fwd, g_bwd, d_out)
    _check_scan_shapes(q, k, v, g_fwd, g_bwd, d_out)
    B, H, L, dk = k.shape
    dv = v.shape[-1]
    if (dk, dv) not in BWD_HEAD_DIMS:
        raise NotImplementedError(f"the backward kernels cover (dk, dv) in {sorted(BWD_HEAD_DIMS)}; got ({dk}, {dv})")
    dq, dk_, dv_ = (torch.empty(B, H, L, d, dtype=k.dtype, device=dev) for d in (dk, dk, dv))
    e_f = torch.empty(B, H, L, dk, dtype=torch.float32, device=dev) if dir_mask & 1 else None
    e_b = torch.empty(B, H, L, dk, dtype=torch.float32, device=dev) if dir_mask & 2 else None
    L_ = _lib.lib()
    s3 = lambda t: None if t is None else _lib.strides3(t)
    with torch.cuda.device(dev):
        nbytes = L_.vig_bigla_bwd_workspace_bytes(B, H, L, dk, dv)
        ws = _workspace(nbytes, dev)
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
            # gradient passes where the unclamped fp32 gate is at or above the bound (torch.clamp_min's rule)
            keep = None
            if clamp_min is not None:
                keep = g >= clamp_min
                g = torch.clamp_min(g, clamp_min)
            return g.to(x.dtype), keep
        gf, keep_f = to_log(g_fwd)
        gb, keep_b = to_log(g_bwd)
        with torch.no_grad():
            o = bi_gla(q, k, v, gf, gb, scale=scale, out_scale=out_scale, dir_mask=dir_mask, impl=impl)
        ctx.save_for_backward(q, k, v, g_fwd, g_bwd, gf, gb, keep_f, keep_b)
        ctx.cfg = (scale, out_scale, gate_norm, clamp_min, dir_mask)
        return o

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, x_f, x_b, gf, gb, keep_f, keep_b = ctx.saved_tensors
        scale, out_scale, gate_norm, clamp_min, dir_mask = ctx.cfg
        dq, dk, dv, dg_f, dg_b = bi_gla_backward(q, k, v, gf, gb, d_out.contiguous(), scale, out_scale, dir_mask)

        def through_gate(dg, x, keep):
            if dg is None or x is None:
                return None
            if keep is not None:
                dg = dg * keep
            if gate_norm > 0:                                       # d logsigmoid(x) / dx = sigmoid(-x)
                dg = dg * torch.sigmoid(-x.float()) / gate_norm
            return dg.to(x.dtype)
        return dq, dk, dv, through_gate(dg_f, x_f, keep_f), through_gate(dg_b, x_b, keep_b), None, None, None, None, None, None


def bi_gla_noalloc(q, k, v, g_fwd, g_bwd, out, scale=-1, out_scale=1.0, gate_logit_normalizer=0.0, clamp_min=None,
                   impl=_lib.IMPL_AUTO, status=None):
    """``bi_gla`` through the entry point that allocates nothing: the caller supplies ``out`` and the scan's
    scratch is a fixed array inside the library (see ``vig_bigla_fwd_noalloc`` in the header for who needs
    this and for its size limit).  Calls on one device must not overlap on the GPU.  ``status``: as in ``bi_gla``;
    pass a tensor of your own if even the status word's one-time allocation is unwelcome."""
    dev = _same_device(q, k, v, g_fwd, g_bwd, out, status)
    if q is None or g_fwd is None or g_bwd is None or out is None:
        raise ValueError("q, both gate tensors and out are required")
    _check_scan_shapes(q, k, v, g_fwd, g_bwd, out)
    B, H, L, dk = k.shape
    dv = v.shape[-1]
    with torch.cuda.device(dev):
        st = _lib.lib().vig_bigla_fwd_noalloc(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g_fwd), _lib.ptr(g_bwd), _lib.ptr(out), B, H, L, dk, dv,
            _lib.dtype_code(k), _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(g_fwd), _lib.strides3(g_bwd),
            _lib.strides3(out), float(scale if scale is not None else -1), float(out_scale), float(gate_logit_normalizer),
            _NAN if clamp_min is None else float(clamp_min), impl, _status_ptr(status, dev), _lib.stream_ptr())
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
def dwconv3x3(x, weight_tap_major, bias, hw, act_silu, out=None, top=None, bottom=None):
    """Depthwise 3x3 (+SiLU) on ``[B, h*w, C]`` tokens; ``weight_tap_major`` is ``[9, C]``.  ``top`` / ``bottom``
    (``[B, w, C]``, 16-bit types): the image rows just above / below when ``x`` is a band of a taller image."""
    _lib.require_cuda(x, weight_tap_major, top, bottom)
    B, L, C = x.shape
    h, w = hw
    if h * w != L or not x.is_contiguous():
        raise ValueError("x must be contiguous [B, h*w, C]")
    y = torch.empty_like(x) if out is None else out
    if top is not None or bottom is not None:
        for t in (top, bottom):
            if t is not None and (t.shape != (B, w, C) or not t.is_contiguous() or t.dtype != x.dtype):
                raise ValueError("halo rows must be contiguous [B, w, C] tensors of x's dtype")
        st = _lib.lib().vig_dwconv3x3_halo_fwd(_lib.ptr(x), _lib.ptr(top), _lib.ptr(bottom), _lib.ptr(weight_tap_major),
                                               _lib.ptr(bias), _lib.ptr(y), B, h, w, C, int(bool(act_silu)),
                                               _lib.dtype_code(x), _lib.stream_ptr())
        _lib.check(st, "vig_dwconv3x3_halo_fwd")
        return y
    st = _lib.lib().vig_dwconv3x3_fwd(_lib.ptr(x), _lib.ptr(weight_tap_major), _lib.ptr(bias), _lib.ptr(y),
                                      B, h, w, C, int(bool(act_silu)), _lib.dtype_code(x), _status_ptr(None, x.device), _lib.stream_ptr())
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


def layernorm_act(x, weight, bias, eps=1e-5, act_swish=False, pre_bias=None, post_add=None, rms_weight=None, rms_eps=1e-6):
    """LayerNorm over the last (contiguous) dimension with affine parameters and optional swish
    (``LayerNorm2d`` of ``classification/models/vig.py:619-624`` on channels-last data).  ``pre_bias`` is an
    optional per-channel vector added to ``x`` first (the bias of the convolution that produced ``x``);
    ``post_add`` an optional ``[P, N]`` tensor added to row ``r`` as ``post_add[r % P]`` (the position embedding).
    With ``rms_weight`` the RMSNorm of the result comes out of the same pass: returns ``(y, RMSNorm(y) * rms_weight)``."""
    _lib.require_cuda(x, weight, bias)
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    N = x.shape[-1]
    y = torch.empty_like(x)
    if rms_weight is not None:
        _lib.require_cuda(rms_weight)
        if rms_weight.dtype != x.dtype or rms_weight.numel() != N:
            raise ValueError("rms_weight must be an [N] vector of x's dtype")
        pa = post_add.reshape(-1, N).to(x.dtype).contiguous() if post_add is not None else None
        h = torch.empty_like(x)
        st = _lib.lib().vig_layernorm_act_add_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(pre_bias), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(pa),
                                                          pa.shape[0] if pa is not None else 1, _lib.ptr(y), _lib.ptr(rms_weight.contiguous()),
                                                          float(rms_eps), _lib.ptr(h), x.numel() // N, N, float(eps), int(bool(act_swish)),
                                                          _lib.dtype_code(x), _lib.stream_ptr())
        _lib.check(st, "vig_layernorm_act_add_rmsnorm_fwd")
        return y, h
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
                                               _lib.ptr(out_r), _lib.ptr(out_h), M, K, N, float(eps), _lib.dtype_code(x),
                                               _status_ptr(None, x.device), _lib.stream_ptr())
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


def stem_fold(x):
    """Fold of a 16-bit image into cells of 8 x 8 pixels on 8-pixel boundaries: ``[B,3,H,W] -> [B, H/8, W/8, 192]`` with
    ``cells[b, cy, cx, (dy*3 + ic)*8 + dx] = x[b, ic, 8cy + dy, 8cx + dx]`` (see ``vig_stem_fold_fwd``)."""
    _lib.require_cuda(x)
    B, Cin, H, W = x.shape
    x = x.contiguous()
    cells = torch.empty(B, H // 8, W // 8, 64 * Cin, dtype=x.dtype, device=x.device)
    with torch.cuda.device_of(x):
        st = _lib.lib().vig_stem_fold_fwd(_lib.ptr(x), _lib.ptr(cells), B, Cin, H, W, _lib.dtype_code(x), _lib.stream_ptr())
    _lib.check(st, "vig_stem_fold_fwd")
    return cells


def stem_conv_ln_supported(cells, out_channels):
    """True when ``stem_conv_ln`` has a kernel for these cells (bf16 / fp16, cells of 192 values, 96 output channels)."""
    if not (cells.is_cuda and cells.dtype in (torch.bfloat16, torch.float16) and cells.dim() == 4 and cells.is_contiguous()):
        return False
    B, CH, CW, cell = cells.shape
    return bool(_lib.lib().vig_stem_conv_ln_supported(B, CH, CW, cell, int(out_channels), _lib.dtype_code(cells)))


def stem_conv_ln_supported_for_image(x, out_channels):
    """The same question asked of the image ``[B, 3, H, W]`` before it is folded (``stem_fold`` then ``stem_conv_ln``)."""
    if not (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.dim() == 4 and x.shape[1] == 3):
        return False
    B, _, H, W = x.shape
    if H % 8 or W % 8:
        return False
    return bool(_lib.lib().vig_stem_conv_ln_supported(B, H // 8, W // 8, 192, int(out_channels), _lib.dtype_code(x)))


def stem_conv_ln(cells, w2, conv_bias, ln_weight, ln_bias, eps=1e-5, act_swish=True):
    """The stem's first convolution on unfolded cells + bias + LayerNorm over channels (+ swish) in one tensor-core
    kernel (see ``vig_stem_conv_ln_fwd``).  cells: ``[B, CH, CW, 192]`` from ``stem_fold``, w2: ``[96, 512]``; returns
    ``[B, CH, CW, 96]``."""
    _lib.require_cuda(cells, w2, ln_weight, ln_bias)
    B, CH, CW, cell = cells.shape
    N = w2.shape[0]
    if w2.dtype != cells.dtype or tuple(w2.shape) != (N, 2 * cell + 128) or not w2.is_contiguous() or not cells.is_contiguous():
        raise ValueError("w2 must be a contiguous [N, 2*cell + 128] matrix of the cells' dtype, cells contiguous")
    for t in (conv_bias, ln_weight, ln_bias):
        if t is not None and (t.dtype != cells.dtype or t.numel() != N or t.device != cells.device):
            raise ValueError("conv_bias / ln_weight / ln_bias must be [N] vectors of the cells' dtype on the cells' device")
    y = torch.empty(B, CH, CW, N, dtype=cells.dtype, device=cells.device)
    with torch.cuda.device_of(cells):
        st = _lib.lib().vig_stem_conv_ln_fwd(_lib.ptr(cells), _lib.ptr(w2), _lib.ptr(conv_bias), _lib.ptr(ln_weight.contiguous()),
                                             _lib.ptr(ln_bias.contiguous()), _lib.ptr(y), B, CH, CW, cell, N, float(eps),
                                             int(bool(act_swish)), _lib.dtype_code(cells), _status_ptr(None, cells.device),
                                             _lib.stream_ptr())
    _lib.check(st, "vig_stem_conv_ln_fwd")
    return y


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
                                          _lib.dtype_code(x), _status_ptr(None, x.device), _lib.stream_ptr())
    _lib.check(st, "vig_linear_swiglu_fwd")
    return out


def linear_bias_supported(x, weight):
    """True when ``linear_bias`` has a kernel for this input (bf16 / fp16, K % 64 == 0, K <= 192, N % 8 == 0, at least 256
    rows per SM -- the stacked input projection of the block at widths up to 192 and large batches)."""
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or weight.dtype != x.dtype or not weight.is_contiguous():
        return False
    K, N = x.shape[-1], weight.shape[0]
    with torch.cuda.device(x.device):
        return bool(_lib.lib().vig_linear_bias_supported(x.numel() // K, K, N, _lib.dtype_code(x)))


def linear_bias(x, weight, bias=None):
    """``F.linear(x, weight, bias)`` as this library's tensor-core GEMM (the stacked ``qkv_proj`` / ``g_proj`` / ``gk_proj``
    of ``GatedLinearAttention``, ``vig.py:283-290``): x ``[..., K]``, weight ``[N, K]``, bias ``[N]`` or None."""
    _lib.require_cuda(x, weight, bias)
    K, N = x.shape[-1], weight.shape[0]
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if bias is not None and (bias.dtype != x.dtype or not bias.is_contiguous() or bias.shape != (N,)):
        raise ValueError("bias must be a contiguous [N] tensor of x's dtype")
    out = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.lib().vig_linear_bias_fwd(_lib.ptr(x2), x2.stride(0), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(out), N, x2.shape[0],
                                            K, N, _lib.dtype_code(x), _status_ptr(None, x.device), _lib.stream_ptr())
    _lib.check(st, "vig_linear_bias_fwd")
    return out


def swiglu_linear(x, y, weight, bias):
    """``fla/modules/activations.py:150-174``: ``F.linear(swiglu(x, y), weight, bias)``."""
    return torch.nn.functional.linear(swiglu(x, y), weight, bias)
