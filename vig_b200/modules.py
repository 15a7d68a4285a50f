"""Host-side mirror of the reference's ViG block: same class names, parameter names and forward
arguments as ``classification/models/vig.py`` (``GatedLinearAttention`` :241-464, ``GLAMLP`` :469-497,
``GLABlock`` :530-618) and ``fla/modules/rmsnorm.py:491-512`` (``RMSNorm``), so a reference state dict
loads unchanged.  Inference only: the forward is the reference's ``eval()`` branch, with the scan, the
depthwise conv, the gating injection, the norms and SwiGLU running as the library's CUDA kernels and the
dense projections as cuBLAS GEMMs (``F.linear``).
"""
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


class RMSNorm(nn.Module):
    """``RMSNorm(hidden_size, eps)(x, residual=None, prenorm=False)``; weight only, no bias."""

    def __init__(self, hidden_size, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.register_parameter("bias", None)

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return ops.add_rmsnorm(x, self.weight, residual=residual, eps=self.eps, prenorm=prenorm)


class GatedLinearAttention(nn.Module):
    def __init__(self, d_model=1024, expand_v=2.0, expand_k=1.0, num_heads=4, gate_fn="swish", layernorm_eps=1e-5,
                 gate_logit_normalizer=16, gate_low_rank_dim=16, mode="fused_chunk", clamp_min=None, use_out_act=False,
                 use_act_in_conv=True, use_bias_in_dwconv=False, **kwargs):
        super().__init__()
        if gate_fn not in ("swish", "silu"):
            raise NotImplementedError("only the swish gate function of the shipped configurations is implemented")
        self.d_model, self.mode, self.clamp_min = d_model, mode, clamp_min
        self.value_dim, self.key_dim = int(d_model * expand_v), int(d_model * expand_k)
        assert self.key_dim % num_heads == 0, f"key dim must be divisible by num_heads of {num_heads}"
        assert self.value_dim % num_heads == 0, f"value dim must be divisible by num_heads of {num_heads}"
        if self.value_dim != d_model:
            raise ValueError("the locality injection adds the conv output to the scan output: expand_v must be 1")
        self.num_heads = num_heads
        self.head_qk_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.use_out_act, self.use_act_in_conv = use_out_act, use_act_in_conv
        self.gate_logit_normalizer = gate_logit_normalizer
        self.in_proj = nn.Sequential(
            nn.Conv2d(d_model, d_model, kernel_size=3, padding=1, groups=d_model, bias=use_bias_in_dwconv),
            nn.SiLU() if use_act_in_conv else nn.Identity())
        self.qkv_proj = nn.Linear(d_model, 2 * self.key_dim + self.value_dim, bias=False)
        self.gk_proj = nn.Sequential(nn.Linear(d_model, gate_low_rank_dim, bias=False),
                                     nn.Linear(gate_low_rank_dim, self.key_dim * 2, bias=True))
        self.o_proj = nn.Linear(self.value_dim, d_model, bias=False)
        self.g_norm = RMSNorm(self.head_v_dim, eps=layernorm_eps)
        self.l_norm = RMSNorm(self.head_v_dim, eps=layernorm_eps)
        self.g_proj = nn.Linear(d_model, self.value_dim, bias=True)
        self._packed = None
        # scale of the summed directions: the operator wrapper halves the sum (recurrent_fuse.py:442) and ViG's eval branch
        # halves it again (vig.py:443); GLA2D of the hierarchical model keeps the single halving (vig_h.py:577-578)
        self.out_scale = 0.25
        # inference-time weight folding of the gate bottleneck (16-bit runs only; fp32 keeps the reference's two steps)
        self.fold_gate_bottleneck = True
        self.own_in_proj_gemm = False

    def _pack(self):
        """Derived weight layouts, built once per dtype/device: the conv taps as [9, C] and one stacked
        matrix for the three projections that read the conv output (qkv, gate low-rank, output gate)."""
        w = self.in_proj[0].weight
        key = (w.dtype, w.device, w._version, self.qkv_proj.weight._version)
        if self._packed is None or self._packed[0] != key:
            C = self.d_model
            taps = w.detach().reshape(C, 9).t().contiguous()
            stacked = torch.cat([self.qkv_proj.weight, self.g_proj.weight, self.gk_proj[0].weight], dim=0).detach().contiguous()
            bias = torch.cat([torch.zeros(self.qkv_proj.out_features, dtype=w.dtype, device=w.device), self.g_proj.bias.detach(),
                              torch.zeros(self.gk_proj[0].out_features, dtype=w.dtype, device=w.device)])
            # the rank-16 gate bottleneck folded into one [2*key_dim, d_model] matrix (product in fp32, rounded once):
            # a K = d_model GEMM of a friendly width replaces the 16 odd columns of the stacked projection plus a K = 16 GEMM
            folded = (self.gk_proj[1].weight.detach().float() @ self.gk_proj[0].weight.detach().float()).to(w.dtype).contiguous()
            # with the bottleneck folded, its rows join the stacked projection: one GEMM reads the conv output once
            n_main = self.qkv_proj.out_features + self.g_proj.out_features
            gk_bias = self.gk_proj[1].bias
            gk_bias = torch.zeros(folded.shape[0], dtype=w.dtype, device=w.device) if gk_bias is None else gk_bias.detach()
            merged = (torch.cat([stacked[:n_main], folded], dim=0).contiguous(), torch.cat([bias[:n_main], gk_bias]))
            self._packed = (key, taps, stacked, bias, merged)
        return self._packed[1:]

    def forward(self, x, lower_bound=0, **kwargs):
        if self.training:
            raise NotImplementedError("vig_b200 implements the inference (eval) forward only")
        B, L, C = x.shape
        hw = kwargs["patch_resolution"]
        H, dk, dv, kd, vd = self.num_heads, self.head_qk_dim, self.head_v_dim, self.key_dim, self.value_dim
        taps, w_in, b_in, merged = self._pack()
        # ``local_fn`` / ``scan_fn`` let a caller substitute the two steps that look beyond the tokens at hand (the
        # 3x3 neighbourhood and the scan) -- the sequence-parallel driver supplies halo and boundary-state versions
        local_fn, scan_fn = kwargs.get("local_fn"), kwargs.get("scan_fn")
        if local_fn is None:
            xs = ops.dwconv3x3(x, taps, self.in_proj[0].bias, hw, self.use_act_in_conv)
        else:
            xs = local_fn(x, taps, self.in_proj[0].bias, hw, self.use_act_in_conv)
        fold = self.fold_gate_bottleneck and x.dtype != torch.float32
        n_main = 2 * kd + 2 * vd
        # one GEMM for [q | k | v | output-gate logits | low-rank gate features] (folded: | raw gate logits)
        w_z, b_z = (merged[0], merged[1]) if fold else (w_in, b_in)
        # the vendor GEMM by default: the library's own kernel for this product (``ops.linear_bias``) measures 171 us against
        # 160-165 us at the benchmark's shape; ``own_in_proj_gemm`` switches it in where it is supported
        use_own = self.own_in_proj_gemm and ops.linear_bias_supported(xs, w_z)
        z = ops.linear_bias(xs, w_z, b_z) if use_own else F.linear(xs, w_z, b_z)
        heads = lambda t, d: t.unflatten(-1, (H, d)).permute(0, 2, 1, 3)           # [B,H,L,d] views, no copy
        q, k, v = heads(z[..., :kd], dk), heads(z[..., kd:2 * kd], dk), heads(z[..., 2 * kd:2 * kd + vd], dv)
        gate_logits = z[..., 2 * kd + vd:2 * kd + 2 * vd]
        # raw gate logits [B,L,2*kd]: bias and the strided low-rank slice go straight into one GEMM call
        if fold:
            gk = z[..., n_main:]
        else:
            gk = torch.addmm(self.gk_proj[1].bias, z.view(B * L, -1)[:, 2 * kd + 2 * vd:], self.gk_proj[1].weight.t()).view(B, L, 2 * kd)
        g_fwd, g_bwd = heads(gk[..., :kd], dk), heads(gk[..., kd:], dk)
        o = torch.empty(B, L, H, dv, dtype=x.dtype, device=x.device).permute(0, 2, 1, 3)
        # reference: (o_f + o_b) / 2 in the operator wrapper, / 2 again in the eval branch (vig.py:443)
        scan_kw = dict(out_scale=self.out_scale, out=o, gate_logit_normalizer=float(self.gate_logit_normalizer), clamp_min=self.clamp_min)
        if scan_fn is None:
            ops.bi_gla(q, k, v, g_fwd, g_bwd, **scan_kw)
        else:
            scan_fn(q, k, v, g_fwd, g_bwd, **scan_kw)
        y = ops.gate_inject(o, xs, gate_logits, self.g_norm.weight, self.l_norm.weight, self.g_norm.eps, self.use_out_act)
        if kwargs.get("skip_o_proj"):                         # the caller fuses the output projection with the next norm
            return y
        return self.o_proj(y)


class GLAMLP(nn.Module):
    def __init__(self, hidden_size, hidden_ratio: Optional[int] = None, intermediate_size: Optional[int] = None,
                 hidden_act="swish"):
        super().__init__()
        if hidden_ratio is None:
            hidden_ratio = 4
        if intermediate_size is None:
            intermediate_size = int(hidden_size * hidden_ratio * 2 / 3)
            intermediate_size = 256 * ((intermediate_size + 256 - 1) // 256)
        self.hidden_size, self.hidden_ratio, self.intermediate_size = hidden_size, hidden_ratio, intermediate_size
        self.gate_proj = nn.Linear(hidden_size, intermediate_size * 2, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        if ops.linear_swiglu_supported(x, self.gate_proj.weight, preferred=True):
            # gate projection and SwiGLU in one tensor-core kernel: the [.., 2I] intermediate never reaches HBM
            return F.linear(ops.linear_swiglu(x, self.gate_proj.weight), self.down_proj.weight, self.down_proj.bias)
        y = self.gate_proj(x)
        gate, y = y.chunk(2, -1)
        return ops.swiglu_linear(gate, y, self.down_proj.weight, self.down_proj.bias)


class GLABlock(nn.Module):
    """``config`` needs: hidden_size, num_attention_heads, expand_k, expand_v, rms_norm_eps, use_out_act,
    use_act_in_conv, use_bias_in_dwconv, clamp_min, attn_mode, intermediate_size (or None)."""

    def __init__(self, config, layer_idx=0, drop_path=0.0, is_attn=False):
        super().__init__()
        g = lambda n, d=None: getattr(config, n, d)
        self.hidden_size = config.hidden_size
        self.attn_norm = RMSNorm(config.hidden_size, eps=g("rms_norm_eps", 1e-6))
        self.attn = GatedLinearAttention(
            d_model=config.hidden_size, expand_k=g("expand_k", 0.5), expand_v=g("expand_v", 1.0),
            num_heads=config.num_attention_heads, gate_fn=g("hidden_act", "swish"), layernorm_eps=g("rms_norm_eps", 1e-6),
            mode=g("attn_mode", "fused_chunk"), clamp_min=g("clamp_min"), use_out_act=g("use_out_act", False),
            use_act_in_conv=g("use_act_in_conv", True), use_bias_in_dwconv=g("use_bias_in_dwconv", False))
        self.mlp_norm = RMSNorm(config.hidden_size, eps=g("rms_norm_eps", 1e-6))
        self.mlp = GLAMLP(config.hidden_size, intermediate_size=g("intermediate_size"), hidden_act=g("hidden_act", "swish"))

    def forward(self, hidden_states, lower_bound=None, **kwargs):
        """Reference signature: returns a 1-tuple with ``residual + mlp(norm(residual))``."""
        h, residual = self.forward_deferred(hidden_states, None, **kwargs)
        return (residual + h,)

    def fused_epilogues_supported(self, x):
        """True when both projections of the block can run with the residual add and the following RMSNorm as their
        epilogue (``ops.linear_add_rmsnorm``: 16-bit CUDA tensors, hidden size <= 384, no projection bias)."""
        return (self.attn.o_proj.bias is None and self.mlp.down_proj.bias is None and x.shape[-1] <= 192 and
                ops.linear_add_rmsnorm_supported(x, self.attn.o_proj.weight) and
                x.shape[-1] == self.mlp.down_proj.weight.shape[0] and self.mlp.down_proj.weight.shape[1] % 64 == 0)

    def forward_prenormed(self, h, residual, next_norm, **kwargs):
        """The block with its norms moved into the projections' epilogues: takes ``h = attn_norm(residual stream)`` and
        the residual stream, returns ``(next_norm(new residual stream), new residual stream)`` -- ``next_norm`` is the
        next block's ``attn_norm`` or the model's final norm.  Same arithmetic as ``forward_deferred`` chained."""
        y = self.attn(h, skip_o_proj=True, **kwargs)
        h2, residual = ops.linear_add_rmsnorm(y, self.attn.o_proj.weight, residual, self.mlp_norm.weight, self.mlp_norm.eps)
        m = self.mlp
        if ops.linear_swiglu_supported(h2, m.gate_proj.weight, preferred=True):
            z = ops.linear_swiglu(h2, m.gate_proj.weight)
        else:
            gate, yy = m.gate_proj(h2).chunk(2, -1)
            z = ops.swiglu(gate, yy)
        return ops.linear_add_rmsnorm(z, m.down_proj.weight, residual, next_norm.weight, next_norm.eps)

    def forward_deferred(self, hidden_states, residual, **kwargs):
        """Same block, but the trailing residual add is left to the caller's next norm: takes the pair
        (branch output, residual stream) of the previous block and returns this block's pair, so every
        add is fused into an RMSNorm kernel."""
        if residual is None:
            residual = hidden_states
            h = self.attn_norm(hidden_states)
        else:
            h, residual = self.attn_norm(hidden_states, residual, True)
        h = self.attn(h, **kwargs)
        h, residual = self.mlp_norm(h, residual, True)
        return self.mlp(h), residual
