"""Gradients of the bi-GLA operator (vig_bigla_bwd through torch.autograd) against autograd through the CPU oracle
(fp64 restatement of the naive recurrence, fla/ops/gla/naive.py:13-58)."""
import pytest
import torch

import oracle
from conftest import rel_err

pytestmark = pytest.mark.gpu


def _reference_grads(q, k, v, gf, gb, d_out, out_scale, dir_mask):
    """Autograd through the naive recurrence in fp64 (differentiable torch ops, CPU)."""
    q, k, v, gf, gb = (t.detach().double().requires_grad_() for t in (q, k, v, gf, gb))
    B, H, L, dk = q.shape
    c = dk ** -0.5 * out_scale

    def scan(g, reverse):
        h = torch.zeros(B, H, dk, v.shape[-1], dtype=torch.float64)
        o = [None] * L
        for i in (range(L - 1, -1, -1) if reverse else range(L)):
            h = h * g[:, :, i].exp()[..., None] + k[:, :, i, :, None] * v[:, :, i, None, :]
            o[i] = c * (q[:, :, i, :, None] * h).sum(-2)
        return torch.stack(o, 2)
    o = 0
    if dir_mask & 1:
        o = o + scan(gf, False)
    if dir_mask & 2:
        o = o + scan(gb, True)
    o.backward(d_out.double())
    zero = lambda t: t.grad if t.grad is not None else torch.zeros_like(t)
    return o.detach(), [zero(t) for t in (q, k, v, gf, gb)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,L,dk,dv,dir_mask", [(2, 2, 150, 32, 64, 3), (1, 3, 196, 64, 64, 3), (1, 2, 65, 64, 64, 1),
                                                   (1, 1, 300, 32, 64, 2), (1, 2, 40, 16, 32, 3), (1, 1, 130, 64, 128, 3)])
def test_gradients_match_autograd_through_the_oracle(dtype, B, H, L, dk, dv, dir_mask):
    import vig_b200
    q, k, v, gf, gb = [t.to(dtype) for t in oracle.make_bigla_inputs(B, H, L, dk, dv, seed=L + dk)]
    d_out = torch.randn(B, H, L, dv, generator=torch.Generator().manual_seed(1)).to(dtype)
    _, ref = _reference_grads(q.float(), k.float(), v.float(), gf.float(), gb.float(), d_out.float(), 0.5, dir_mask)
    dev = [t.cuda().requires_grad_() for t in (q, k, v, gf, gb)]
    o = vig_b200.bi_gla(*dev, out_scale=0.5, dir_mask=dir_mask)
    o.backward(d_out.cuda())
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    names = ["dq", "dk", "dv", "dg_fwd", "dg_bwd"]
    errs = {}
    for name, t, r, active in zip(names, dev, ref, [True, True, True, dir_mask & 1, dir_mask & 2]):
        if not active:
            continue
        assert t.grad is not None, name
        errs[name] = rel_err(t.grad.float(), r)
    print(f"backward {dtype} B{B} H{H} L{L} dk{dk} dv{dv}: " + " ".join(f"{n} {e:.2e}" for n, e in errs.items()))
    assert all(e < tol for e in errs.values()), errs


def test_gradients_through_raw_gate_logits_and_reference_entry_point():
    """fused_chunk_gla (one direction, chunk_fuse.py:554-572) is differentiable; raw logits go through logsigmoid / 16."""
    import vig_b200
    B, H, L, dk, dv = 1, 2, 100, 32, 64
    q, k, v, _, _ = oracle.make_bigla_inputs(B, H, L, dk, dv, seed=7)
    x = 3 * torch.randn(B, H, L, dk, generator=torch.Generator().manual_seed(2))
    d_out = torch.randn(B, H, L, dv, generator=torch.Generator().manual_seed(3))
    # reference: autograd through the oracle with g = logsigmoid(x) / 16
    xr = x.double().requires_grad_()
    g = torch.nn.functional.logsigmoid(xr) / 16
    qd, kd, vd = (t.double().requires_grad_() for t in (q, k, v))
    h = torch.zeros(B, H, dk, dv, dtype=torch.float64)
    outs = []
    for i in range(L):
        h = h * g[:, :, i].exp()[..., None] + kd[:, :, i, :, None] * vd[:, :, i, None, :]
        outs.append(dk ** -0.5 * (qd[:, :, i, :, None] * h).sum(-2))
    torch.stack(outs, 2).backward(d_out.double())
    dev = [t.cuda().requires_grad_() for t in (q, k, v, x)]
    o = vig_b200.bi_gla(dev[0], dev[1], dev[2], dev[3], None, dir_mask=1, gate_logit_normalizer=16.0)
    o.backward(d_out.cuda())
    for t, r in zip(dev, (qd, kd, vd, xr)):
        assert rel_err(t.grad, r.grad) < 1e-4
    # the reference's name for the causal scan
    dev2 = [t.cuda().requires_grad_() for t in (q, k, v, (torch.nn.functional.logsigmoid(x) / 16))]
    o2, _ = vig_b200.fused_chunk_gla(*dev2)
    o2.backward(d_out.cuda())
    assert rel_err(dev2[0].grad, qd.grad) < 1e-4 and rel_err(dev2[2].grad, vd.grad) < 1e-4


def test_clamped_gates_pass_gradient_like_torch_clamp_min():
    """bf16 gates with a clamp bound that bf16 cannot represent: the gradient mask comes from the unrounded fp32 gate
    with >=, the rule of torch.clamp_min (classification/models/vig.py:440-441)."""
    import vig_b200
    B, H, L, dk, dv = 1, 2, 96, 32, 64
    q, k, v, _, _ = oracle.make_bigla_inputs(B, H, L, dk, dv, seed=9)
    x = (4 * torch.randn(B, H, L, dk, generator=torch.Generator().manual_seed(5))).bfloat16()
    d_out = torch.randn(B, H, L, dv, generator=torch.Generator().manual_seed(6))
    clamp = -0.3 / 16
    xr = x.double().requires_grad_()
    g = torch.clamp_min(torch.nn.functional.logsigmoid(xr) / 16, clamp)
    qd, kd, vd = (t.bfloat16().double().requires_grad_() for t in (q, k, v))
    h = torch.zeros(B, H, dk, dv, dtype=torch.float64)
    outs = []
    for i in range(L):
        h = h * g[:, :, i].exp()[..., None] + kd[:, :, i, :, None] * vd[:, :, i, None, :]
        outs.append(dk ** -0.5 * (qd[:, :, i, :, None] * h).sum(-2))
    torch.stack(outs, 2).backward(d_out.double())
    dev = [t.cuda().bfloat16().requires_grad_() for t in (q, k, v)] + [x.cuda().requires_grad_()]
    o = vig_b200.bi_gla(dev[0], dev[1], dev[2], dev[3], None, dir_mask=1, gate_logit_normalizer=16.0, clamp_min=clamp)
    o.backward(d_out.cuda().bfloat16())
    clamped = (torch.nn.functional.logsigmoid(x.float()) / 16) < clamp
    assert clamped.any() and not clamped.all()
    assert float(dev[3].grad.float().cpu()[clamped].abs().max()) == 0.0        # no gradient through clamped entries
    err = rel_err(dev[3].grad.float(), xr.grad)
    print(f"gate-logit gradient with clamp, bf16: {err:.2e}")
    assert err < 2e-2
