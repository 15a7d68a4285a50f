"""Parity of the CUDA bi-GLA operator (through the C ABI) with the CPU oracle and the reference's vectors.

Tolerances: fp32 <= 1e-4, bf16/fp16 <= 2e-2, both as max|a-b| / max|b| against the fp32 reference.
"""
import pytest
import torch

import oracle
from conftest import rel_err

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}
IMPLS = {"simt": 1, "auto": 0}


def _cuda(ts, dtype):
    return [t.to("cuda", dtype) for t in ts]


def _run(q, k, v, gf, gb, dtype, impl=0, **kw):
    import vig_b200
    qd, kd, vd, gfd, gbd = _cuda((q, k, v, gf, gb), dtype)
    out = vig_b200.bi_gla(qd, kd, vd, gfd, gbd, impl=impl, **kw)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("name", ["cfg1", "dk32", "L1", "L17", "L300"])
@pytest.mark.parametrize("impl", ["simt", "auto"])
def test_fp32_matches_reference_vectors(golden_bigla, name, impl):
    B, H, L, dk, dv, seed = (int(x) for x in golden_bigla[f"bigla_{name}_shape"])
    ins = oracle.make_bigla_inputs(B, H, L, dk, dv, seed)
    o = _run(*ins, torch.float32, IMPLS[impl])
    assert rel_err(o, golden_bigla[f"bigla_{name}_o"]) < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("impl", ["simt", "auto"])
@pytest.mark.parametrize("name", ["cfg1", "dk32", "L300"])
def test_half_precision_matches_fp32_reference(golden_bigla, name, dtype, impl):
    B, H, L, dk, dv, seed = (int(x) for x in golden_bigla[f"bigla_{name}_shape"])
    ins = oracle.make_bigla_inputs(B, H, L, dk, dv, seed)
    o = _run(*ins, dtype, IMPLS[impl])
    assert rel_err(o.float(), golden_bigla[f"bigla_{name}_o"]) < 2e-2


@pytest.mark.parametrize("L", [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 196, 208, 257, 513])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_lengths(L, dtype):
    ins = oracle.make_bigla_inputs(2, 3, L, 64, 64, seed=L)
    ref = oracle.naive_bi_gla(*[t.to(dtype).float() for t in ins])
    o = _run(*ins, dtype)
    assert rel_err(o.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("dk,dv", [(16, 32), (32, 64), (64, 64), (128, 128), (64, 128), (128, 64)])
def test_head_dims_simt(dk, dv):
    ins = oracle.make_bigla_inputs(1, 2, 150, dk, dv, seed=dk + dv)
    ref = oracle.naive_bi_gla(*ins)
    assert rel_err(_run(*ins, torch.float32, 1), ref) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_strided_views_of_packed_projections(dtype):
    """q/k/v and the gates as [B,H,L,d] views of [B,L,(h d)] projections, output written as [B,L,H,dv]."""
    import vig_b200
    B, H, L, dk, dv = 2, 3, 196, 32, 64
    gen = torch.Generator().manual_seed(5)
    z = torch.randn(B, L, 2 * H * dk + H * dv, generator=gen).to(dtype)
    graw = torch.randn(B, L, 2 * H * dk, generator=gen).to(dtype)
    heads = lambda t, d: t.unflatten(-1, (H, d)).permute(0, 2, 1, 3)
    split = lambda zz, gg: (heads(zz[..., :H * dk], dk), heads(zz[..., H * dk:2 * H * dk], dk), heads(zz[..., 2 * H * dk:], dv),
                            heads(gg[..., :H * dk], dk), heads(gg[..., H * dk:], dk))
    q, k, v, gf, gb = split(z.float(), graw.float())
    lf = lambda t: torch.nn.functional.logsigmoid(t) / 16
    ref = oracle.naive_bi_gla(q, k, v, lf(gf), lf(gb), out_scale=0.25)
    zc, gc = z.cuda(), graw.cuda()
    qd, kd, vd, gfd, gbd = split(zc, gc)
    o = torch.empty(B, L, H, dv, dtype=dtype, device="cuda").permute(0, 2, 1, 3)
    vig_b200.bi_gla(qd, kd, vd, gfd, gbd, out_scale=0.25, out=o, gate_logit_normalizer=16.0)
    assert rel_err(o.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_direction_with_states(golden_bigla, dtype):
    import vig_b200
    q, k, v, g, _ = oracle.make_bigla_inputs(1, 2, 64, 64, 64, 5)
    h0 = torch.randn(1, 2, 64, 64, generator=torch.Generator().manual_seed(6))
    o, hT = vig_b200.fused_chunk_gla(*_cuda((q, k, v, g), dtype), initial_state=h0.cuda(), output_final_state=True)
    tol = TOL[dtype]
    assert rel_err(o.float(), golden_bigla["gla_state_o"]) < tol
    assert rel_err(hT, golden_bigla["gla_state_hT"]) < tol
    # reverse scan == forward scan of the flipped sequence
    o_r, h_r = vig_b200.fused_recurrent_gla(*_cuda((q, k, v, g), dtype), None, reverse=True, output_final_state=True)
    ref_o, ref_h = oracle.naive_gla(*[t.to(dtype).float() for t in (q, k, v, g)], reverse=True)
    assert rel_err(o_r.float(), ref_o) < tol and rel_err(h_r, ref_h) < tol


def test_reference_entry_point_bid_fused_recurrent(golden_bigla):
    import vig_b200
    B, H, L, dk, dv, seed = (int(x) for x in golden_bigla["bigla_cfg1_shape"])
    q, k, v, gf, gb = _cuda(oracle.make_bigla_inputs(B, H, L, dk, dv, seed), torch.float32)
    o, state = vig_b200.bid_fused_recurrent_gla(q, k, v, torch.cat([gf, gb], 0), None)
    assert state is None
    assert rel_err(o, golden_bigla["bigla_cfg1_o"] / 2) < 1e-4


def test_states_for_sequence_split():
    """Final states + total log-decay of two halves chain to the full-sequence result."""
    import vig_b200
    B, H, L, dk, dv = 1, 2, 256, 64, 64
    ins = oracle.make_bigla_inputs(B, H, L, dk, dv, seed=9)
    ref = oracle.naive_bi_gla(*ins)
    q, k, v, gf, gb = _cuda(ins, torch.float32)
    half = L // 2
    lo = [t[:, :, :half] for t in (q, k, v, gf, gb)]
    hi = [t[:, :, half:] for t in (q, k, v, gf, gb)]
    _, ex_lo = vig_b200.bi_gla(*lo, output_final_state=True, output_logdecay=True, want_output=False)
    _, ex_hi = vig_b200.bi_gla(*hi, output_final_state=True, output_logdecay=True, want_output=False)
    o_lo = vig_b200.bi_gla(*lo, init_state_bwd=ex_hi["final_bwd"])
    o_hi = vig_b200.bi_gla(*hi, init_state_fwd=ex_lo["final_fwd"])
    assert rel_err(torch.cat([o_lo, o_hi], 2), ref) < 1e-4
    assert rel_err(ex_lo["logdecay_fwd"], ins[3][:, :, :half].sum(2)) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_properties_at_full_size(dtype):
    """Sizes the CPU oracle cannot finish quickly (the L=4096 benchmark shape): flip symmetry and linearity in v."""
    import vig_b200
    B, H, L, dk, dv = 4, 3, 4096, 64, 64
    q, k, v, gf, gb = _cuda(oracle.make_bigla_inputs(B, H, L, dk, dv, seed=1), dtype)
    o = vig_b200.bi_gla(q, k, v, gf, gb)
    flip = lambda t: t.flip(2).contiguous()
    o_flip = vig_b200.bi_gla(flip(q), flip(k), flip(v), flip(gb), flip(gf))      # reversing time swaps the two scans
    tol = TOL[dtype]
    assert rel_err(o_flip.flip(2).float(), o.float()) < tol
    o2 = vig_b200.bi_gla(q, k, (2 * v).contiguous(), gf, gb)
    assert rel_err(o2.float(), 2 * o.float()) < tol
    # first 300 tokens of batch 0 with the backward scan off depend only on those tokens: check them against the oracle
    o_f = vig_b200.bi_gla(q, k, v, gf, None, dir_mask=1)
    ref, _ = oracle.naive_gla(*[t[:1, :, :300].float().cpu() for t in (q, k, v, gf)])
    assert rel_err(o_f[:1, :, :300].float(), ref) < tol


def test_empty_batch_and_errors():
    import vig_b200
    z = torch.zeros(0, 3, 16, 64, device="cuda")
    assert vig_b200.bi_gla(z, z, z, z, z).shape == (0, 3, 16, 64)
    bad = torch.zeros(1, 1, 8, 48, device="cuda")
    with pytest.raises(RuntimeError):
        vig_b200.bi_gla(bad, bad, bad, bad, bad)


@pytest.mark.parametrize("shape", [(2, 3, 1300, 64), (1, 2, 4096, 32), (3, 1, 700, 64)])
def test_single_launch_form_matches_oracle_and_three_launch_form(shape):
    """The persistent single-launch form of the tensor-core path (impl 3): same result as the default form up to
    bf16 rounding of the cross-segment term, final states and total decay included, with initial states."""
    import vig_b200
    from vig_b200 import _lib
    B, H, L, dk = shape
    ins = oracle.make_bigla_inputs(B, H, L, dk, 64, seed=L)
    g = torch.Generator().manual_seed(3)
    i_f, i_b = torch.randn(B, H, dk, 64, generator=g), torch.randn(B, H, dk, 64, generator=g)
    dev = _cuda(ins, torch.bfloat16)
    kw = dict(init_state_fwd=i_f.cuda(), init_state_bwd=i_b.cuda(), output_final_state=True, output_logdecay=True)
    o1, ex1 = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_SINGLE, **kw)
    o0, ex0 = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC, **kw)
    ref, s_f, s_b = oracle.naive_bi_gla(*[t.float().cpu() for t in dev], init_fwd=i_f, init_bwd=i_b, return_states=True)
    assert rel_err(o1.float(), ref) < 2e-2
    assert rel_err(o1.float(), o0.float()) < 1e-2
    assert rel_err(ex1["final_fwd"], s_f) < 2e-2 and rel_err(ex1["final_bwd"], s_b) < 2e-2
    assert rel_err(ex1["logdecay_fwd"], ex0["logdecay_fwd"]) < 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,dir_mask,init", [((2, 3, 1300), 3, True), ((1, 1, 128), 3, False), ((3, 2, 196), 3, False),
                                                 ((2, 2, 1024), 1, True), ((2, 2, 700), 2, False), ((30, 3, 1000), 3, False),
                                                 # enough chains for long work items: 8 chunks with a tail of 4, 4, 1 (ragged last chunk),
                                                 # one direction only, 4 chunks with a tail of 2, 2
                                                 ((50, 3, 2100), 3, True), ((100, 3, 2100), 1, True), ((100, 3, 1500), 2, False)])
def test_wavefront_form_matches_oracle(shape, dir_mask, init, dtype):
    """The warp-specialised wavefront form (impl 5): every state passes from segment to segment through the
    mailbox, the two directions of a chunk meet in the output tensor (store, then reduction); small batches run
    work items of 2 chunks, large ones 4 or 8 with shorter items at the end of every chain."""
    import vig_b200
    from vig_b200 import _lib
    B, H, L = shape
    ins = oracle.make_bigla_inputs(B, H, L, 64, 64, seed=L + dir_mask)
    g = torch.Generator().manual_seed(5)
    i_f, i_b = torch.randn(B, H, 64, 64, generator=g), torch.randn(B, H, 64, 64, generator=g)
    dev = _cuda(ins, dtype)
    kw = dict(output_final_state=True, output_logdecay=True, dir_mask=dir_mask)
    if init:
        kw.update(init_state_fwd=i_f.cuda(), init_state_bwd=i_b.cuda())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o1, ex1 = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_WAVE, status=status, **kw)
    o0, ex0 = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_SPLIT, **kw)
    assert int(status.item()) == 0
    assert rel_err(o1.float(), o0.float()) < 1.5e-2    # two bf16 results: a couple of output ulps apart at most
    for name in ex0:                                   # operands rounded differently (packed scaling), gates summed in another order
        tol = 1e-5 if name.startswith("logdecay") else 1e-2
        assert rel_err(ex1[name], ex0[name]) < tol, name
    if B * L <= 4096:                                  # the naive oracle is a token loop
        f32 = [t.float().cpu() for t in dev]
        if dir_mask == 3:
            ref = oracle.naive_bi_gla(*f32, init_fwd=i_f if init else None, init_bwd=i_b if init else None)
            assert rel_err(o1.float(), ref) < 2e-2


@pytest.mark.parametrize("shape,dir_mask,impl_wave", [((2, 3, 1300), 3, True), ((50, 3, 2100), 3, False), ((100, 3, 1500), 1, False),
                                                      ((3, 2, 196), 2, True)])
def test_wavefront_form_states_only(shape, dir_mask, impl_wave):
    """A call without an output tensor (end states and summed log-gates only: the summary pass of the sequence split) runs
    the wavefront kernel without its score / output half -- on request, and by default for large batches -- and gives the
    states of the full call and of the three-launch form."""
    import vig_b200
    from vig_b200 import _lib
    B, H, L = shape
    dev = _cuda(oracle.make_bigla_inputs(B, H, L, 64, 64, seed=L + 7), torch.bfloat16)
    kw = dict(output_final_state=True, output_logdecay=True, dir_mask=dir_mask)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _, ex = vig_b200.bi_gla(*dev, want_output=False, status=status, impl=_lib.IMPL_TC_WAVE if impl_wave else _lib.IMPL_AUTO, **kw)
    assert int(status.item()) == 0
    _, ex_full = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_WAVE, **kw)
    _, ex_split = vig_b200.bi_gla(*dev, want_output=False, impl=_lib.IMPL_TC_SPLIT, **kw)
    assert set(ex) == set(ex_full) == set(ex_split)
    for name in ex:
        assert torch.equal(ex[name], ex_full[name]), name               # the same state chain, bit for bit
        tol = 1e-5 if name.startswith("logdecay") else 1e-2
        assert rel_err(ex[name], ex_split[name]) < tol, name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,dir_mask,init,impl_wave", [((2, 3, 1300), 3, True, True), ((50, 3, 2100), 3, False, False),
                                                           ((100, 3, 1500), 2, True, False), ((3, 2, 196), 3, False, True)])
def test_wavefront_form_dk32(shape, dir_mask, init, impl_wave, dtype):
    """The reference's shipped head size (dk = 32, dv = 64) in the wavefront form: the q / k / gate boxes are 64 channels
    wide over 32-channel tensors, the upper half zero-filled by the TMA unit; initial states go in and final states and
    log-decays come out as [.., 32, ..] tensors.  Against the three-launch form (which has a dk = 32 kernel of its own) and,
    where the token loop is affordable, the fp32 oracle; the states-only call gives the same states bit for bit."""
    import vig_b200
    from vig_b200 import _lib
    B, H, L = shape
    ins = oracle.make_bigla_inputs(B, H, L, 32, 64, seed=L + dir_mask)
    g = torch.Generator().manual_seed(9)
    i_f, i_b = torch.randn(B, H, 32, 64, generator=g), torch.randn(B, H, 32, 64, generator=g)
    dev = _cuda(ins, dtype)
    kw = dict(output_final_state=True, output_logdecay=True, dir_mask=dir_mask)
    if init:
        kw.update(init_state_fwd=i_f.cuda(), init_state_bwd=i_b.cuda())
    impl = _lib.IMPL_TC_WAVE if impl_wave else _lib.IMPL_AUTO
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o1, ex1 = vig_b200.bi_gla(*dev, impl=impl, status=status, **kw)
    o0, ex0 = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_SPLIT, **kw)
    assert int(status.item()) == 0
    assert rel_err(o1.float(), o0.float()) < 1.5e-2
    for name in ex0:
        assert ex1[name].shape == ex0[name].shape
        tol = 1e-5 if name.startswith("logdecay") else 1e-2
        assert rel_err(ex1[name], ex0[name]) < tol, name
    _, ex_so = vig_b200.bi_gla(*dev, want_output=False, impl=impl, **kw)
    for name in ex1:
        assert torch.equal(ex_so[name], ex1[name]), name
    if B * L <= 4096 and dir_mask == 3:
        f32 = [t.float().cpu() for t in dev]
        ref = oracle.naive_bi_gla(*f32, init_fwd=i_f if init else None, init_bwd=i_b if init else None)
        assert rel_err(o1.float(), ref) < 2e-2


def test_wavefront_form_is_the_default_for_large_batches():
    """Enough (sequence, direction) chains to fill the GPU and more than one segment: the default routes to the
    wavefront form; results agree with the three-launch form and a second call gives the same bits."""
    import vig_b200
    from vig_b200 import _lib
    B, H, L = 40, 3, 768
    dev = _cuda(oracle.make_bigla_inputs(B, H, L, 64, 64, seed=11), torch.bfloat16)
    o_auto = vig_b200.bi_gla(*dev)
    o_wave = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_WAVE)
    o_split = vig_b200.bi_gla(*dev, impl=_lib.IMPL_TC_SPLIT)
    assert torch.equal(o_auto, o_wave)
    assert torch.equal(o_auto, vig_b200.bi_gla(*dev))
    assert rel_err(o_auto.float(), o_split.float()) < 1e-2


def _strong_gate_inputs(per_token, L=300, seed=2):
    q, k, v, _, _ = oracle.make_bigla_inputs(1, 2, L, 64, 64, seed=seed)
    gen = torch.Generator().manual_seed(seed + 100)
    gf = -per_token * (0.5 + torch.rand(1, 2, L, 64, generator=gen))
    gb = -per_token * (0.5 + torch.rand(1, 2, L, 64, generator=gen))
    return q, k, v, gf, gb


def test_strong_gates_inside_the_factorisation_range():
    """Gates of about -0.8 per token: the CTA-wide vote takes the clamped code path, nothing is clamped."""
    import vig_b200
    from vig_b200 import _lib
    ins = [t.bfloat16() for t in _strong_gate_inputs(0.8)]
    ref = oracle.naive_bi_gla(*[t.float() for t in ins])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o = vig_b200.bi_gla(*[t.cuda() for t in ins], impl=_lib.IMPL_TC, status=status)
    assert rel_err(o.float(), ref) < 2e-2
    assert int(status.item()) == 0


def test_gates_beyond_the_range_are_flagged_and_exact_on_the_simt_path():
    import vig_b200
    from vig_b200 import _lib
    ins = [t.bfloat16() for t in _strong_gate_inputs(4.0)]
    ref = oracle.naive_bi_gla(*[t.float() for t in ins])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o = vig_b200.bi_gla(*[t.cuda() for t in ins], impl=_lib.IMPL_TC, status=status)
    assert int(status.item()) & 2                                  # reported, not trapped
    assert torch.isfinite(o.float()).all()
    o_simt = vig_b200.bi_gla(*[t.cuda() for t in ins], impl=_lib.IMPL_SIMT, status=status)
    assert rel_err(o_simt.float(), ref) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamp_min_and_raw_logits(dtype):
    """vig.py:439-441: g = clamp_min(logsigmoid(x) / 16, c)."""
    import vig_b200
    q, k, v, _, _ = oracle.make_bigla_inputs(2, 2, 200, 32, 64, seed=4)
    gen = torch.Generator().manual_seed(9)
    xf, xb = 8 * torch.randn(2, 2, 200, 32, generator=gen), 8 * torch.randn(2, 2, 200, 32, generator=gen)
    ins = [t.to(dtype) for t in (q, k, v, xf, xb)]
    lf = lambda t: torch.clamp_min(torch.nn.functional.logsigmoid(t.float()) / 16, -0.3)
    ref = oracle.naive_bi_gla(ins[0].float(), ins[1].float(), ins[2].float(), lf(ins[3]), lf(ins[4]))
    o = vig_b200.bi_gla(*[t.cuda() for t in ins], gate_logit_normalizer=16.0, clamp_min=-0.3)
    assert rel_err(o.float(), ref) < TOL[dtype]


def test_wavefront_form_raw_logits_clamp_and_range_flag():
    """The wavefront kernel's gate path: raw logits with `logsigmoid(x) / 16` and a lower clamp inside the kernel
    (vig.py:439-441), strong gates inside the factorisation range, and gates beyond it (flagged, finite)."""
    import vig_b200
    from vig_b200 import _lib
    q, k, v, _, _ = oracle.make_bigla_inputs(2, 2, 600, 64, 64, seed=6)
    gen = torch.Generator().manual_seed(10)
    xf, xb = 8 * torch.randn(2, 2, 600, 64, generator=gen), 8 * torch.randn(2, 2, 600, 64, generator=gen)
    ins = [t.bfloat16() for t in (q, k, v, xf, xb)]
    lf = lambda t: torch.clamp_min(torch.nn.functional.logsigmoid(t.float()) / 16, -0.3)
    ref = oracle.naive_bi_gla(ins[0].float(), ins[1].float(), ins[2].float(), lf(ins[3]), lf(ins[4]))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o = vig_b200.bi_gla(*[t.cuda() for t in ins], gate_logit_normalizer=16.0, clamp_min=-0.3, impl=_lib.IMPL_TC_WAVE, status=status)
    assert rel_err(o.float(), ref) < 2e-2 and int(status.item()) == 0
    # about -0.8 per token: exponents reach ~50 around the reference token, nothing is clamped
    strong = [t.bfloat16() for t in _strong_gate_inputs(0.8, L=600)]
    o = vig_b200.bi_gla(*[t.cuda() for t in strong], impl=_lib.IMPL_TC_WAVE, status=status)
    assert rel_err(o.float(), oracle.naive_bi_gla(*[t.float() for t in strong])) < 2e-2 and int(status.item()) == 0
    # about -4 per token: beyond the range; reported in the status word, output finite
    wild = [t.bfloat16() for t in _strong_gate_inputs(4.0, L=600)]
    o = vig_b200.bi_gla(*[t.cuda() for t in wild], impl=_lib.IMPL_TC_WAVE, status=status)
    assert int(status.item()) & 2 and torch.isfinite(o.float()).all()
