"""The element-wise glue of the DiT block around the MoE block (models.py:514-520) inside this package's
kernels, against the oracle: LayerNorm + modulation in one pass, the gated residual inside the combine kernel,
and ``SparseMoeBlock.forward_with_glue`` as a whole.  fp32 within 1e-5, bf16 within 2e-2."""
import pytest
import torch
import torch.nn.functional as F

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _ops():
    from dice_b200 import ops

    return ops


@pytest.mark.parametrize("b,t,h", [(1, 1, 64), (3, 77, 1152), (2, 256, 1792), (5, 33, 1408), (2, 9, 2048)])
@pytest.mark.parametrize("dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                             (torch.float32, torch.bfloat16)])
def test_ln_modulate(cuda_device, b, t, h, dtype, out_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(b * 1000 + t + h)
    x = (torch.randn(b, t, h, generator=g) * 1.7 + 0.3).to(dtype)
    shift = (torch.randn(b, h, generator=g) * 0.2).to(dtype)
    scale = (torch.randn(b, h, generator=g) * 0.2).to(dtype)
    got = ops.ln_modulate(x.to(cuda_device), shift.to(cuda_device), scale.to(cuda_device), 1e-6, out_dtype=out_dtype)
    assert got.dtype == out_dtype and got.shape == x.shape
    want = O.modulate(F.layer_norm(x.float(), (h,), None, None, 1e-6), shift.float(), scale.float())
    if out_dtype == torch.float32:
        torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-5)
    else:
        torch.testing.assert_close(got.cpu().float(), want, rtol=1e-2, atol=1e-2)  # one bf16 rounding of the result
    # shift / scale may be column slices of the adaLN output, as DiTBlock passes them
    six = torch.randn(b, 6 * h, generator=g).to(dtype).to(cuda_device)
    s3, s4 = six.chunk(6, dim=1)[3], six.chunk(6, dim=1)[4]
    got2 = ops.ln_modulate(x.to(cuda_device), s3, s4, 1e-6, out_dtype=out_dtype)
    want2 = O.modulate(F.layer_norm(x.float(), (h,), None, None, 1e-6), s3.cpu().float(), s4.cpu().float())
    torch.testing.assert_close(got2.cpu().float(), want2, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_combine_applies_the_gated_residual(cuda_device, dtype):
    ops = _ops()
    b, t, h, e = 3, 50, 256, 8
    n = b * t
    g = torch.Generator().manual_seed(6)
    rows_in = torch.randn(n, h, generator=g).to(dtype)
    flat = torch.randint(0, e, (2 * n,), generator=g)
    w = torch.rand(n, 2, generator=g)
    addend = torch.randn(n, h, generator=g).to(dtype)
    resid = torch.randn(n, h, generator=g).to(dtype)
    gate = torch.randn(b, h, generator=g).to(dtype)
    pos, _, _ = ops.permute_plan(flat.to(cuda_device), e)
    rows = ops.permute_rows(rows_in.to(cuda_device), pos, 2)
    wd = w.to(cuda_device)
    out = ops.unpermute_combine(rows, pos[0::2], rows, pos[1::2], wd[:, 0], wd[:, 1], n, addend=addend.to(cuda_device),
                                resid=resid.to(cuda_device), gate=gate.to(cuda_device), tokens_per_sample=t)
    y = rows_in.float() * (w[:, 0] + w[:, 1]).view(-1, 1) + addend.float()
    want = resid.float() + gate.float().repeat_interleave(t, dim=0) * y
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.cpu().float(), want, **tol)
    # a gate without a residual, and a residual without a gate
    only_gate = ops.unpermute_combine(rows, pos[0::2], None, None, None, None, n, gate=gate.to(cuda_device), tokens_per_sample=t)
    torch.testing.assert_close(only_gate.cpu().float(), gate.float().repeat_interleave(t, dim=0) * rows_in.float(), **tol)
    only_res = ops.unpermute_combine(rows, pos[0::2], None, None, None, None, n, resid=resid.to(cuda_device))
    torch.testing.assert_close(only_res.cpu().float(), resid.float() + rows_in.float(), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_forward_with_glue(cuda_device, dtype):
    """x + gate * moe(modulate(LayerNorm(x))) through the fused path equals the oracle's restatement of
    models.py:518-519 around the oracle's block (fp32: routing exact, 1e-5; bf16: the oracle on the kernel's
    routing of the fused input, 2e-2) and the package's own unfused formulation."""
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    ops = _ops()
    torch.manual_seed(8)
    b, t, h, e = 3, 111, 128, 8
    blk = SparseMoeBlock(h, 4, e, 2, 1, 0, 1, ParaMode()).to(device=cuda_device, dtype=dtype).eval()
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(b, t, h, generator=g, device=cuda_device).to(dtype)
    ada = (torch.randn(b, 6 * h, generator=g, device=cuda_device) * 0.3).to(dtype)
    _, _, _, shift, scale, gate = ada.chunk(6, dim=1)
    y = blk.forward_with_glue(x, shift, scale, gate)
    blk.check_status()
    assert y.shape == x.shape and y.dtype == dtype
    sd = {k: v.detach().float().cpu() for k, v in blk.state_dict().items()}
    ex = [[sd[f"experts.{i}.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj")] for i in range(e)]
    sh = [sd[f"shared_experts.{p}.weight"] for p in ("gate_proj", "up_proj", "down_proj")]
    xc, sc, scl, gc = x.cpu().float(), shift.cpu().float(), scale.cpu().float(), gate.cpu().float()
    if dtype == torch.float32:
        want = O.dit_block_moe_half(xc, sc, scl, gc, lambda z: O.moe_block_forward(z, sd["gate.weight"], ex, sh)["out"])
        torch.testing.assert_close(y.cpu(), want, rtol=1e-5, atol=1e-5)
    else:
        x_in = ops.ln_modulate(x, shift.contiguous(), scale.contiguous(), 1e-6)
        idx, w, _, _ = ops.router_top2(x_in.view(-1, h), blk.gate.weight.detach())

        def moe_fn(z):  # the oracle's block on the kernel's routing
            z2 = x_in.cpu().float().view(-1, h)
            out = O.moe_infer(z2, idx.cpu().view(-1), w.cpu().view(-1), ex, "swiglu") + O.run_expert(z2, sh, "swiglu")
            return out.view(b, t, h)

        want = O.dit_block_moe_half(xc, sc, scl, gc, moe_fn)
        err = ((y.cpu().float() - want).norm() / want.norm()).item()
        assert err < 2e-2, err
    # the plain formulation through the same block
    normed = F.layer_norm(x.float(), (h,), None, None, 1e-6).to(dtype)
    plain = x + gate.unsqueeze(1) * blk(normed * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1))
    err = ((y.float() - plain.float()).norm() / plain.float().norm()).item()
    assert err < (1e-5 if dtype == torch.float32 else 2e-2), err
