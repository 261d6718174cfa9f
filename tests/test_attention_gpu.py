"""The tcgen05 attention kernels against a plain fp32 PyTorch attention
(explicit scores, causal mask, softmax, autograd for the gradients)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(qkv, dctx, B, S, nq, nkv, hd):
    x = qkv.float().detach().requires_grad_(True)
    v = x.view(B, S, nq + 2 * nkv, hd)
    q = v[:, :, :nq].transpose(1, 2)
    k = v[:, :, nq:nq + nkv].transpose(1, 2).repeat_interleave(nq // nkv, 1)
    vv = v[:, :, nq + nkv:].transpose(1, 2).repeat_interleave(nq // nkv, 1)
    att = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    att = att.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(att, -1)
    out = torch.softmax(att, -1) @ vv
    ctx = out.transpose(1, 2).reshape(B * S, nq * hd)
    ctx.backward(dctx.float())
    return ctx.detach(), lse.detach(), x.grad


@pytest.mark.parametrize("B,S,nq,nkv,hd", [(2, 256, 4, 2, 64), (1, 300, 4, 1, 64), (2, 512, 4, 2, 128),
                                           (1, 200, 2, 2, 128), (1, 1024, 8, 2, 64)])
def test_native_attention_matches_fp32_reference(B, S, nq, nkv, hd):
    from sga_b200 import kernels as K
    from sga_b200.ops import attention as A

    dev = "cuda"
    torch.manual_seed(S + hd)
    T = B * S
    qkv = (torch.randn(T, (nq + 2 * nkv) * hd, device=dev) * 0.8).to(torch.bfloat16)
    dctx = (torch.randn(T, nq * hd, device=dev) * 0.5).to(torch.bfloat16)
    assert A.native_available(qkv, hd), "the native attention kernels must be the CUDA path"
    ctx, saved = A.attn_fwd(qkv, B, S, nq, nkv, hd)
    assert saved[0] == "native"
    dqkv = A.attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd)
    torch.cuda.synchronize()
    assert int(K.gemm_err_word(dev).item()) == 0
    ref_ctx, ref_lse, ref_d = _reference(qkv, dctx, B, S, nq, nkv, hd)
    assert torch.allclose(saved[2], ref_lse, atol=2e-2, rtol=1e-3)
    err = (ctx.float() - ref_ctx).abs().max().item()
    assert err < 3e-2, f"context differs by {err}"
    scale = ref_d.abs().max().item()
    derr = (dqkv.float() - ref_d).abs().max().item()
    assert derr < 0.03 * scale + 2e-2, f"d(qkv) differs by {derr} (scale {scale})"
    # reproducible bit for bit
    dqkv2 = A.attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd)
    assert torch.equal(dqkv, dqkv2)


@pytest.mark.parametrize("B,S,nq,nkv,hd", [(1, 640, 4, 2, 64), (1, 512, 2, 1, 128)])
def test_native_attention_growing_scores(B, S, nq, nkv, hd):
    """Keys grow with their position, so a row's maximum moves by far more than a factor of 2^8 from one
    key block to the next: the forward must re-express what it has accumulated against the new maximum
    (the common case of the test above never needs to after the first block)."""
    from sga_b200 import kernels as K
    from sga_b200.ops import attention as A

    dev = "cuda"
    torch.manual_seed(7 * S + hd)
    T = B * S
    qkv = (torch.randn(T, (nq + 2 * nkv) * hd, device=dev) * 0.8)
    ramp = 1.0 + 12.0 * (torch.arange(T, device=dev) % S).float() / S
    qkv[:, :nq * hd] *= 2.0
    qkv[:, nq * hd:(nq + nkv) * hd] *= ramp[:, None]
    qkv = qkv.to(torch.bfloat16)
    dctx = (torch.randn(T, nq * hd, device=dev) * 0.5).to(torch.bfloat16)
    ctx, saved = A.attn_fwd(qkv, B, S, nq, nkv, hd)
    assert saved[0] == "native"
    dqkv = A.attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd)
    torch.cuda.synchronize()
    assert int(K.gemm_err_word(dev).item()) == 0
    ref_ctx, ref_lse, ref_d = _reference(qkv, dctx, B, S, nq, nkv, hd)
    # the scores reach a few hundred here: compare the log-sum-exp relative to that
    assert torch.allclose(saved[2], ref_lse, atol=5e-2, rtol=2e-3)
    err = (ctx.float() - ref_ctx).abs().max().item()
    assert err < 5e-2, f"context differs by {err}"
    scale = ref_d.abs().max().item()
    derr = (dqkv.float() - ref_d).abs().max().item()
    assert derr < 0.03 * scale + 2e-2, f"d(qkv) differs by {derr} (scale {scale})"
