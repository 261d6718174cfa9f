"""The hand-scheduled forward/backward of the GPT model against PyTorch autograd
on the same parameters (fp32 reference of the same architecture)."""
import math

import pytest
import torch

from sga_b200.models.gpt import GPT, get_config
from sga_b200.ops import functional as F


def _autograd_reference(model, tokens, targets):
    c = model.cfg
    P = {s.name: s.main.detach().clone().to(torch.bfloat16).float().requires_grad_() for s in model.arena.slots}
    dev = tokens.device
    B, S = tokens.shape
    cs, sn = F.rope_tables(c.seq_len, c.head_dim, c.rope_theta, dev)

    def rms(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def rope(x):  # [B, S, H, hd]
        half = c.head_dim // 2
        a, b = x[..., :half], x[..., half:]
        co, si = cs[:S][None, :, None, :], sn[:S][None, :, None, :]
        return torch.cat([a * co - b * si, b * co + a * si], -1)

    x = P["embedding.word_embeddings.weight"][tokens]
    nq, nkv, hd = c.n_heads, c.n_kv_heads, c.head_dim
    for i in range(c.num_layers):
        p = f"decoder.layers.{i}."
        h = rms(x, P[p + "input_layernorm.weight"], c.norm_eps)
        qkv = h @ P[p + "self_attention.linear_qkv.weight"].t()
        qkv = qkv.view(B, S, nq + 2 * nkv, hd)
        q, k, v = qkv[:, :, :nq], qkv[:, :, nq:nq + nkv], qkv[:, :, nq + nkv:]
        if c.qk_norm:
            q = rms(q, P[p + "self_attention.q_layernorm.weight"], c.norm_eps)
            k = rms(k, P[p + "self_attention.k_layernorm.weight"], c.norm_eps)
        q, k = rope(q), rope(k)
        rep = nq // nkv
        kk = k.repeat_interleave(rep, 2).transpose(1, 2)
        vv = v.repeat_interleave(rep, 2).transpose(1, 2)
        att = (q.transpose(1, 2) @ kk.transpose(-1, -2)) / math.sqrt(hd)
        att = att.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=dev).tril(), float("-inf"))
        ctx = (torch.softmax(att, -1) @ vv).transpose(1, 2).reshape(B, S, nq * hd)
        x = x + ctx @ P[p + "self_attention.linear_proj.weight"].t()
        h = rms(x, P[p + "pre_mlp_layernorm.weight"], c.norm_eps)
        gu = h @ P[p + "mlp.linear_fc1.weight"].t()
        x = x + (torch.nn.functional.silu(gu[..., :c.ffn]) * gu[..., c.ffn:]) @ P[p + "mlp.linear_fc2.weight"].t()
    hf = rms(x, P["decoder.final_layernorm.weight"], c.norm_eps)
    head = P["embedding.word_embeddings.weight"] if c.tied_embeddings else P["output_layer.weight"]
    logits = hf @ head.t()
    loss = torch.nn.functional.cross_entropy(logits.view(B * S, -1), targets.reshape(-1))
    loss.backward()
    return loss.detach(), {k: v.grad for k, v in P.items()}


def _check(device, name, tol, expect_native_attention=False):
    cfg = get_config(name)
    if expect_native_attention:
        from sga_b200.ops import attention as A

        paths = []
        inner = A.attn_fwd

        def spy(*args, **kw):
            out = inner(*args, **kw)
            paths.append(out[1][0])
            return out

        A.attn_fwd = spy
        try:
            _check(device, name, tol)
        finally:
            A.attn_fwd = inner
        assert paths and all(p == "native" for p in paths), f"attention did not take the native kernels: {paths}"
        return
    model = GPT(cfg, device=device, bucket_elems=20000, seed=3)
    # make the norm weights non-trivial
    g = torch.Generator().manual_seed(1)
    for s in model.arena.slots:
        if s.spec.init == "ones":
            s.main.copy_((1 + 0.1 * torch.randn(s.main.shape, generator=g)).to(s.main.device))
    model.arena.sync_model_from_main()
    B, S = 2, cfg.seq_len
    tokens = torch.randint(0, cfg.vocab, (B, S), generator=g).to(device)
    targets = torch.randint(0, cfg.vocab, (B, S), generator=g).to(device)
    seen = []
    loss = model.forward_backward(tokens, targets, on_param_done=lambda s: seen.append(s.name))
    ref_loss, ref_grads = _autograd_reference(model, tokens, targets)
    assert abs(loss.item() - ref_loss.item()) < tol * 2
    assert sorted(seen) == sorted(s.name for s in model.arena.slots), "every parameter must be reported exactly once"
    # gradients become final in arena order
    order = [s.name for s in model.arena.slots]
    assert seen == order, "parameters must finish in arena (bucket) order"
    for s in model.arena.slots:
        rg = ref_grads[s.name]
        err = (s.grad - rg).abs().max().item()
        scale = rg.abs().max().item() + 1e-6
        assert err <= tol * scale + 1e-5, f"{s.name}: err {err} scale {scale}"


@pytest.mark.parametrize("name", ["test_tiny", "test_tiny_qk"])
def test_model_matches_autograd_cpu(name):
    _check("cpu", name, 0.05)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["test_tiny", "test_tiny_qk"])
def test_model_matches_autograd_gpu(name):
    _check("cuda:0", name, 0.08)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["test_hd64", "test_hd128_qk"])
def test_model_with_native_attention_matches_autograd_gpu(name):
    """The whole model on its production path (CTA-pair tcgen05 GEMMs, native attention at head
    dimension 64 and 128, QK-norm, sequence length not a multiple of the attention tile) against autograd."""
    _check("cuda:0", name, 0.08, expect_native_attention=True)

