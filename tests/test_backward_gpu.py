"""Backward operators through autograd on the gcu device against CPU autograd on
the same inputs: silu, softmax, layer_norm, embedding, and one training step of an
unfused Llama-style decoder layer (every op of it, forward and backward, on the device)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch_gcu  # noqa: F401
    return torch.device("gcu", 0)


def grads(fn, inputs, g_out, device):
    xs = [t.detach().clone().to(device).requires_grad_(t.is_floating_point()) for t in inputs]
    y = fn(*xs)
    y.backward(g_out.to(device))
    return y.detach().cpu(), [x.grad.cpu() if x.grad is not None else None for x in xs]


def check(fn, inputs, g_out, dev, rtol, atol, normwise=False):
    """normwise: 16-bit cases with cancellation (g - p * sum(g)): the CPU rounds its intermediates to
    16 bits, the device keeps fp32 until the store, so single elements differ by an ulp of the large
    terms; the tensors are compared by relative norm instead."""
    y_d, g_d = grads(fn, inputs, g_out, dev)
    y_c, g_c = grads(fn, inputs, g_out, "cpu")
    if normwise:
        assert (y_d.float() - y_c.float()).norm() <= rtol * y_c.float().norm() + atol
        for a, b in zip(g_d, g_c):
            assert a.dtype == b.dtype and a.shape == b.shape
            assert (a.float() - b.float()).norm() <= rtol * b.float().norm() + atol
        return
    assert torch.allclose(y_d.float(), y_c.float(), rtol=rtol, atol=atol)
    for a, b in zip(g_d, g_c):
        assert (a is None) == (b is None)
        if a is not None:
            assert a.dtype == b.dtype and a.shape == b.shape
            assert torch.allclose(a.float(), b.float(), rtol=rtol, atol=atol), (a.float() - b.float()).abs().max()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2 ** -7)])
def test_silu_and_softmax_backward(dev, dtype, tol):
    g = torch.Generator().manual_seed(21)
    x = torch.randn(33, 257, generator=g).to(dtype)
    go = torch.randn(33, 257, generator=g).to(dtype)
    check(F.silu, [x], go, dev, tol, tol)
    check(lambda t: torch.softmax(t, -1), [x], go, dev, tol, tol)
    x3 = torch.randn(4, 50, 6, generator=g).to(dtype)
    check(lambda t: torch.softmax(t, 1), [x3], torch.randn(4, 50, 6, generator=g).to(dtype), dev, tol, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_layer_norm_backward(dev, dtype, tol):
    g = torch.Generator().manual_seed(22)
    x = torch.randn(700, 192, generator=g).to(dtype)
    w = (torch.randn(192, generator=g) * 0.1 + 1).to(dtype)
    b = (torch.randn(192, generator=g) * 0.1).to(dtype)
    go = torch.randn(700, 192, generator=g).to(dtype)
    check(lambda t, ww, bb: F.layer_norm(t, (192,), ww, bb, 1e-5), [x, w, b], go, dev, tol, tol * 30)
    check(lambda t: F.layer_norm(t, (192,)), [x], go, dev, tol, tol)


def test_embedding_backward_is_ordered_and_exact(dev):
    g = torch.Generator().manual_seed(23)
    w = torch.randn(50, 64, generator=g)
    idx = torch.randint(0, 50, (7, 40), generator=g)
    go = torch.randn(7, 40, 64, generator=g)
    y_d, g_d = grads(lambda ww: F.embedding(idx.to(ww.device), ww, padding_idx=3), [w], go, dev)
    y_c, g_c = grads(lambda ww: F.embedding(idx, ww, padding_idx=3), [w], go, "cpu")
    assert torch.equal(y_d, y_c)
    assert torch.equal(g_d[0], g_c[0])      # same summation order as the CPU: bit for bit


def _layer(x, p, heads, kv_heads, head_dim):
    """An unfused Llama-style decoder layer out of registered ATen ops only."""
    B, S, H = x.shape

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    def rope(t):
        half = head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))   # tables on the host
        ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
        cos = torch.cat((ang.cos(), ang.cos()), -1)[None, :, None, :].to(t.device)
        sin = torch.cat((ang.sin(), ang.sin()), -1)[None, :, None, :].to(t.device)
        rot = torch.cat((-t[..., half:], t[..., :half]), -1)
        return t * cos + rot * sin

    h = rms(x, p["n1"])
    q = rope((h @ p["wq"].t()).view(B, S, heads, head_dim)).transpose(1, 2)
    k = rope((h @ p["wk"].t()).view(B, S, kv_heads, head_dim)).transpose(1, 2)
    v = (h @ p["wv"].t()).view(B, S, kv_heads, head_dim).transpose(1, 2)
    rep = heads // kv_heads
    k = k[:, :, None].expand(B, kv_heads, rep, S, head_dim).reshape(B, heads, S, head_dim)
    v = v[:, :, None].expand(B, kv_heads, rep, S, head_dim).reshape(B, heads, S, head_dim)
    s = (q @ k.transpose(-1, -2)) * head_dim ** -0.5
    mask = torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    att = torch.softmax(s, -1) @ v
    r = x + att.transpose(1, 2).reshape(B, S, heads * head_dim) @ p["wo"].t()
    h2 = rms(r, p["n2"])
    return r + (F.silu(h2 @ p["wg"].t()) * (h2 @ p["wu"].t())) @ p["wd"].t()


def test_decoder_layer_training_step(dev):
    g = torch.Generator().manual_seed(24)
    H, heads, kvh, d, ffn, B, S = 128, 4, 2, 32, 256, 2, 48
    shapes = dict(n1=(H,), n2=(H,), wq=(heads * d, H), wk=(kvh * d, H), wv=(kvh * d, H), wo=(H, heads * d),
                  wg=(ffn, H), wu=(ffn, H), wd=(H, ffn))
    params = {k: (torch.randn(s, generator=g) * (0.08 if len(s) == 2 else 0.02) + (0 if len(s) == 2 else 1)) for k, s in shapes.items()}
    x = torch.randn(B, S, H, generator=g)
    target = torch.randn(B, S, H, generator=g)

    def run(device):
        p = {k: v.clone().to(device).requires_grad_() for k, v in params.items()}
        y = _layer(x.to(device), p, heads, kvh, d)
        loss = ((y - target.to(device)) ** 2).mean()
        loss.backward()
        return loss.detach().cpu(), {k: v.grad.cpu() for k, v in p.items()}

    loss_d, g_d = run(dev)
    loss_c, g_c = run("cpu")
    assert torch.allclose(loss_d, loss_c, rtol=1e-4, atol=1e-5)
    for k in params:
        rel = (g_d[k] - g_c[k]).norm() / g_c[k].norm()
        assert rel < 1e-3, (k, rel)


def test_sdpa_trains_through_the_flash_kernels(dev):
    """F.scaled_dot_product_attention with head dim 128 takes the flash forward and, under
    autograd, the flash backward; gradients against CPU autograd in fp32."""
    g = torch.Generator().manual_seed(25)
    bf = torch.bfloat16
    q = torch.randn(2, 4, 256, 128, generator=g).to(bf)
    k = torch.randn(2, 2, 256, 128, generator=g).to(bf)
    v = torch.randn(2, 2, 256, 128, generator=g).to(bf)
    go = torch.randn(2, 4, 256, 128, generator=g).to(bf)
    qd, kd, vd = (t.to(dev).requires_grad_() for t in (q, k, v))
    out = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=True)
    out.backward(go.to(dev))
    qc, kc, vc = (t.float().requires_grad_() for t in (q, k, v))
    ref = F.scaled_dot_product_attention(qc, kc.repeat_interleave(2, 1), vc.repeat_interleave(2, 1), is_causal=True)
    ref.backward(go.float())
    assert torch.allclose(out.detach().cpu().float(), ref.detach(), rtol=2e-2, atol=2e-2)
    for got, want in ((qd.grad, qc.grad), (kd.grad, kc.grad), (vd.grad, vc.grad)):
        rel = (got.cpu().float() - want).norm() / want.norm()
        assert rel < 2e-2, rel


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_log_softmax_and_cross_entropy(dev, dtype, tol):
    g = torch.Generator().manual_seed(26)
    logits = (torch.randn(300, 1000, generator=g) * 3).to(dtype)
    target = torch.randint(0, 1000, (300,), generator=g)
    target[::7] = -100                                        # ignored rows
    w = (torch.rand(1000, generator=g) + 0.5).to(dtype)
    go = torch.randn(300, 1000, generator=g).to(dtype)
    nw = dtype != torch.float32
    check(lambda t: F.log_softmax(t, -1), [logits], go, dev, tol, tol, normwise=nw)
    check(lambda t: F.log_softmax(t, 0), [logits], go, dev, tol, tol, normwise=nw)
    one = torch.ones((), dtype=dtype)
    for kwargs in ({}, {"weight": w}, {"reduction": "sum"}):
        def loss(t, kw=kwargs):
            kw = {k: (v.to(t.device) if torch.is_tensor(v) else v) for k, v in kw.items()}
            return F.cross_entropy(t, target.to(t.device), **kw)
        check(loss, [logits], one, dev, tol, tol, normwise=nw)
    check(lambda t: F.cross_entropy(t, target.to(t.device), reduction="none"), [logits], torch.randn(300, generator=g).to(dtype), dev, tol, tol,
          normwise=nw)


def test_tiny_language_model_step(dev):
    """Embedding -> unfused decoder layer -> tied output projection -> cross-entropy: loss and every
    gradient against CPU autograd."""
    g = torch.Generator().manual_seed(27)
    V, H, heads, kvh, d, ffn, B, S = 97, 128, 4, 2, 32, 256, 2, 40
    shapes = dict(emb=(V, H), n1=(H,), n2=(H,), wq=(heads * d, H), wk=(kvh * d, H), wv=(kvh * d, H), wo=(H, heads * d),
                  wg=(ffn, H), wu=(ffn, H), wd=(H, ffn))
    params = {k: (torch.randn(s, generator=g) * (0.08 if len(s) == 2 else 0.02) + (0 if len(s) == 2 else 1)) for k, s in shapes.items()}
    tokens = torch.randint(0, V, (B, S), generator=g)
    labels = torch.randint(0, V, (B, S), generator=g)

    def run(device):
        p = {k: v.clone().to(device).requires_grad_() for k, v in params.items()}
        x = F.embedding(tokens.to(device), p["emb"])
        y = _layer(x, p, heads, kvh, d)
        logits = y.reshape(B * S, H) @ p["emb"].t()
        loss = F.cross_entropy(logits, labels.reshape(-1).to(device))
        loss.backward()
        return loss.detach().cpu(), {k: v.grad.cpu() for k, v in p.items()}

    loss_d, g_d = run(dev)
    loss_c, g_c = run("cpu")
    assert torch.allclose(loss_d, loss_c, rtol=1e-4, atol=1e-5)
    for k in params:
        rel = (g_d[k] - g_c[k]).norm() / g_c[k].norm()
        assert rel < 1e-3, (k, rel)
