"""The CPU reference paths of the operators against stock PyTorch (no GPU needed)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_reference_layouts(a_mn, b_mn):
    from necklace_b200.ops import gemm
    A, B = torch.randn(20, 12), torch.randn(9, 12)
    out = gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B,
               a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert torch.allclose(out, A @ B.t(), atol=1e-5)


def test_linear_mlp_autograd_cpu():
    from necklace_b200.ops import linear, mlp
    torch.manual_seed(0)
    x = torch.randn(3, 5, 16, requires_grad=True)
    w1, b1 = torch.randn(32, 16, requires_grad=True), torch.randn(32, requires_grad=True)
    w2, b2 = torch.randn(16, 32, requires_grad=True), torch.randn(16, requires_grad=True)
    y = linear(mlp(x, w1, b1, w2, b2, residual=x), w1, b1)
    y.pow(2).mean().backward()
    got = [t.grad.clone() for t in (x, w1, b1, w2, b2)]
    for t in (x, w1, b1, w2, b2):
        t.grad = None
    yr = F.linear(F.linear(F.gelu(F.linear(x, w1, b1), approximate="tanh"), w2, b2) + x, w1, b1)
    yr.pow(2).mean().backward()
    assert torch.allclose(y, yr, atol=1e-4)
    for g, t in zip(got, (x, w1, b1, w2, b2)):
        assert torch.allclose(g, t.grad, atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("rms", [False, True])
def test_norm_cpu(rms):
    from necklace_b200.ops.norm import NormFn
    x = torch.randn(7, 24, requires_grad=True)
    w = torch.randn(24, requires_grad=True)
    b = None if rms else torch.randn(24, requires_grad=True)
    dy = torch.randn(7, 24)
    NormFn.apply(x, w, b, 1e-5, rms).backward(dy)
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    if rms:
        yr = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    else:
        yr = F.layer_norm(x, (24,), w, b, 1e-5)
    yr.backward(dy)
    assert torch.allclose(gx, x.grad, atol=1e-4) and torch.allclose(gw, w.grad, atol=1e-4)


def test_lm_head_loss_cpu():
    from necklace_b200.ops import lm_head_loss
    x = torch.randn(2, 6, 16, requires_grad=True)
    w = torch.randn(40, 16, requires_grad=True)  # 37 valid + 3 pad rows
    tg = torch.randint(0, 37, (2, 6))
    loss = lm_head_loss(x, w, tg, 37)
    (loss * 2.0).backward()
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    ref = F.cross_entropy(F.linear(x, w[:37]).view(-1, 37), tg.view(-1))
    (ref * 2.0).backward()
    assert torch.allclose(loss, ref, atol=1e-5)
    assert torch.allclose(gx, x.grad, atol=1e-5) and torch.allclose(gw, w.grad, atol=1e-5)


def test_attention_cpu_matches_sdpa():
    from necklace_b200.ops import attention_qkv
    B, S, H, D = 2, 10, 3, 8
    qkv = torch.randn(B, S, 3 * H * D, requires_grad=True)
    out = attention_qkv(qkv, H, True)
    out.pow(2).sum().backward()
    g = qkv.grad.clone()
    qkv.grad = None
    q, k, v = (t.view(B, S, H, D).transpose(1, 2) for t in qkv.split(H * D, -1))
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, -1)
    ref.pow(2).sum().backward()
    assert torch.allclose(out, ref, atol=1e-5) and torch.allclose(g, qkv.grad, atol=1e-4)


def _numpy_codec(a, thr):
    """Plain restatement of the reference kernels' arithmetic (quantize.py:16-91)."""
    n = a.shape[0]
    m = (n + 15) // 16
    C = np.zeros((m,) + a.shape[1:], dtype=np.uint32)
    R = np.zeros_like(a)
    for x in range(m):
        for i in range(16):
            xm = 16 * x + i
            if xm >= n:
                break
            row = a[xm]
            pos, neg = row >= thr, row <= -thr
            code = np.where(pos, 1, np.where(neg, 2, 0)).astype(np.uint32)
            R[xm] = np.where(pos, row - thr, np.where(neg, row + thr, row))
            C[x] |= code << np.uint32(2 * i)
    return C, R


def test_quant_matches_numpy_restatement():
    from necklace_b200.ops import matrix_quantize, matrix_dequantize, quantize_flat
    A = torch.randn(50, 7)
    codes, R = matrix_quantize(A, 0.5)
    C_np, R_np = _numpy_codec(A.numpy(), 0.5)
    assert np.array_equal(codes.numpy().view(np.uint32), C_np)
    assert np.allclose(R.numpy(), R_np)
    back = matrix_dequantize(codes, 50, 0.5)
    assert torch.allclose(back + R, A, atol=1e-6)
    g = torch.randn(100)
    res = torch.zeros(100)
    cf = quantize_flat(g, res, 0.5)
    C_np, R_np = _numpy_codec(g.numpy()[:, None], 0.5)
    assert np.array_equal(cf.numpy().view(np.uint32), C_np[:, 0])
    assert np.allclose(res.numpy(), R_np[:, 0])


def test_adam_sgd_cpu():
    from necklace_b200.ops import adam_step, sgd_step
    p0, g = torch.randn(100), torch.randn(100)
    master, m, v = p0.clone(), torch.zeros(100), torch.zeros(100)
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for step in (1, 2, 3):
        adam_step(master, m, v, g, None, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1,
                  step=step)
        ref.grad = g.clone()
        opt.step()
    assert torch.allclose(master, ref.data, atol=1e-6)
    master, mom = p0.clone(), torch.zeros(100)
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9)
    for step in (1, 2):
        sgd_step(master, mom, g, None, lr=0.1, momentum=0.9, first_step=step == 1)
        ref.grad = g.clone()
        opt.step()
    assert torch.allclose(master, ref.data, atol=1e-6)


def test_norm_split_cpu_matches_plain_composition():
    import torch.nn.functional as F
    from necklace_b200.ops.norm import LayerNorm
    torch.manual_seed(3)
    ln = LayerNorm(32, dtype=torch.float32)
    x = torch.randn(5, 32, requires_grad=True)
    xa, h = ln.split(x)
    ((xa * 2 + h * 3).sum() + (h ** 2).sum()).backward()
    g = x.grad.clone()
    x.grad = None
    h2 = F.layer_norm(x, (32,), ln.weight, ln.bias, ln.eps)
    ((x * 2 + h2 * 3).sum() + (h2 ** 2).sum()).backward()
    assert torch.allclose(g, x.grad, atol=1e-5)
