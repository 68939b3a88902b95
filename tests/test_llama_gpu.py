"""Rotary / SwiGLU kernels and a small Llama block against fp32 PyTorch references (GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("H,D,S", [(4, 64, 33), (2, 128, 128)])
def test_rope_and_inverse(H, D, S):
    from necklace_b200.ops.rotary import _apply, _rope_ref
    torch.manual_seed(0)
    qkv = torch.randn(2, S, 3 * H * D, device="cuda").bfloat16()
    ref = _rope_ref(qkv.float(), H, 10000.0, 1.0)
    got = _apply(qkv.clone(), H, 10000.0, False, 0)
    assert _rel(got, ref) < 1e-2
    back = _apply(got.clone(), H, 10000.0, True, 0)
    assert _rel(back, qkv) < 1e-2
    assert torch.equal(got[..., 2 * H * D:], qkv[..., 2 * H * D:])  # v untouched


def test_swiglu_fwd_bwd():
    from necklace_b200.ops.rotary import swiglu
    torch.manual_seed(1)
    gu = torch.randn(5, 37, 2 * 256, device="cuda").bfloat16().requires_grad_(True)
    dh = torch.randn(5, 37, 256, device="cuda").bfloat16()
    h = swiglu(gu)
    h.backward(dh)
    r = gu.detach().float().requires_grad_(True)
    hr = torch.nn.functional.silu(r[..., :256]) * r[..., 256:]
    hr.backward(dh.float())
    assert _rel(h, hr) < 1e-2 and _rel(gu.grad, r.grad) < 2e-2


def test_tiny_llama_trains_and_matches_cpu_fp32():
    from necklace_b200.models.llama import Llama, LlamaConfig
    from necklace_b200.ops import check_status
    cfg = LlamaConfig(n_layer=2, d_model=256, n_head=4, d_ff=512, vocab=1000, max_seq=128)
    gpu = Llama(cfg, device="cuda")
    cfg32 = LlamaConfig(n_layer=2, d_model=256, n_head=4, d_ff=512, vocab=1000, max_seq=128,
                        dtype=torch.float32)
    cpu = Llama(cfg32)
    with torch.no_grad():
        for a, b in zip(cpu.parameters(), gpu.parameters()):
            a.copy_(b.float().cpu())
    tok = torch.randint(0, 1000, (2, 129))
    l_gpu = gpu(tok[:, :-1].cuda(), tok[:, 1:].cuda())
    l_cpu = cpu(tok[:, :-1], tok[:, 1:])
    l_gpu.backward()
    l_cpu.backward()
    check_status()
    assert abs(float(l_gpu) - float(l_cpu)) < 5e-2
    for (n, a), b in zip(cpu.named_parameters(), gpu.parameters()):
        assert _rel(b.grad.cpu(), a.grad) < 8e-2, n
