"""tcgen05 GEMM against a plain PyTorch fp32 reference (one GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, bias=None):
    out = a.float() @ b.float().t()
    if bias is not None:
        out = out + bias.float()
    return out


# The second line are shapes whose last round of tiles is cut into column pieces on a 148-SM GPU: 448 tiles (4 left:
# 32-column pieces), 512 tiles (68 left: 128-column pieces), 474 tiles (30 left: 64-column pieces), 149 tiles with
# a ragged N (pieces that start beyond N), 150 tiles.
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 128), (1024, 1792, 4096), (384, 200, 72),
                                   (100, 40, 8), (8192, 4096, 1792),
                                   (8192, 1792, 512), (4096, 4096, 256), (10112, 1536, 64), (19072, 200, 72),
                                   (3840, 1280, 128)])
def test_gemm_matches_fp32_reference(shape):
    from nano_nccl_b200.ops.gemm import gemm_bf16, gemm_last_error

    m, n, k = shape
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16() if n % 2 == 0 else None
    out = gemm_bf16(a, b, bias)
    torch.cuda.synchronize()
    assert gemm_last_error() == 0
    want = _ref(a, b, bias)
    err = (out.float() - want).abs()
    tol = 1e-2 * want.abs().clamp(min=1.0)  # bf16 output rounding
    assert bool((err <= tol).all()), f"max err {err.max().item()} at shape {shape}"


def test_gemm_guard_rows_untouched():
    """Partial tiles must not write outside [M, N]."""
    from nano_nccl_b200.ops.gemm import gemm_bf16

    m, n, k = 200, 264, 64
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    full = torch.full((m + 2, n), -9137.25, device="cuda").bfloat16()
    gemm_bf16(a, b, out=full[1:m + 1])
    torch.cuda.synchronize()
    assert (full[0] == full[0, 0]).all() and (full[-1] == full[0, 0]).all()
    want = _ref(a, b)
    assert bool(((full[1:m + 1].float() - want).abs() <= 0.02 * want.abs().clamp(min=1)).all())


def test_nano_linear_matches_torch_linear():
    import torch.nn as nn

    from nano_nccl_b200.ops.linear import NanoLinear

    torch.manual_seed(0)
    ref = nn.Linear(256, 384).cuda().bfloat16()
    mine = NanoLinear(256, 384).cuda().bfloat16()
    mine.load_state_dict(ref.state_dict())
    x1 = torch.randn(4, 64, 256, device="cuda").bfloat16().requires_grad_()
    x2 = x1.detach().clone().requires_grad_()
    y1, y2 = ref(x1), mine(x2)
    assert bool(((y1.float() - y2.float()).abs() <= 2e-2 * y1.float().abs().clamp(min=1)).all())
    y1.float().square().mean().backward()
    y2.float().square().mean().backward()
    for a, b in [(x1.grad, x2.grad), (ref.weight.grad, mine.weight.grad), (ref.bias.grad, mine.bias.grad)]:
        assert bool(((a.float() - b.float()).abs() <= 3e-2 * a.float().abs().max().clamp(min=1e-3)).all())
