"""GPU parity tests of the rotation and trapezoidal-coefficient operators against the oracle's eager
definitions (pinned bit-exactly to the reference's own, tests/golden/PINNING.txt).  Shapes, seeds' structure and
tolerances follow the reference's tests (tests/kernels/test_rope.py:51-260, tests/kernels/test_trapezoidal.py:
37-150): fp32 forward 1e-5 absolute, bf16 forward 1e-2 absolute and no worse than eager bf16, gradients 1e-3.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

ROPE_SHAPES = [(2, 256, 8, 16), (4, 512, 8, 32), (1, 1024, 4, 8), (2, 128, 64, 128), (1, 64, 3, 6)]
TRAP_SHAPES = [(2, 256, 8), (4, 1024, 8), (1, 2048, 16), (16, 4096, 64), (3, 50, 24)]


def _rope_inputs(B, T, H, D, dtype, seed=0, ang_scale=2.0, per_head=False):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(B, T, H, D, generator=g, device=DEV, dtype=dtype)
    angles = torch.randn(B, T, H if per_head else 1, D // 2, generator=g, device=DEV, dtype=dtype) * ang_scale
    return x, angles


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("shape", ROPE_SHAPES)
def test_rope_forward_fp32(pkg, cabi, oracle, shape, per_head):
    x, angles = _rope_inputs(*shape, torch.float32, per_head=per_head)
    y = pkg.fused_rope(x, angles)
    assert y.shape == x.shape and y.dtype == x.dtype
    assert (y - oracle.apply_rope(x, angles)).abs().max().item() < 1e-5


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("shape", ROPE_SHAPES[:4])
def test_rope_forward_bf16(pkg, cabi, oracle, shape, per_head):
    B, T, H, D = shape
    g = torch.Generator(device=DEV).manual_seed(0)
    x_bf = (torch.randn(B, T, H, D, generator=g, device=DEV) * 0.5).bfloat16()
    a_bf = torch.randn(B, T, H if per_head else 1, D // 2, generator=g, device=DEV).bfloat16()
    y_oracle = oracle.apply_rope(x_bf.float(), a_bf.float())
    err_eager = (oracle.apply_rope(x_bf, a_bf).float() - y_oracle).abs().max().item()
    y = pkg.fused_rope(x_bf, a_bf)
    assert y.dtype == torch.bfloat16
    err = (y.float() - y_oracle).abs().max().item()
    assert err < 1e-2 and err <= err_eager + 1e-3, (err, err_eager)


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("shape", ROPE_SHAPES)
def test_rope_backward_fp32(pkg, cabi, oracle, shape, per_head):
    x, angles = _rope_inputs(*shape, torch.float32, seed=42, per_head=per_head)
    g = torch.randn_like(x)
    xr, ar = x.clone().requires_grad_(True), angles.clone().requires_grad_(True)
    oracle.apply_rope(xr, ar).backward(g)
    xk, ak = x.clone().requires_grad_(True), angles.clone().requires_grad_(True)
    pkg.fused_rope(xk, ak).backward(g)
    assert ak.grad.shape == angles.shape
    assert (xk.grad - xr.grad).abs().max().item() < 1e-3
    # the broadcast case sums over heads: compare relative to the size of the sum
    scale = max(1.0, ar.grad.abs().max().item())
    assert (ak.grad - ar.grad).abs().max().item() < 1e-3 * scale


def test_rope_rejects_bad_inputs(pkg, cabi):
    x = torch.zeros(1, 4, 2, 6, device=DEV)
    with pytest.raises(AssertionError):
        pkg.fused_rope(x, torch.zeros(1, 4, 3, 3, device=DEV))      # neither 1 nor H heads
    with pytest.raises(AssertionError):
        pkg.fused_rope(torch.zeros(1, 4, 2, 5, device=DEV), torch.zeros(1, 4, 1, 2, device=DEV))  # odd last dim
    with pytest.raises(AssertionError):
        pkg.fused_rope(x.cpu(), torch.zeros(1, 4, 1, 3))            # CPU tensors


def _trap_inputs(B, T, H, dtype, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    dt_raw = (torch.randn(B, T, H, generator=g, device=DEV) * 0.5).to(dtype)
    lam_raw = (torch.randn(B, T, H, generator=g, device=DEV) * 0.5).to(dtype)
    dt_bias = (torch.randn(H, generator=g, device=DEV) * 0.1).to(dtype)
    A_log = (torch.randn(H, generator=g, device=DEV) * 0.1).to(dtype)
    return dt_raw, lam_raw, dt_bias, A_log


@pytest.mark.parametrize("shape", TRAP_SHAPES)
def test_trapezoidal_forward_fp32(pkg, cabi, oracle, shape):
    ins = _trap_inputs(*shape, torch.float32)
    outs = pkg.fused_trapezoidal(*ins)
    for got, ref in zip(outs, oracle.trapezoid_from_raw(*ins)):
        assert got.shape == ins[0].shape and got.dtype == torch.float32
        assert (got - ref).abs().max().item() < 1e-5


@pytest.mark.parametrize("shape", TRAP_SHAPES[:4])
def test_trapezoidal_forward_bf16(pkg, cabi, oracle, shape):
    ins = _trap_inputs(*shape, torch.bfloat16)
    outs = pkg.fused_trapezoidal(*ins)
    refs = oracle.trapezoid_from_raw(*[t.float() for t in ins])
    for got, ref in zip(outs, refs):
        assert got.dtype == torch.bfloat16
        assert (got.float() - ref).abs().max().item() < 1e-2


@pytest.mark.parametrize("shape", TRAP_SHAPES)
def test_trapezoidal_backward_fp32(pkg, cabi, oracle, shape):
    ins = _trap_inputs(*shape, torch.float32, seed=7)
    gs = [torch.randn_like(ins[0]) for _ in range(4)]
    lr = [t.clone().requires_grad_(True) for t in ins]
    gr = torch.autograd.grad(list(oracle.trapezoid_from_raw(*lr)), lr, gs)
    lk = [t.clone().requires_grad_(True) for t in ins]
    gk = torch.autograd.grad(list(pkg.fused_trapezoidal(*lk)), lk, gs)
    for name, a, b in zip(("d_dt_raw", "d_lam_raw", "d_dt_bias", "d_A_log"), gk, gr):
        scale = max(1.0, b.abs().max().item())   # the parameter gradients are sums over all rows
        assert (a - b).abs().max().item() < 1e-3 * scale, name
    # deterministic reductions
    gk2 = torch.autograd.grad(list(pkg.fused_trapezoidal(*lk)), lk, gs)
    assert all(torch.equal(a, b) for a, b in zip(gk, gk2))


def test_trapezoidal_rejects_bad_inputs(pkg, cabi):
    dt_raw = torch.zeros(2, 8, 4, device=DEV)
    with pytest.raises(AssertionError):
        pkg.fused_trapezoidal(dt_raw, torch.zeros(2, 8, 5, device=DEV), torch.zeros(4, device=DEV), torch.zeros(4, device=DEV))
    with pytest.raises(AssertionError):
        pkg.fused_trapezoidal(dt_raw, dt_raw, torch.zeros(3, device=DEV), torch.zeros(4, device=DEV))
    with pytest.raises(AssertionError):
        pkg.fused_trapezoidal(dt_raw.cpu(), dt_raw.cpu(), torch.zeros(4), torch.zeros(4))


NORM_SHAPES = [(2, 256, 128), (4, 512, 256), (1, 1024, 96), (2, 64, 4, 32), (1, 128, 8, 16), (2, 64, 4096), (3, 7, 50)]
EPS = 1e-6


def _eager_rmsnorm(x, w, eps=EPS):
    """The reference tests' eager definition (tests/kernels/test_rmsnorm.py:35-38)."""
    return torch.nn.functional.rms_norm(x, (x.shape[-1],), w.to(x.dtype), eps)


@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_rmsnorm_forward_fp32(pkg, cabi, shape):
    torch.manual_seed(0)
    x = torch.randn(*shape, device=DEV)
    w = torch.randn(shape[-1], device=DEV) * 0.5 + 1.0
    y = pkg.fused_rmsnorm(x, w, EPS)
    assert y.shape == x.shape and y.dtype == x.dtype
    assert (y - _eager_rmsnorm(x, w)).abs().max().item() < 1e-5


@pytest.mark.parametrize("shape", NORM_SHAPES[:6])
def test_rmsnorm_forward_bf16(pkg, cabi, shape):
    torch.manual_seed(1)
    x = torch.randn(*shape, device=DEV).bfloat16()
    w = (torch.randn(shape[-1], device=DEV) * 0.5 + 1.0).bfloat16()
    y = pkg.fused_rmsnorm(x, w, EPS)
    assert y.dtype == torch.bfloat16
    assert (y.float() - _eager_rmsnorm(x.float(), w.float())).abs().max().item() < 1e-2 * 4  # |y| reaches ~4 here; bf16 ulp scales


@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_rmsnorm_backward_fp32(pkg, cabi, shape):
    torch.manual_seed(3)
    x = torch.randn(*shape, device=DEV)
    w = torch.randn(shape[-1], device=DEV) * 0.5 + 1.0
    g = torch.randn(*shape, device=DEV)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    _eager_rmsnorm(xr, wr).backward(g)
    xk, wk = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    pkg.fused_rmsnorm(xk, wk, EPS).backward(g)
    assert (xk.grad - xr.grad).abs().max().item() < 1e-3
    assert (wk.grad - wr.grad).abs().max().item() < 1e-3 * max(1.0, wr.grad.abs().max().item())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 5e-2)])
@pytest.mark.parametrize("shape", [(2, 128, 4096), (2, 64, 256), (1, 33, 96)])
def test_gate_norm_matches_block_epilogue(pkg, cabi, shape, dtype, tol):
    """norm(y) * silu(z) as the block composes it (src/mamba_base_engine.py:189-191), forward and gradients."""
    torch.manual_seed(5)
    y = torch.randn(*shape, device=DEV).to(dtype)
    z = torch.randn(*shape, device=DEV).to(dtype)
    w = torch.randn(shape[-1], device=DEV) * 0.5 + 1.0
    g = torch.randn(*shape, device=DEV).to(dtype)
    lr = [t.float().clone().requires_grad_(True) for t in (y, z, w)]
    ref = _eager_rmsnorm(lr[0], lr[2]) * torch.nn.functional.silu(lr[1])
    gr = torch.autograd.grad([ref], lr, [g.float()])
    lk = [t.clone().requires_grad_(True) for t in (y, z, w)]
    out = pkg.fused_gate_norm(lk[0], lk[1], lk[2], EPS)
    gk = torch.autograd.grad([out], lk, [g])
    assert out.dtype == dtype
    assert (out.float() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
    gtol = 1e-3 if dtype == torch.float32 else 5e-2
    for name, a, b in zip(("dy", "dz", "dw"), gk, gr):
        assert (a.float() - b).abs().max().item() < gtol * max(1.0, b.abs().max().item()), name


def test_rmsnorm_module_swap(pkg, cabi):
    torch.manual_seed(6)
    ref = torch.nn.RMSNorm(128, eps=EPS).to(DEV)
    with torch.no_grad():
        ref.weight.copy_(torch.randn(128, device=DEV) * 0.5 + 1.0)
    mod = pkg.FusedRMSNormModule(128, EPS).to(DEV)
    with torch.no_grad():
        mod.weight.copy_(ref.weight)
    x = torch.randn(4, 64, 128, device=DEV)
    assert (mod(x) - ref(x)).abs().max().item() < 1e-5
    # three-argument apply, as the reference's module calls it, and its backward
    xk = x.clone().requires_grad_(True)
    pkg.FusedRMSNorm.apply(xk, mod.weight, EPS).sum().backward()
    assert xk.grad is not None and mod.weight.grad is not None
