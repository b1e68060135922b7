"""Size-independent properties at the benchmark's full sizes (where the CPU oracle cannot follow):
statistics of the normalised rows, linearity of the backward in dy, scale invariance of RMSNorm,
shift invariance of LayerNorm and Softmax, rows of Softmax summing to one, idempotence of normalize.
Each holds to rounding of the storage type; the bars are those of the parity tests."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from b200norm import functional as Fn
from b200norm import ops as P
from b200norm import softmax as S

DEV = "cuda:0"


def draw(M, N, dtype, seed, mu=0.0, sigma=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    out = torch.empty((M, N), device=DEV, dtype=dtype)
    step = max(1, (1 << 26) // N)
    for r in range(0, M, step):
        e = min(M, r + step)
        out[r:e] = (torch.randn((e - r, N), device=DEV, generator=g) * sigma + mu).to(dtype)
    return out


def close(a, b, tol, what):
    """max|a - b| <= tol * max|b|, evaluated in chunks of rows in fp32."""
    err = scale = 0.0
    step = max(1, (1 << 26) // a.shape[-1])
    for r in range(0, a.shape[0], step):
        x, y = a[r:r + step].float(), b[r:r + step].float()
        err = max(err, (x - y).abs().max().item())
        scale = max(scale, y.abs().max().item())
    assert err <= tol * scale, f"{what}: {err:.3e} > {tol:.1e} * {scale:.3e}"


# (M, N, dtype, tolerance): c2's and c4's shapes, and an fp32 one
SHAPES = [(32768, 4096, torch.bfloat16, 1e-2), (32768, 16384, torch.bfloat16, 1e-2), (16384, 5120, torch.float32, 1e-5)]


@pytest.mark.parametrize("M,N,dtype,tol", SHAPES)
def test_normalised_rows_have_zero_mean_and_unit_power(M, N, dtype, tol):
    x = draw(M, N, dtype, 0, mu=3.0, sigma=2.0)
    y, mean, rstd = Fn._layernorm_fwd(x, None, None, 1e-6)
    yr, rstd_r = Fn._rmsnorm_fwd(x, None, 1e-6)
    rows = torch.arange(0, M, max(1, M // 4096), device=DEV)
    ys, yrs = y[rows].float(), yr[rows].float()
    assert ys.mean(-1).abs().max().item() <= 10 * tol          # mean 0 (each element carries a rounding of `tol`)
    assert (ys.pow(2).mean(-1) - 1).abs().max().item() <= 4 * tol + 1e-4
    assert (yrs.pow(2).mean(-1) - 1).abs().max().item() <= 4 * tol + 1e-4
    xs = x[rows].float()
    torch.testing.assert_close(mean[rows], xs.mean(-1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rstd[rows], (xs.var(-1, unbiased=False) + 1e-6).rsqrt(), rtol=2e-5, atol=0)
    torch.testing.assert_close(rstd_r[rows], (xs.pow(2).mean(-1) + 1e-6).rsqrt(), rtol=2e-5, atol=0)


@pytest.mark.parametrize("M,N,dtype,tol", SHAPES)
@pytest.mark.parametrize("rms", [False, True])
def test_backward_is_linear_in_dy(M, N, dtype, tol, rms):
    x, d1, d2 = draw(M, N, dtype, 1), draw(M, N, dtype, 2), draw(M, N, dtype, 3)
    w = (1 + 0.1 * torch.randn(N, device=DEV)).to(dtype)
    b = None if rms else (0.1 * torch.randn(N, device=DEV)).to(dtype)
    if rms:
        _, rstd = Fn._rmsnorm_fwd(x, w, 1e-6)
        bwd = lambda dy: Fn._rmsnorm_bwd(x, dy, w, rstd, 1e-6)
    else:
        _, mean, rstd = Fn._layernorm_fwd(x, w, b, 1e-6)
        bwd = lambda dy: Fn._layernorm_bwd(x, dy, w, b, mean, rstd, 1e-6)
    r1, r2, r12 = bwd(d1), bwd(d2), bwd((d1.float() + d2.float()).to(dtype))
    # d1 + d2 is itself rounded to the storage type: one more rounding than the parity bar
    close(r12[0], (r1[0].float() + r2[0].float()), 3 * tol, "dx")
    for k in range(1, 2 if rms else 3):
        close(r12[k].float().unsqueeze(0), (r1[k].float() + r2[k].float()).unsqueeze(0), 3 * tol, "dw/db")


@pytest.mark.parametrize("M,N,dtype,tol", SHAPES)
def test_scale_and_shift_invariances(M, N, dtype, tol):
    x = draw(M, N, dtype, 4)
    w = (1 + 0.1 * torch.randn(N, device=DEV)).to(dtype)
    # powers of two scale x exactly in every storage type; with eps = 0 RMSNorm does not see the scale
    y1, _ = Fn._rmsnorm_fwd(x, w, 0.0)
    y2, _ = Fn._rmsnorm_fwd(x * 4, w, 0.0)
    close(y2, y1, tol, "rmsnorm(4x) vs rmsnorm(x)")
    # LayerNorm does not see a shift of the row (checked in fp32 storage, where x + 8 is nearly exact)
    if dtype == torch.float32:
        z1 = Fn._layernorm_fwd(x, w, None, 1e-6)[0]
        z2 = Fn._layernorm_fwd(x + 8, w, None, 1e-6)[0]
        close(z2, z1, 5e-5, "layernorm(x + 8) vs layernorm(x)")
        s1, s2 = S._fwd(x, False), S._fwd(x + 8, False)
        close(s2, s1, 5e-5, "softmax(x + 8) vs softmax(x)")


@pytest.mark.parametrize("M,N,dtype,tol", SHAPES)
def test_softmax_rows_sum_to_one_and_normalize_is_idempotent(M, N, dtype, tol):
    x = draw(M, N, dtype, 5, sigma=3.0)
    y = S._fwd(x, False)
    rows = torch.arange(0, M, max(1, M // 4096), device=DEV)
    sums = y[rows].float().sum(-1)
    assert (sums - 1).abs().max().item() <= tol * 2
    ly = S._fwd(x, True)
    assert (ly[rows].float().exp().sum(-1) - 1).abs().max().item() <= tol * 8
    x3 = x.unsqueeze(0)
    n1, _ = P._normalize_fwd(x3, 2, 1e-12)
    n2, norms2 = P._normalize_fwd(n1, 2, 1e-12)
    close(n2[0], n1[0], tol, "normalize(normalize(x)) vs normalize(x)")
    assert (norms2.float() - 1).abs().max().item() <= 2 * tol
    # the backward of normalize is orthogonal to the output: sum_k y_k * dx_k = 0 for p = 2
    g = draw(M, N, dtype, 6).unsqueeze(0)
    _, norms = P._normalize_fwd(x3, 2, 1e-12)
    dx = P._normalize_bwd(x3, n1, norms, g, 2)
    dots = (n1[0][rows].float() * dx[0][rows].float()).sum(-1).abs()
    scale = (dx[0][rows].float().abs().sum(-1) * n1[0][rows].float().abs().max(-1).values).clamp_min(1e-30)
    assert (dots / scale).max().item() <= 4 * tol
