"""sm_100a elementwise / normalisation / optimizer kernels against their PyTorch fp32 restatements."""
import pytest
import torch

from llm_distillery_b200.ops import basic, _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cpu(fn, *args, **kw):
    """Run the oracle path of an op: same function, CPU tensors."""
    conv = [a.detach().cpu() if isinstance(a, torch.Tensor) else a for a in args]
    kwc = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    return fn(*conv, **kwc)


@pytest.mark.parametrize("rows,h", [(7, 256), (300, 2048), (5000, 2048), (2500, 1024), (77, 512), (64, 4096), (33, 8192)])
def test_rmsnorm_fwd_bwd(rows, h):
    torch.manual_seed(0)
    x = torch.randn(rows, h, device=DEV).bfloat16()
    res = torch.randn(rows, h, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(h, device=DEV)).bfloat16()
    for r in (None, res):
        y, hh, rstd = basic.rmsnorm_fwd(x, w, 1e-6, r)
        y0, h0, rstd0 = _cpu(basic.rmsnorm_fwd, x, w, 1e-6, r)
        assert torch.allclose(hh.float().cpu(), h0.float(), atol=1e-2, rtol=1e-2)
        assert torch.allclose(rstd.cpu(), rstd0, atol=1e-4, rtol=1e-3)
        assert torch.allclose(y.float().cpu(), y0.float(), atol=3e-2, rtol=2e-2)
        dy = torch.randn(rows, h, device=DEV).bfloat16()
        dres = torch.randn(rows, h, device=DEV).bfloat16()
        dh, dw = basic.rmsnorm_bwd(dy, hh, w, rstd, dres)
        dh0, dw0 = _cpu(basic.rmsnorm_bwd, dy, hh, w, rstd, dres)
        assert torch.allclose(dh.float().cpu(), dh0.float(), atol=5e-2, rtol=3e-2)
        assert torch.allclose(dw.cpu(), dw0, atol=5e-2 * rows ** 0.5, rtol=2e-2)
    # accumulate into an existing fp32 grad
    acc = torch.ones(h, device=DEV)
    basic.rmsnorm_bwd(dy, hh, w, rstd, None, dw_out=acc, dw_accumulate=True)
    _, dw1 = _cpu(basic.rmsnorm_bwd, dy, hh, w, rstd, None)
    assert torch.allclose(acc.cpu(), 1 + dw1, atol=5e-2 * rows ** 0.5, rtol=2e-2)


@pytest.mark.parametrize("T,nh,d", [(17, 4, 64), (300, 32, 64), (128, 8, 128)])
def test_rope_roundtrip_and_reference(T, nh, d):
    torch.manual_seed(1)
    width = nh * d + 2 * d  # extra columns must stay untouched
    x = torch.randn(T, width, device=DEV).bfloat16()
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    cos, sin = basic.rope_tables(512, d, 10000.0, DEV)
    ref = _cpu(basic.rope_, x.clone(), pos, cos, sin, nh, d)
    y = basic.rope_(x.clone(), pos, cos, sin, nh, d)
    assert torch.allclose(y.float().cpu(), ref.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(y[:, nh * d:], x[:, nh * d:])
    back = basic.rope_(y.clone(), pos, cos, sin, nh, d, inverse=True)
    assert torch.allclose(back.float(), x.float(), atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("T,nh,d,rot", [(33, 6, 128, 96), (300, 8, 64, 32), (17, 3, 80, 16)])
def test_partial_rope(T, nh, d, rot):
    """Only the first ``rot`` elements of a head rotate; the rest of the head and the columns past the heads stay."""
    torch.manual_seed(11)
    x = torch.randn(T, nh * d + 24, device=DEV).bfloat16()
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    cos, sin = basic.rope_tables(512, rot, 10000.0, DEV)
    ref = _cpu(basic.rope_, x.clone(), pos, cos, sin, nh, d)
    y = basic.rope_(x.clone(), pos, cos, sin, nh, d)
    assert torch.allclose(y.float().cpu(), ref.float(), atol=2e-2, rtol=2e-2)
    heads = y[:, : nh * d].view(T, nh, d)
    assert torch.equal(heads[..., rot:], x[:, : nh * d].view(T, nh, d)[..., rot:])
    assert torch.equal(y[:, nh * d:], x[:, nh * d:])
    back = basic.rope_(y.clone(), pos, cos, sin, nh, d, inverse=True)
    assert torch.allclose(back.float(), x.float(), atol=5e-2, rtol=5e-2)
    with pytest.raises(ValueError, match="multiple of 16"):
        basic.rope_(x.clone(), pos, *basic.rope_tables(512, 24, 10000.0, DEV), nh, d)


@pytest.mark.parametrize("T,f", [(5, 64), (257, 5632), (1024, 8192)])
def test_swiglu(T, f):
    torch.manual_seed(2)
    gu = torch.randn(T, 2 * f, device=DEV).bfloat16()
    d = torch.randn(T, f, device=DEV).bfloat16()
    a = basic.swiglu_fwd(gu)
    assert torch.allclose(a.float().cpu(), _cpu(basic.swiglu_fwd, gu).float(), atol=2e-2, rtol=2e-2)
    g = basic.swiglu_bwd(gu, d)
    assert torch.allclose(g.float().cpu(), _cpu(basic.swiglu_bwd, gu, d).float(), atol=3e-2, rtol=3e-2)


def test_embedding():
    torch.manual_seed(3)
    V, h, T = 1000, 256, 4096
    w = torch.randn(V, h, device=DEV).bfloat16()
    ids = torch.randint(0, V, (T,), device=DEV)
    out = basic.embed_fwd(ids, w)
    assert torch.equal(out, w[ids])
    dout = torch.randn(T, h, device=DEV).bfloat16()
    dw = torch.zeros(V, h, device=DEV)
    basic.embed_bwd(ids, dout, dw)
    ref = torch.zeros(V, h).index_add_(0, ids.cpu(), dout.float().cpu())
    assert torch.allclose(dw.cpu(), ref, atol=1e-3, rtol=1e-3)


def test_casts():
    x = torch.randn(100003, device=DEV)
    pad = torch.zeros(100008, device=DEV)
    pad[:100003] = x
    o = torch.empty(100008, device=DEV, dtype=torch.bfloat16)
    basic.cast_to_bf16(pad, o, 0.5)
    assert torch.equal(o, (pad * 0.5).bfloat16())
    acc = torch.ones(100008, device=DEV)
    basic.cast_to_f32(o, acc, 2.0, accumulate=True)
    assert torch.allclose(acc, 1 + o.float() * 2)
    assert _lib.take_device_error() == 0


@pytest.mark.parametrize("T,N", [(5, 64), (1000, 2560), (4097, 1152)])
def test_bias_add_and_grad(T, N):
    torch.manual_seed(4)
    wide = torch.randn(T, N + 16, device=DEV).bfloat16()       # row-padded view: the stride is not the width
    x = wide[:, :N]
    b = torch.randn(N, device=DEV).bfloat16()
    ref = (x.float() + b.float()).bfloat16()
    keep = wide[:, N:].clone()
    basic.bias_add_(x, b)
    assert torch.equal(x, ref) and torch.equal(wide[:, N:], keep)
    dy = torch.randn(T, N, device=DEV).bfloat16()
    g = basic.bias_grad(dy)
    r = dy.float().sum(0)
    assert torch.allclose(g, r, atol=2e-3 * T ** 0.5, rtol=1e-3)
    acc = torch.full((N,), 2.0, device=DEV)
    basic.bias_grad(dy, out=acc, accumulate=True)
    assert torch.allclose(acc, r + 2.0, atol=2e-3 * T ** 0.5, rtol=1e-3)
    basic.bias_grad(dy, out=acc, accumulate=False)
    assert torch.allclose(acc, r, atol=2e-3 * T ** 0.5, rtol=1e-3)


@pytest.mark.parametrize("T,H,Hkv,d", [(37, 4, 2, 64), (1000, 8, 2, 128), (5000, 16, 4, 128), (3, 2, 1, 64)])
def test_per_head_qk_norm_fwd_bwd(T, H, Hkv, d):
    """Qwen3's q_norm / k_norm on fused qkv rows: kernels against the fp32 restatement of the same function."""
    torch.manual_seed(T + d)
    cols = (H + 2 * Hkv) * d
    qkv = torch.randn(T, cols, device=DEV).bfloat16()
    wq = (1 + 0.2 * torch.randn(d, device=DEV)).bfloat16()
    wk = (1 + 0.2 * torch.randn(d, device=DEV)).bfloat16()
    y, rstd = basic.headnorm_fwd(qkv, wq, wk, H, Hkv, d, 1e-6)
    y_ref, rstd_ref = _cpu(basic.headnorm_fwd, qkv.float(), wq.float(), wk.float(), H, Hkv, d, 1e-6)
    assert torch.allclose(rstd.cpu(), rstd_ref, rtol=1e-4, atol=1e-5)
    assert torch.allclose(y.float().cpu(), y_ref, atol=3e-2, rtol=2e-2)
    assert torch.equal(y[:, (H + Hkv) * d:], qkv[:, (H + Hkv) * d:])          # value heads are copied bit for bit
    g = torch.randn(T, cols, device=DEV).bfloat16()
    g_ref = g.float().cpu().clone()
    g_in = g.clone()
    dwq, dwk = basic.headnorm_bwd_(g, qkv, wq, wk, rstd, H, Hkv, d)
    dwq_ref, dwk_ref = basic.headnorm_bwd_(g_ref, qkv.float().cpu(), wq.float().cpu(), wk.float().cpu(), rstd.cpu(), H, Hkv, d)
    assert torch.allclose(g.float().cpu(), g_ref, atol=4e-2, rtol=3e-2)
    assert torch.equal(g[:, (H + Hkv) * d:], g_in[:, (H + Hkv) * d:])
    scale = max(1.0, float(dwq_ref.abs().max()))
    assert torch.allclose(dwq.cpu(), dwq_ref, atol=2e-2 * scale, rtol=2e-2)
    assert torch.allclose(dwk.cpu(), dwk_ref, atol=2e-2 * scale, rtol=2e-2)
    assert _lib.take_device_error() == 0
