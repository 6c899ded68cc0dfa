"""tcgen05 GEMM (all three operand layouts, epilogue options) against fp32 PyTorch matmul."""
import pytest
import torch

from llm_distillery_b200.ops import basic, _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(a, b, a_mn, b_mn):
    A = (a.t() if a_mn else a).float()
    B = (b if b_mn else b.t()).float()
    return A @ B


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (384, 640, 200), (1000, 1000, 1000), (2048, 2560, 2048),
                                   (130, 72, 8)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(M * 7 + N * 3 + K)
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned row stride")
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV).bfloat16()
    out = basic.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert _lib.take_device_error() == 0
    r = _ref(a, b, a_mn, b_mn)
    tol = 1e-2 * max(1.0, r.abs().max().item())
    assert (out.float() - r).abs().max().item() <= tol


def test_gemm_epilogues():
    torch.manual_seed(5)
    a = torch.randn(300, 136, device=DEV).bfloat16()
    b = torch.randn(520, 136, device=DEV).bfloat16()
    r = a.float() @ b.float().t()
    # fp32 output, overwrite then accumulate
    c = torch.empty(300, 520, device=DEV)
    basic.gemm(a, b, out=c)
    assert torch.allclose(c, r, atol=1e-3, rtol=1e-3)
    basic.gemm(a, b, out=c, accumulate=True, alpha=0.5)
    assert torch.allclose(c, 1.5 * r, atol=2e-3, rtol=1e-3)
    # bf16 accumulate and residual
    rsd = torch.randn(300, 520, device=DEV).bfloat16()
    o = basic.gemm(a, b, residual=rsd)
    assert torch.allclose(o.float(), (r + rsd.float()), atol=0.15, rtol=2e-2)
    # fp16 operands
    o16 = basic.gemm(a.half(), b.half())
    assert torch.allclose(o16.float(), a.half().float() @ b.half().float().t(), atol=0.1, rtol=1e-2)
    # strided (row-padded) operands and output
    big = torch.randn(300, 256, device=DEV).bfloat16()
    outbig = torch.zeros(300, 1024, device=DEV, dtype=torch.bfloat16)
    basic.gemm(big[:, :136], b, out=outbig[:, 8:528])
    assert torch.allclose(outbig[:, 8:528].float(), big[:, :136].float() @ b.float().t(), atol=0.15, rtol=2e-2)
    assert outbig[:, :8].abs().max() == 0 and outbig[:, 528:].abs().max() == 0
    assert _lib.take_device_error() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(True, True), (False, False)])
def test_split_k_fp32_output_overwrite_accumulate_and_strided(a_mn, b_mn):
    """Long reduction, few tiles, fp32 output: the CTA-pair kernel splits K and adds the slices of a tile in the order
    of their index, so the result repeats bit for bit."""
    torch.manual_seed(11)
    M, N, K = 1280, 1000, 8192
    a = (torch.randn((K, M) if a_mn else (M, K), device=DEV) * 0.1).bfloat16()
    b = (torch.randn((K, N) if b_mn else (N, K), device=DEV) * 0.1).bfloat16()
    r = _ref(a, b, a_mn, b_mn)
    wide = torch.full((M, N + 24), 7.0, device=DEV)          # row-padded output: the memset must respect the stride
    c = wide[:, 8:8 + N]
    basic.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c)
    assert torch.allclose(c, r, atol=2e-2, rtol=2e-3), (c - r).abs().max()
    assert (wide[:, :8] == 7).all() and (wide[:, 8 + N:] == 7).all()
    first = c.clone()
    for _ in range(3):
        basic.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c)
        assert torch.equal(c, first)
    basic.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c, accumulate=True)
    assert torch.allclose(c, 2 * r, atol=4e-2, rtol=2e-3)
    assert _lib.take_device_error() == 0


def test_linear_helpers_match_autograd():
    torch.manual_seed(6)
    x = torch.randn(512, 256, device=DEV).bfloat16()
    w = torch.randn(384, 256, device=DEV).bfloat16() * 0.05
    dy = torch.randn(512, 384, device=DEV).bfloat16()
    xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
    (xf @ wf.t()).backward(dy.float())
    assert torch.allclose(basic.linear_fwd(x, w).float(), (x.float() @ w.float().t()), atol=5e-2, rtol=2e-2)
    assert torch.allclose(basic.linear_dgrad(dy, w).float(), xf.grad, atol=5e-2, rtol=2e-2)
    g = torch.zeros(384, 256, device=DEV)
    basic.linear_wgrad(dy, x, out=g, accumulate=True)
    assert torch.allclose(g, wf.grad, atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("T,f,K", [(1000, 1408, 512), (4096, 5632, 2048), (513, 128, 64), (2048, 1280, 200)])
def test_gate_up_gemm_with_swiglu_in_the_epilogue(T, f, K):
    """One launch writes gu = x W^T and act = silu(gate) * up; both must equal the two-kernel path bit for bit (act is
    computed from the rounded gate / up values), and nothing may be written outside the outputs."""
    torch.manual_seed(T + f)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(2 * f, K, device=DEV) * 0.05).bfloat16()
    gu, act = basic.linear_swiglu_fwd(x, w)
    assert _lib.take_device_error() == 0
    gu_ref = basic.linear_fwd(x, w)
    act_ref = basic.swiglu_fwd(gu_ref)
    assert torch.equal(gu, gu_ref)
    assert torch.equal(act, act_ref)
    r = x.float() @ w.float().t()
    assert torch.allclose(gu.float(), r, atol=2e-2 * max(1.0, r.abs().max().item()), rtol=2e-2)
    want = torch.nn.functional.silu(r[:, :f]) * r[:, f:]
    assert torch.allclose(act.float(), want, atol=3e-2 * max(1.0, want.abs().max().item()), rtol=3e-2)


@pytest.mark.parametrize("T,f,h", [(1000, 1408, 512), (4096, 5632, 2048), (513, 128, 64), (2048, 1280, 200)])
def test_down_projection_dgrad_with_swiglu_backward_in_the_epilogue(T, f, h):
    """dgu from one launch equals dgrad GEMM + SwiGLU backward kernel bit for bit (d(act) is rounded to bf16 before the
    activation's derivative is applied, exactly as when it is stored in between)."""
    torch.manual_seed(T + f + 1)
    dy = torch.randn(T, h, device=DEV).bfloat16()
    w_d = (torch.randn(h, f, device=DEV) * 0.05).bfloat16()
    gu = torch.randn(T, 2 * f, device=DEV).bfloat16()
    dgu = basic.linear_dgrad_swiglu_bwd(dy, w_d, gu)
    assert _lib.take_device_error() == 0
    dact = basic.linear_dgrad(dy, w_d)
    ref = basic.swiglu_bwd(gu, dact)
    assert torch.equal(dgu, ref)
    g, u, d = gu[:, :f].float(), gu[:, f:].float(), dy.float() @ w_d.float()
    sg = torch.sigmoid(g)
    want = torch.cat([d * u * (sg + g * sg * (1 - sg)), d * g * sg], 1)
    assert torch.allclose(dgu.float(), want, atol=3e-2 * max(1.0, want.abs().max().item()), rtol=3e-2)


@pytest.mark.parametrize("T,H,Hkv,d,K", [(1000, 8, 2, 64, 512), (4096, 32, 4, 64, 2048), (2048, 8, 2, 128, 1024),
                                         (513, 2, 1, 128, 64)])
def test_qkv_gemm_with_rotary_embedding_in_the_epilogue(T, H, Hkv, d, K):
    """One launch = GEMM + rope kernel, bit for bit; the value heads (the last Hkv) are stored unrotated."""
    torch.manual_seed(T + d)
    N = (H + 2 * Hkv) * d
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    L = 257
    pos = (torch.arange(T, device=DEV, dtype=torch.int32) * 7) % L
    cos, sin = basic.rope_tables(L, d, 10000.0, DEV)
    got = basic.linear_rope_fwd(x, w, pos, cos, sin, H + Hkv, d)
    assert _lib.take_device_error() == 0
    plain = basic.linear_fwd(x, w)
    ref = basic.rope_(plain.clone(), pos, cos, sin, H + Hkv, d)
    assert torch.equal(got, ref)
    assert torch.equal(got[:, (H + Hkv) * d:], plain[:, (H + Hkv) * d:])
    assert not torch.equal(got[:, : H * d], plain[:, : H * d])
