"""Guard-band checks: kernels that write into caller-provided memory must not touch a byte outside it.

Every output lives in the middle of a larger allocation whose head and tail are filled with a marker value; after the
kernel the marker must still be there. Shapes have tails in every tiled dimension (rows and columns that are no
multiple of the 128-wide tiles, element counts that are no multiple of the vector width), because that is where a
missing bound shows. This stands in for a memory checker, which the pool does not offer.
"""
import pytest
import torch

from llm_distillery_b200.engine.optim import FlatOptimizer, FlatParams
from llm_distillery_b200.ops import basic, _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"
MARK = 1536.0          # exactly representable in bf16, fp16 and fp32
PAD = 8192             # elements on each side (keeps the payload 16 KiB-aligned for every dtype used here)


def guarded(shape, dtype, fill=None):
    n = 1
    for s in shape:
        n *= s
    big = torch.full((n + 2 * PAD,), MARK, dtype=dtype, device=DEV)
    view = big[PAD:PAD + n].view(shape)
    if fill is not None:
        view.copy_(fill)
    return big, view


def intact(big, view) -> bool:
    n = view.numel()
    return bool((big[:PAD] == MARK).all() and (big[PAD + n:] == MARK).all())


@pytest.mark.parametrize("M,N,K", [(300, 200, 136), (130, 72, 8), (1000, 1000, 1000), (129, 136, 4104)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gemm_output_stays_inside(M, N, K, dtype):
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    big, out = guarded((M, N), dtype)
    basic.gemm(a, b, out=out)
    torch.cuda.synchronize()
    assert _lib.take_device_error() == 0
    assert intact(big, out)
    r = a.float() @ b.float().t()
    assert (out.float() - r).abs().max().item() <= 2e-2 * max(1.0, r.abs().max().item())


@pytest.mark.parametrize("T,N,K", [(2048, 200, 136), (4096, 264, 520), (16384, 128, 256)])
def test_weight_gradient_accumulation_stays_inside(T, N, K):
    """fp32 accumulate (+=), including the shapes that take the split-K path (atomic adds into the output)."""
    torch.manual_seed(T + N)
    dy = torch.randn(T, N, device=DEV).bfloat16()
    x = torch.randn(T, K, device=DEV).bfloat16()
    big, out = guarded((N, K), torch.float32, fill=torch.ones(N, K, device=DEV))
    basic.linear_wgrad(dy, x, out=out, accumulate=True)
    torch.cuda.synchronize()
    assert _lib.take_device_error() == 0
    assert intact(big, out)
    r = dy.float().t() @ x.float() + 1.0
    assert (out - r).abs().max().item() <= 2e-2 * max(1.0, r.abs().max().item())


@pytest.mark.parametrize("rows,h", [(1000, 2048), (37, 4096), (513, 1024), (5, 8192)])
def test_rmsnorm_and_bias_outputs_stay_inside(rows, h):
    torch.manual_seed(rows)
    x = torch.randn(rows, h, device=DEV).bfloat16()
    w = torch.randn(h, device=DEV).bfloat16()
    big, out = guarded((rows, h), torch.bfloat16)
    y, _, rstd = basic.rmsnorm_fwd(x, w, 1e-5, out=out)
    torch.cuda.synchronize()
    assert intact(big, out)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert (y.float() - ref).abs().max().item() < 0.1
    bigb, outb = guarded((h,), torch.float32)
    basic.bias_grad(x, out=outb)
    torch.cuda.synchronize()
    assert intact(bigb, outb)
    assert torch.allclose(outb, x.float().sum(0), atol=0.5, rtol=1e-2)
    bigx, xin = guarded((rows, h), torch.bfloat16, fill=x)
    basic.bias_add_(xin, w)
    torch.cuda.synchronize()
    assert intact(bigx, xin)
    assert _lib.take_device_error() == 0


def test_rope_in_place_stays_inside():
    B, L, H, Hkv, d = 2, 77, 4, 2, 64
    width = (H + 2 * Hkv) * d
    torch.manual_seed(3)
    src = torch.randn(B * L, width, device=DEV).bfloat16()
    big, qkv = guarded((B * L, width), torch.bfloat16, fill=src)
    cos, sin = basic.rope_tables(128, d, 10000.0, DEV)
    pos = torch.arange(L, dtype=torch.int32, device=DEV).repeat(B)
    basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
    torch.cuda.synchronize()
    assert intact(big, qkv)
    assert torch.equal(qkv[:, (H + Hkv) * d:], src[:, (H + Hkv) * d:])      # v columns are not rotated
    assert _lib.take_device_error() == 0


def test_embedding_gradient_and_casts_stay_inside():
    V, h, T = 1000, 264, 777
    torch.manual_seed(4)
    ids = torch.randint(0, V, (T,), device=DEV)
    dout = torch.randn(T, h, device=DEV).bfloat16()
    big, dw = guarded((V, h), torch.float32, fill=torch.zeros(V, h, device=DEV))
    basic.embed_bwd(ids, dout, dw)
    torch.cuda.synchronize()
    assert intact(big, dw)
    ref = torch.zeros(V, h, device=DEV).index_add_(0, ids, dout.float())
    assert torch.allclose(dw, ref, atol=1e-2, rtol=1e-2)
    n = 100003                                                             # odd: exercises the scalar tail of the casts
    src = torch.randn(n, device=DEV)
    bigc, dst = guarded((n,), torch.bfloat16)
    basic.cast_to_bf16(src, dst, 0.5)
    bigf, dstf = guarded((n,), torch.float32, fill=torch.ones(n, device=DEV))
    basic.cast_to_f32(dst, dstf, 2.0, accumulate=True)
    torch.cuda.synchronize()
    assert intact(bigc, dst) and intact(bigf, dstf)
    assert torch.allclose(dstf, 1.0 + 2.0 * (src * 0.5).bfloat16().float(), atol=1e-3)
    assert _lib.take_device_error() == 0


@pytest.mark.parametrize("name", ["adamw", "adamw8bit", "sgd", "rmsprop", "adagrad"])
def test_optimizer_kernels_stay_inside_the_flat_buffers(name):
    torch.manual_seed(6)
    ps = [torch.nn.Parameter(torch.randn(s, device=DEV).bfloat16()) for s in ((37, 129), (1000,), (64, 64))]
    total = sum((p.numel() + 63) // 64 * 64 for p in ps)
    total = (total + 255) // 256 * 256
    bigm, model = guarded((total,), torch.bfloat16, fill=torch.zeros(total, device=DEV))
    bigg, grad = guarded((total,), torch.float32, fill=torch.zeros(total, device=DEV))
    flat = FlatParams(ps, buffers={"model": model, "grad": grad})
    assert flat.total == total
    opt = FlatOptimizer(flat, name, lr=1e-2)
    before = model.clone()
    for s in flat.slots:
        s.buf.normal_()
        s.fresh = False
    opt.step()
    opt.step()
    torch.cuda.synchronize()
    assert intact(bigm, model) and intact(bigg, grad)
    assert not torch.equal(before, model)
    assert _lib.take_device_error() == 0
