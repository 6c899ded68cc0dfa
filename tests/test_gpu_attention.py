"""sm_100a flash attention (forward and backward) against the fp32 PyTorch restatement."""
import pytest
import torch

from llm_distillery_b200.ops import attention, _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"

CASES = [(1, 128, 1, 1, 64), (1, 128, 2, 1, 64), (2, 256, 4, 2, 64), (2, 384, 8, 2, 64), (1, 200, 4, 4, 64), (3, 1024, 4, 1, 64),
         (1, 128, 2, 1, 128), (2, 320, 4, 2, 128), (1, 1024, 8, 2, 128)]


@pytest.mark.parametrize("B,L,H,Hkv,d", CASES)
def test_flash_fwd(B, L, H, Hkv, d):
    torch.manual_seed(B * 1000 + L + d)
    qkv = (torch.randn(B * L, (H + 2 * Hkv) * d, device=DEV) * 1.5).bfloat16()
    out, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d)
    assert _lib.take_device_error() == 0
    ro, rl = attention.attention_reference_fwd(qkv.float(), B, L, H, Hkv, d)
    assert torch.allclose(lse, rl, atol=2e-2, rtol=1e-3), (lse - rl).abs().max()
    assert torch.allclose(out.float(), ro, atol=3e-2, rtol=3e-2), (out.float() - ro).abs().max()


@pytest.mark.parametrize("B,L,H,Hkv,d", CASES)
def test_flash_bwd(B, L, H, Hkv, d):
    torch.manual_seed(B * 77 + L + d)
    qkv = (torch.randn(B * L, (H + 2 * Hkv) * d, device=DEV)).bfloat16()
    dout = torch.randn(B * L, H * d, device=DEV).bfloat16()
    out, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d)
    dqkv = attention.attention_bwd(dout, qkv, out, lse, B, L, H, Hkv, d)
    assert _lib.take_device_error() == 0
    ro, rl = attention.attention_reference_fwd(qkv.float(), B, L, H, Hkv, d)
    ref = attention.attention_reference_bwd(dout.float(), qkv.float(), ro, rl, B, L, H, Hkv, d)
    err = (dqkv.float() - ref).abs().max().item()
    assert err <= 6e-2 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("B,L,H,Hkv,d", [(2, 384, 8, 2, 64), (1, 1000, 4, 4, 128), (3, 130, 6, 3, 64)])
def test_backward_with_the_inverse_rotation_of_dq_in_the_conversion_pass(B, L, H, Hkv, d):
    """dQ is rotated back where its fp32 accumulator becomes bf16, dK by the rope kernel on the key columns only: the
    result equals attention backward + inverse rope over q and k bit for bit."""
    from llm_distillery_b200.ops import basic
    torch.manual_seed(L + d)
    qkv = torch.randn(B * L, (H + 2 * Hkv) * d, device="cuda").bfloat16()
    out, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d)
    dout = torch.randn_like(out)
    pos = torch.arange(L, dtype=torch.int32, device="cuda").repeat(B)
    cos, sin = basic.rope_tables(L, d, 10000.0, "cuda")
    got = attention.attention_bwd_unrotated(dout, qkv, out, lse, B, L, H, Hkv, d, pos, cos, sin)
    assert _lib.take_device_error() == 0
    ref = attention.attention_bwd(dout, qkv, out, lse, B, L, H, Hkv, d)
    v_cols = slice((H + Hkv) * d, None)
    # dQ accumulates through TMA reduce-add in an order that varies from run to run: compare to rounding, and the
    # untouched value columns and the rotation itself exactly on a copy of the SAME backward result
    same = ref.clone()
    basic.rope_(same, pos, cos, sin, H + Hkv, d, inverse=True)
    assert torch.allclose(got.float(), same.float(), atol=3e-2 * max(1.0, same.float().abs().max().item()), rtol=3e-2)
    assert torch.allclose(got[:, v_cols].float(), ref[:, v_cols].float(), atol=2e-2, rtol=2e-2)
    # exactness of the fused conversion: feed one accumulator through both paths
    acc = torch.randn(B * L, H * d, device="cuda")
    a = torch.zeros(B * L, (H + 2 * Hkv) * d, device="cuda", dtype=torch.bfloat16)
    a[:, : H * d] = acc.bfloat16()
    basic.rope_(a, pos, cos, sin, H, d, inverse=True)
    from llm_distillery_b200.ops import flash  # noqa: F401  (registers the entry point)
    b = torch.zeros_like(a)
    _lib.check(_lib.kernels().b200_dq_convert_rope(_lib.ptr(acc), _lib.ptr(b), _lib.ptr(pos), _lib.ptr(cos), _lib.ptr(sin),
                                                   B * L, H, d, b.stride(0), _lib.stream()), "b200_dq_convert_rope")
    assert torch.equal(a[:, : H * d], b[:, : H * d])


@pytest.mark.parametrize("B,L,H,Hkv,d,window", [(2, 300, 4, 2, 64, 128), (1, 1000, 8, 8, 128, 256)])
def test_sequences_longer_than_a_sliding_window(B, L, H, Hkv, d, window):
    """Beyond the window the flash kernels step aside for the band-masked library path: forward and backward on the
    GPU (bf16) against the same path in fp32 on the CPU; inside the window the flash kernels still run."""
    torch.manual_seed(L + window)
    qkv = torch.randn(B * L, (H + 2 * Hkv) * d, device=DEV).bfloat16()
    dout = torch.randn(B * L, H * d, device=DEV).bfloat16()
    out, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d, window)
    dqkv = attention.attention_bwd(dout, qkv, out, lse, B, L, H, Hkv, d, window)
    assert out.dtype == torch.bfloat16 and dqkv.shape == qkv.shape
    ro, _ = attention.attention_fwd(qkv.float().cpu(), B, L, H, Hkv, d, window)
    rd = attention.attention_bwd(dout.float().cpu(), qkv.float().cpu(), ro, None, B, L, H, Hkv, d, window)
    assert torch.allclose(out.float().cpu(), ro, atol=3e-2, rtol=3e-2), (out.float().cpu() - ro).abs().max()
    err = (dqkv.float().cpu() - rd).abs().max().item()
    assert err <= 6e-2 * max(1.0, rd.abs().max().item()), err
    causal, _ = attention.attention_reference_fwd(qkv.float().cpu(), B, L, H, Hkv, d)
    assert (causal - ro).abs().max() > 0.1                    # the window matters at this length
    # a chunk against the key / value cache
    kv = Hkv * d
    kc = qkv[:, H * d:H * d + kv].reshape(B, L, kv).contiguous()
    vc = qkv[:, H * d + kv:].reshape(B, L, kv).contiguous()
    n, c0 = 128, L - 128 - (L - 128) % 8
    rows = torch.cat([qkv[b * L + c0: b * L + c0 + n] for b in range(B)])
    got = attention.attention_fwd_cached(rows.contiguous(), kc, vc, B, n, c0, H, Hkv, d, window)
    want = torch.cat([ro[b * L + c0: b * L + c0 + n] for b in range(B)])
    assert torch.allclose(got.float().cpu(), want, atol=3e-2, rtol=3e-2)
    # a window that covers the sequence: the flash kernels, bit for bit what they give without one
    a, _ = attention.attention_fwd(qkv, B, L, H, Hkv, d, L)
    b, _ = attention.attention_fwd(qkv, B, L, H, Hkv, d)
    assert torch.equal(a, b) and _lib.take_device_error() == 0
