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
