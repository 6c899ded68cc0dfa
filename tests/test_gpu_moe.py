"""Mixture-of-experts decoder on the GPU kernels (bf16) against the same model in fp32 on the CPU restatements."""
import pytest
import torch

from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _cos(a, b):
    a, b = a.detach().double().flatten().cpu(), b.detach().double().flatten().cpu()
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))


@pytest.mark.parametrize("family", ["mixtral", "qwen2_moe", "olmoe", "granitemoeshared"])
def test_experts_forward_and_backward_match_the_fp32_restatement(family):
    """Mixtral's routed experts; Qwen2-MoE adds the q/k/v bias and the gated shared expert (a dense MLP on the fused
    SwiGLU GEMMs); OLMoE normalises the whole query / key projections; Granite MoE scales both branches by a residual
    multiplier and adds an ungated shared MLP."""
    cfg = LlamaConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=512, model_type=family, num_local_experts=4,
                      num_experts_per_tok=2,
                      **(dict(shared_expert_intermediate_size=384, attention_bias=True, moe_renormalize=False)
                         if family == "qwen2_moe" else dict(qk_norm_full=True, moe_renormalize=False)
                         if family == "olmoe" else
                         dict(shared_expert_intermediate_size=384, shared_expert_gated=False, residual_multiplier=0.3,
                              embedding_multiplier=6.0, attention_multiplier=0.1, logits_scaling=4.0)
                         if family == "granitemoeshared" else {}))
    ref = build_model(cfg, dtype=torch.float32, device="cpu", seed=4)
    with torch.no_grad():
        for l in ref.layers:
            l.router.mul_(20.0)          # clear routing decisions: bf16 rounding must not flip many of them
            if family == "qwen2_moe":
                l.shared_expert_gate.mul_(20.0)
            if family == "olmoe":
                l.q_norm.uniform_(0.5, 1.5)
                l.k_norm.uniform_(0.5, 1.5)
    gpu = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=None)
    with torch.no_grad():
        for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
            p.copy_(q.to(torch.bfloat16))
            q.copy_(p.float().cpu())     # both sides hold the bf16-rounded weights
    x = torch.randint(0, 1024, (4, 512))       # ~1000 rows per expert: the experts' GEMMs take the fused SwiGLU epilogues
    tgt = torch.randint(0, 1024, (4 * 512,))
    out_g = gpu(x.cuda())
    out_r = ref(x)
    assert _lib.take_device_error() == 0
    assert _cos(out_g.float(), out_r) > 0.998
    torch.nn.functional.cross_entropy(out_g.float().reshape(-1, 1024), tgt.cuda()).backward()
    torch.nn.functional.cross_entropy(out_r.reshape(-1, 1024), tgt).backward()
    assert _lib.take_device_error() == 0
    for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
        assert torch.isfinite(p.grad).all(), n
        loose = "router" in n or "shared_expert_gate" in n
        assert _cos(p.grad.float(), q.grad) > (0.95 if loose else 0.985), (n, _cos(p.grad.float(), q.grad))
    # inference in chunks against the K/V cache takes the same expert path
    with torch.no_grad():
        full = gpu.hidden_states(x.cuda())
        chunked = gpu.hidden_states_chunked(x.cuda(), 256)
    assert _cos(full.float(), chunked.float()) > 0.999
