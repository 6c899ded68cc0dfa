"""models/llama.py on CPU (fp32): hand-written backward of the fused decoder layer vs autograd of a plain model."""
import torch

from llm_distillery_b200.models.llama import LlamaConfig, build_model, GradSlot
from tests import ref_llama


def _tiny(tied=False, kv=2):
    return LlamaConfig(vocab_size=97, hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=kv, rms_norm_eps=1e-6, max_position_embeddings=64, tie_word_embeddings=tied)


def test_forward_and_backward_match_autograd():
    torch.manual_seed(0)
    m = build_model(_tiny(), dtype=torch.float32, seed=1)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    ids = torch.randint(0, 97, (2, 24))
    logits = m(ids)
    ref_params = {n: p.detach().clone().requires_grad_() for n, p in m.named_parameters()}
    ref_logits = ref_llama.forward_logits(m, ids, ref_params)
    assert torch.allclose(logits, ref_logits, atol=1e-4, rtol=1e-4)
    w = torch.randn_like(logits)
    (logits * w).sum().backward()
    (ref_logits * w).sum().backward()
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, ref_params[n].grad, atol=2e-4, rtol=1e-3), n


def test_grad_slots_accumulate_and_checkpointing_matches():
    torch.manual_seed(1)
    m = build_model(_tiny(tied=True, kv=4), dtype=torch.float32, seed=2)
    ids = torch.randint(0, 97, (2, 16))
    (m(ids).float().pow(2).mean()).backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad(set_to_none=True)
    for p in m.parameters():
        p.grad_slot = GradSlot(torch.zeros_like(p, dtype=torch.float32))
    m.grad_checkpointing = True
    for _ in range(2):   # two micro-batches accumulate
        (m(ids).float().pow(2).mean()).backward()
    for n, p in m.named_parameters():
        assert p.grad is None
        assert torch.allclose(p.grad_slot.buf, 2 * ref[n], atol=1e-5, rtol=1e-3), n


def test_hf_state_dict_roundtrip_and_freeze():
    m = build_model(_tiny(), dtype=torch.float32, seed=3)
    sd = {k: v.clone() for k, v in m.to_hf_state_dict().items()}
    assert "model.layers.1.self_attn.k_proj.weight" in sd and "model.layers.0.mlp.up_proj.weight" in sd
    m2 = build_model(_tiny(), dtype=torch.float32, seed=4)
    m2.load_hf_state_dict(sd)
    for (n, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n
    frozen = m2.apply_freeze(["layers.0.mlp.down_proj", "embed_tokens"])
    assert not m2.layers[0].down_proj.requires_grad and not m2.embed_tokens.requires_grad
    assert m2.layers[1].down_proj.requires_grad and len(frozen) == 2
    ids = torch.randint(0, 97, (1, 8))
    m2(ids).sum().backward()
    assert m2.layers[0].down_proj.grad is None and m2.layers[1].down_proj.grad is not None
