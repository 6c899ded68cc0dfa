"""Teacher forward in chunks against a key / value cache equals the whole-sequence pass (CPU restatement here, the
sm_100a kernel with its query offset on a GPU), and the collector's rows do not depend on the chunk length."""
import numpy as np
import pytest
import torch

from llm_distillery_b200.collect.collector import TeacherCollector
from llm_distillery_b200.data.convo import ConvoTokenized
from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.models.teacher import TeacherModel
from llm_distillery_b200.ops import attention


def _model(device, dtype, d=64):
    cfg = LlamaConfig(vocab_size=1024, hidden_size=4 * d, intermediate_size=512, num_hidden_layers=3,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=1024)
    return cfg, build_model(cfg, dtype=dtype, device=device, seed=5)


@pytest.mark.parametrize("chunk", [16, 48, 64])
def test_chunked_forward_equals_the_full_pass_on_cpu(chunk):
    cfg, model = _model("cpu", torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (2, 112))
    with torch.no_grad():
        full = model.hidden_states(ids)
        part = model.hidden_states_chunked(ids, chunk)
    assert torch.allclose(full, part, atol=2e-5, rtol=1e-4), (full - part).abs().max()


def test_collector_rows_do_not_depend_on_the_chunk_length():
    cfg, model = _model("cpu", torch.float32)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, 1000, (2, 96)).astype(np.int64)
    convos = [ConvoTokenized(toks[0], [(3, 50), (60, 96)], 0, False, 0), ConvoTokenized(toks[1], [(0, 96)], 0, False, 1)]
    a = TeacherCollector(model, topk=8, crop_to_size=1000).collect_batch(toks, convos)
    b = TeacherCollector(model, topk=8, crop_to_size=1000, prefill_chunk_len=32).collect_batch(toks, convos)
    for x, y in zip(a, b):
        assert np.array_equal(x.indices, y.indices) and np.allclose(x.values, y.values, atol=2e-3)


def test_chunk_length_policy():
    t = TeacherModel.__new__(TeacherModel)
    t.seq_chunk_len, t.prefill_max_tokens = 256, 8192
    t.chunked_prefill = "true"
    assert t.prefill_chunk_len(4, 2048) == 256 and t.prefill_chunk_len(4, 200) == 0
    t.chunked_prefill = "false"
    assert t.prefill_chunk_len(64, 8192) == 0
    t.chunked_prefill = "auto"
    assert t.prefill_chunk_len(2, 2048) == 0                # 4096 tokens: one pass
    assert t.prefill_chunk_len(4, 8192) == 2048             # 32768 tokens: chunks that keep a pass at 8192 tokens


@pytest.mark.gpu
@pytest.mark.parametrize("d,L,chunk", [(64, 640, 128), (64, 1000, 384), (128, 768, 256), (128, 520, 200)])
def test_cached_attention_kernel_and_chunked_forward_on_gpu(d, L, chunk):
    torch.manual_seed(d + L)
    B, H, Hkv = 2, 4, 2
    qkv = (torch.randn(B * L, (H + 2 * Hkv) * d, device="cuda") * 1.2).bfloat16()
    full, _ = attention.attention_fwd(qkv, B, L, H, Hkv, d)
    q3 = qkv.view(B, L, -1)
    kc = torch.zeros(B, L, Hkv * d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    outs = []
    for c0 in range(0, L, chunk):
        n = min(chunk, L - c0)
        piece = q3[:, c0:c0 + n].reshape(B * n, -1).contiguous()
        kc[:, c0:c0 + n] = piece[:, H * d:(H + Hkv) * d].reshape(B, n, -1)
        vc[:, c0:c0 + n] = piece[:, (H + Hkv) * d:].reshape(B, n, -1)
        o = attention.attention_fwd_cached(piece, kc, vc, B, n, c0, H, Hkv, d)
        ref = attention.attention_cached_reference_fwd(piece.float(), kc.float(), vc.float(), B, n, c0, H, Hkv, d)
        assert torch.allclose(o.float(), ref, atol=3e-2, rtol=3e-2), (o.float() - ref).abs().max()
        outs.append(o.view(B, n, -1))
    got = torch.cat(outs, 1).reshape(B * L, -1)
    assert torch.allclose(got.float(), full.float(), atol=3e-2, rtol=3e-2)
    cfg, model = _model("cuda", torch.bfloat16, d)
    ids = torch.randint(0, cfg.vocab_size, (2, L), device="cuda")
    with torch.no_grad():
        a, b = model.hidden_states(ids), model.hidden_states_chunked(ids, chunk)
    assert (a.float() - b.float()).abs().max() <= 0.06 * a.float().abs().max()
    from llm_distillery_b200.ops import _lib
    assert _lib.take_device_error() == 0
