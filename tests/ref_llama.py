"""Plain-PyTorch Llama forward (autograd does the backward): the oracle for models/llama.py."""
import math

import torch
import torch.nn.functional as F


def rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope(x, pos, theta):  # x [B, L, nh, d]
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = pos[:, None].double() * inv[None, :]
    c, s = ang.cos()[None, :, None, :].to(x.dtype), ang.sin()[None, :, None, :].to(x.dtype)
    a, b = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def forward_hidden(model, ids, params=None):
    """model: LlamaModel (for config + weights); params: optional dict name->tensor overriding weights."""
    cfg = model.cfg
    P = dict(model.named_parameters()) if params is None else params
    B, L = ids.shape
    H, Hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    h = P["embed_tokens"][ids]
    pos = torch.arange(L)
    for i in range(cfg.num_hidden_layers):
        pre = f"layers.{i}."
        n1 = rms(h, P[pre + "input_layernorm"], cfg.rms_norm_eps)
        qkv = n1 @ P[pre + "qkv_proj"].t()
        q = qkv[..., : H * d].reshape(B, L, H, d)
        k = qkv[..., H * d: (H + Hkv) * d].reshape(B, L, Hkv, d)
        v = qkv[..., (H + Hkv) * d:].reshape(B, L, Hkv, d)
        q, k = rope(q, pos, cfg.rope_theta), rope(k, pos, cfg.rope_theta)
        g = H // Hkv
        k, v = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
        s = torch.einsum("blhd,bmhd->bhlm", q, k) / math.sqrt(d)
        s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool).tril(), float("-inf"))
        a = torch.einsum("bhlm,bmhd->blhd", s.softmax(-1), v).reshape(B, L, H * d)
        h = h + a @ P[pre + "o_proj"].t()
        n2 = rms(h, P[pre + "post_attention_layernorm"], cfg.rms_norm_eps)
        gu = n2 @ P[pre + "gate_up_proj"].t()
        f = gu.shape[-1] // 2
        h = h + (F.silu(gu[..., :f]) * gu[..., f:]) @ P[pre + "down_proj"].t()
    return rms(h, P["norm"], cfg.rms_norm_eps)


def forward_logits(model, ids, params=None):
    P = dict(model.named_parameters()) if params is None else params
    return forward_hidden(model, ids, params) @ P["lm_head" if "lm_head" in P else "embed_tokens"].t()
