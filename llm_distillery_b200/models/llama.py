"""Llama-family decoder (Llama 1/2/3, TinyLlama, Mistral: RMSNorm, RoPE, GQA, SwiGLU, optional tied embeddings;
Qwen2 with q/k/v bias, Phi-3 with fused projections, Mixtral with sparse experts - models/moe.py; OLMo 2 and GLM-4
with norms behind the branches - models/sandwich.py)
for both roles: student training (forward + hand-written backward) and teacher inference.

Design. Each decoder layer is ONE autograd node (``DecoderLayerFn``) whose forward and backward are explicit
sequences of the kernels in ``ops`` - 7 GEMMs, 2 RMSNorms, RoPE, flash attention, SwiGLU - so residual adds ride
in GEMM epilogues, the residual-branch gradient is added inside the RMSNorm backward, weight gradients are
accumulated by the wgrad GEMM epilogue straight into fp32 ``main_grad`` buffers, and no autograd bookkeeping or
library elementwise kernel sits between them. QKV and gate/up projections are stored fused ([(H+2Hkv)d, h] and
[2f, h]); HuggingFace checkpoints are split / concatenated at load / save time (``to_hf_state_dict``).

The same code runs on CPU tensors through the PyTorch restatements in ``ops`` (fp32 plumbing runs and tests).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import attention, basic
from .config import PRESETS, LlamaConfig, preset  # noqa: F401  (re-exported: the models' public names live here)


# ---------------------------------------------------------------------------------------------- gradient slots
class GradSlot:
    """fp32 accumulation target of one parameter (a view into the engine's flat gradient buffer). ``fresh`` means
    nothing has been accumulated since the last optimizer step: the next wgrad overwrites instead of adding."""
    __slots__ = ("buf", "fresh")

    def __init__(self, buf: torch.Tensor):
        self.buf = buf
        self.fresh = True


def _slot(p: torch.Tensor):
    return getattr(p, "grad_slot", None) if p.requires_grad else None


def _wgrad(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, slot):
    """Weight gradient of y = x w^T. With a slot: accumulated in place (fp32), returns None. Else returns dW."""
    if not w.requires_grad:
        return None
    if slot is not None:
        basic.linear_wgrad(dy, x, out=slot.buf, accumulate=not slot.fresh)
        slot.fresh = False
        return None
    return basic.linear_wgrad(dy, x, out_dtype=w.dtype)


def _bias_grad(dy: torch.Tensor, b: torch.Tensor | None, slot):
    """Gradient of a bias added to every row of a GEMM output: the column sums of dy."""
    if b is None or not b.requires_grad:
        return None
    if slot is not None:
        basic.bias_grad(dy, out=slot.buf, accumulate=not slot.fresh)
        slot.fresh = False
        return None
    return basic.bias_grad(dy).to(b.dtype)


def _vec_grad(dw: torch.Tensor, w: torch.Tensor, slot):
    if not w.requires_grad:
        return None
    if slot is not None:
        if slot.fresh:
            slot.buf.copy_(dw)
            slot.fresh = False
        else:
            slot.buf.add_(dw)
        return None
    return dw.to(w.dtype)


# ---------------------------------------------------------------------------------------------- autograd nodes
class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w):
        ctx.save_for_backward(ids)
        ctx.w = w
        ctx.slot = _slot(w)
        return basic.embed_fwd(ids, w)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        w, slot = ctx.w, ctx.slot
        if not w.requires_grad:
            return None, None
        if slot is not None:
            if slot.fresh:
                slot.buf.zero_()
                slot.fresh = False
            basic.embed_bwd(ids, dout.contiguous(), slot.buf)
            return None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        basic.embed_bwd(ids, dout.contiguous(), dw)
        return None, dw.to(w.dtype)


# Called with a layer's first parameter when that layer's backward has produced all its weight gradients (and, since
# backward runs from the last layer to the first, those of every later layer): the data-parallel engine starts
# reducing that part of the gradient while the earlier layers are still in backward.
LAYER_BACKWARD_DONE = [None]

# Called with (parameter, backward) just before a unit of the model - the embedding, a decoder layer, the final norm
# + head - reads its parameters, in forward and again at the start of a layer's backward: the full-shard engine
# (parallel/fsdp.py) gathers that unit's weights there and starts gathering the next one.
UNIT_PRE = [None]
# Called with a decoder layer's first parameter just before the layer's matrices are read, in forward and at the start
# of its backward: frozen low-bit weights (ops/quant.py) are expanded into their bf16 buffer there.
LAYER_WEIGHTS_PRE = [None]


class DecoderLayerFn(torch.autograd.Function):
    """h_out = h + Attn(RMSNorm(h)) ; then + MLP(RMSNorm(.)) - one node, explicit backward."""

    @staticmethod
    def forward(ctx, h, pos, cos, sin, w_ln1, w_qkv, w_o, w_ln2, w_gu, w_d, meta, b_qkv=None, w_qn=None, w_kn=None,
                b_o=None, b_gu=None, b_d=None, rmul=1.0):
        B, L, H, Hkv, d, eps, recompute, window = meta
        n1, _, rstd1 = basic.rmsnorm_fwd(h, w_ln1, eps)
        qk_saved = ()
        if b_qkv is None and w_qn is None:                    # rotation in the epilogue of the q/k/v GEMM
            qkv = basic.linear_rope_fwd(n1, w_qkv, pos, cos, sin, H + Hkv, d)
        else:
            qkv = basic.linear_fwd(n1, w_qkv)
            if b_qkv is not None:
                basic.bias_add_(qkv, b_qkv)
            if w_qn is not None:                              # per-head norm of q and k (Qwen3), before the rotation
                qkv_raw = qkv
                qkv, rstd_qk = basic.headnorm_fwd(qkv_raw, w_qn, w_kn, H, Hkv, d, eps)
                qk_saved = (qkv_raw, rstd_qk)
            basic.rope_(qkv, pos, cos, sin, H + Hkv, d)      # q and k heads are adjacent columns
        att, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d, window)
        # rmul (Granite's residual_multiplier) scales a branch, bias included, before it joins the residual stream: it is
        # the alpha of the GEMM whose epilogue adds the residual
        h1 = basic.gemm(att, w_o, residual=h, alpha=rmul)
        if b_o is not None:
            basic.bias_add_(h1, b_o if rmul == 1.0 else b_o * rmul)
        n2, _, rstd2 = basic.rmsnorm_fwd(h1, w_ln2, eps)
        if b_gu is None:
            gu, act = basic.linear_swiglu_fwd(n2, w_gu)
        else:
            gu = basic.bias_add_(basic.linear_fwd(n2, w_gu), b_gu)
            act = basic.swiglu_fwd(gu)
        h2 = basic.gemm(act, w_d, residual=h1, alpha=rmul)
        if b_d is not None:
            basic.bias_add_(h2, b_d if rmul == 1.0 else b_d * rmul)
        ctx.rmul = rmul
        ctx.more_b = (b_o, b_gu, b_d)
        ctx.more_b_slots = tuple(_slot(b) if b is not None else None for b in ctx.more_b)
        ctx.meta = meta
        ctx.weights = (w_ln1, w_qkv, w_o, w_ln2, w_gu, w_d)
        ctx.slots = tuple(_slot(w) for w in ctx.weights)
        ctx.b_qkv = b_qkv
        ctx.b_slot = _slot(b_qkv) if b_qkv is not None else None
        ctx.qk_w = (w_qn, w_kn)
        ctx.qk_slots = (_slot(w_qn), _slot(w_kn)) if w_qn is not None else (None, None)
        if recompute:   # gradient checkpointing: keep only the layer input
            ctx.save_for_backward(h, pos, cos, sin)
        else:
            ctx.save_for_backward(h, pos, cos, sin, rstd1, n1, qkv, att, lse, h1, rstd2, n2, gu, act, *qk_saved)
        return h2

    @staticmethod
    def backward(ctx, dh2):
        B, L, H, Hkv, d, eps, recompute, window = ctx.meta
        w_ln1, w_qkv, w_o, w_ln2, w_gu, w_d = ctx.weights
        s_ln1, s_qkv, s_o, s_ln2, s_gu, s_d = ctx.slots
        if UNIT_PRE[0] is not None:
            UNIT_PRE[0](w_ln1, True)
        if LAYER_WEIGHTS_PRE[0] is not None:
            LAYER_WEIGHTS_PRE[0](w_ln1)
        w_qn, w_kn = ctx.qk_w
        qkv_raw = rstd_qk = None
        if recompute:
            h, pos, cos, sin = ctx.saved_tensors
            n1, _, rstd1 = basic.rmsnorm_fwd(h, w_ln1, eps)
            if ctx.b_qkv is None and w_qn is None:
                qkv = basic.linear_rope_fwd(n1, w_qkv, pos, cos, sin, H + Hkv, d)
            else:
                qkv = basic.linear_fwd(n1, w_qkv)
                if ctx.b_qkv is not None:
                    basic.bias_add_(qkv, ctx.b_qkv)
                if w_qn is not None:
                    qkv_raw = qkv
                    qkv, rstd_qk = basic.headnorm_fwd(qkv_raw, w_qn, w_kn, H, Hkv, d, eps)
                basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
            att, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d, window)
            h1 = basic.gemm(att, w_o, residual=h, alpha=ctx.rmul)
            if ctx.more_b[0] is not None:
                basic.bias_add_(h1, ctx.more_b[0] if ctx.rmul == 1.0 else ctx.more_b[0] * ctx.rmul)
            n2, _, rstd2 = basic.rmsnorm_fwd(h1, w_ln2, eps)
            if ctx.more_b[1] is None:
                gu, act = basic.linear_swiglu_fwd(n2, w_gu)
            else:
                gu = basic.bias_add_(basic.linear_fwd(n2, w_gu), ctx.more_b[1])
                act = basic.swiglu_fwd(gu)
        elif w_qn is not None:
            h, pos, cos, sin, rstd1, n1, qkv, att, lse, h1, rstd2, n2, gu, act, qkv_raw, rstd_qk = ctx.saved_tensors
        else:
            h, pos, cos, sin, rstd1, n1, qkv, att, lse, h1, rstd2, n2, gu, act = ctx.saved_tensors
        dh2 = dh2.contiguous()
        b_o, b_gu, b_d = ctx.more_b
        sb_o, sb_gu, sb_d = ctx.more_b_slots
        # MLP branch (its gradient is the stream's gradient times the branch multiplier)
        rmul = ctx.rmul
        db2 = dh2 if rmul == 1.0 else dh2 * rmul
        g_bd = _bias_grad(db2, b_d, sb_d)
        g_d = _wgrad(db2, act, w_d, s_d)
        del act
        dgu = basic.linear_dgrad_swiglu_bwd(db2, w_d, gu)     # dgrad of the down projection + SwiGLU backward
        del db2
        g_bgu = _bias_grad(dgu, b_gu, sb_gu)
        g_gu = _wgrad(dgu, n2, w_gu, s_gu)
        dn2 = basic.linear_dgrad(dgu, w_gu)
        del dgu
        dh1, dw2 = basic.rmsnorm_bwd(dn2, h1, w_ln2, rstd2, dres=dh2)
        g_ln2 = _vec_grad(dw2, w_ln2, s_ln2)
        # attention branch
        db1 = dh1 if rmul == 1.0 else dh1 * rmul
        g_bo = _bias_grad(db1, b_o, sb_o)
        g_o = _wgrad(db1, att, w_o, s_o)
        datt = basic.linear_dgrad(db1, w_o)
        del db1
        dqkv = attention.attention_bwd_unrotated(datt, qkv, att, lse, B, L, H, Hkv, d, pos, cos, sin, window)
        del datt
        g_qn = g_kn = None
        if w_qn is not None:
            dwq, dwk = basic.headnorm_bwd_(dqkv, qkv_raw, w_qn, w_kn, rstd_qk, H, Hkv, d)
            g_qn = _vec_grad(dwq, w_qn, ctx.qk_slots[0])
            g_kn = _vec_grad(dwk, w_kn, ctx.qk_slots[1])
        g_b = None
        if ctx.b_qkv is not None and ctx.b_qkv.requires_grad:
            if ctx.b_slot is not None:
                basic.bias_grad(dqkv, out=ctx.b_slot.buf, accumulate=not ctx.b_slot.fresh)
                ctx.b_slot.fresh = False
            else:
                g_b = basic.bias_grad(dqkv).to(ctx.b_qkv.dtype)
        g_qkv = _wgrad(dqkv, n1, w_qkv, s_qkv)
        dn1 = basic.linear_dgrad(dqkv, w_qkv)
        del dqkv
        dh, dw1 = basic.rmsnorm_bwd(dn1, h, w_ln1, rstd1, dres=dh1)
        g_ln1 = _vec_grad(dw1, w_ln1, s_ln1)
        if LAYER_BACKWARD_DONE[0] is not None:
            LAYER_BACKWARD_DONE[0](w_ln1)
        return (dh, None, None, None, g_ln1, g_qkv, g_o, g_ln2, g_gu, g_d, None, g_b, g_qn, g_kn, g_bo, g_bgu, g_bd,
                None)


class FinalNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, eps):
        y, _, rstd = basic.rmsnorm_fwd(h, w, eps)
        ctx.save_for_backward(h, rstd)
        ctx.w, ctx.slot = w, _slot(w)
        return y

    @staticmethod
    def backward(ctx, dy):
        h, rstd = ctx.saved_tensors
        dh, dw = basic.rmsnorm_bwd(dy.contiguous(), h, ctx.w, rstd)
        return dh, _vec_grad(dw, ctx.w, ctx.slot), None


class LinearFn(torch.autograd.Function):
    """y = x w^T, used for the LM head when full logits are requested (teacher collection, CPU oracle)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x)
        ctx.w, ctx.slot = w, _slot(w)
        return basic.linear_fwd(x, w)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        return basic.linear_dgrad(dy, ctx.w), _wgrad(dy, x, ctx.w, ctx.slot)


# ---------------------------------------------------------------------------------------------- modules
class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype, device):
        super().__init__()
        h, f = cfg.hidden_size, cfg.intermediate_size
        kw = dict(dtype=dtype, device=device)
        if cfg.pre_norm:
            self.input_layernorm = nn.Parameter(torch.ones(h, **kw))
        self.qkv_proj = nn.Parameter(torch.empty(cfg.q_size + 2 * cfg.kv_size, h, **kw))
        if cfg.attention_bias:
            self.qkv_bias = nn.Parameter(torch.zeros(cfg.q_size + 2 * cfg.kv_size, **kw))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw))
        elif cfg.qk_norm_full:
            self.q_norm = nn.Parameter(torch.ones(cfg.q_size, **kw))
            self.k_norm = nn.Parameter(torch.ones(cfg.kv_size, **kw))
        self.o_proj = nn.Parameter(torch.empty(h, cfg.q_size, **kw))
        if cfg.o_bias:
            self.o_bias = nn.Parameter(torch.zeros(h, **kw))
        if cfg.post_norm:
            self.attn_out_norm = nn.Parameter(torch.ones(h, **kw))
        if cfg.mlp_bias:
            if cfg.num_local_experts:
                raise NotImplementedError("mlp_bias with experts is not built")
            self.gate_up_bias = nn.Parameter(torch.zeros(2 * f, **kw))
            self.down_bias = nn.Parameter(torch.zeros(h, **kw))
        if cfg.pre_norm:
            self.post_attention_layernorm = nn.Parameter(torch.ones(h, **kw))
        E = cfg.num_local_experts
        if E:       # sparse mixture of experts: a router and E stacked expert matrices (models/moe.py)
            self.router = nn.Parameter(torch.empty(E, h, **kw))
            self.gate_up_proj = nn.Parameter(torch.empty(E, 2 * f, h, **kw))
            self.down_proj = nn.Parameter(torch.empty(E, h, f, **kw))
            fs = cfg.shared_expert_intermediate_size
            if fs:
                self.shared_gate_up_proj = nn.Parameter(torch.empty(2 * fs, h, **kw))
                self.shared_down_proj = nn.Parameter(torch.empty(h, fs, **kw))
                if cfg.shared_expert_gated:
                    self.shared_expert_gate = nn.Parameter(torch.empty(1, h, **kw))
        else:
            self.gate_up_proj = nn.Parameter(torch.empty(2 * f, h, **kw))
            self.down_proj = nn.Parameter(torch.empty(h, f, **kw))
        if cfg.post_norm:
            self.mlp_out_norm = nn.Parameter(torch.ones(h, **kw))
        if cfg.sandwich and (E or cfg.o_bias or cfg.mlp_bias or cfg.residual_multiplier != 1.0):
            raise NotImplementedError("output norms / whole-projection q-k norms together with experts, o_proj or MLP "
                                      "biases or a residual multiplier are not built")

    @property
    def first_param(self) -> torch.Tensor:
        """The layer's first registered parameter: the key under which the engines' per-layer hooks know the layer
        (lowest offset of the layer in a flat parameter buffer)."""
        return next(iter(self.parameters()))


class LlamaModel(nn.Module):
    """Parameters use fused projection names; ``named_hf_parameters`` / ``to_hf_state_dict`` expose the HF names
    (``model.layers.N.self_attn.q_proj.weight`` ...), which is also what ``freeze_layers`` substrings match."""

    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = cfg
        if torch.device(device).type == "cuda":
            cfg.check_gpu_kernels()
        kw = dict(dtype=dtype, device=device)
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.layers = nn.ModuleList([LlamaDecoderLayer(cfg, dtype, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        if cfg.tie_word_embeddings:
            self.lm_head = self.embed_tokens
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.grad_checkpointing = False
        self._rope = None
        self.quant = None          # FrozenQuantLinears when the decoder layers' matrices are frozen NF4 / int8

    # ---- init / tables
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "LlamaModel":
        gens: dict = {}
        for name, p in self.named_parameters():
            if name.endswith("_bias"):
                dev = p.device
                if dev not in gens:
                    gens[dev] = torch.Generator(device=dev).manual_seed(seed)
                p.normal_(mean=0.0, std=std, generator=gens[dev])
            elif p.dim() == 1:
                p.fill_(1.0)
            else:
                dev = p.device
                if dev not in gens:
                    gens[dev] = torch.Generator(device=dev).manual_seed(seed)
                p.normal_(mean=0.0, std=std, generator=gens[dev])   # generated where the weights live
        return self

    def rope(self, device, max_pos: int | None = None):
        need = max_pos or self.cfg.max_position_embeddings
        sc = self.cfg.rope_scaling or {}
        regime = None
        if sc.get("rope_type", sc.get("type")) == "longrope":    # the factor set depends on the sequence length
            regime = need > int(sc.get("original_max_position_embeddings") or self.cfg.max_position_embeddings)
        elif sc.get("rope_type", sc.get("type")) == "dynamic" and not sc.get("alpha"):
            regime = need if need > self.cfg.max_position_embeddings else False      # the base follows the length
        if (self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < need
                or getattr(self, "_rope_regime", None) != regime):
            n = max(need, min(self.cfg.max_position_embeddings, 8192))
            if regime is False and sc.get("rope_type", sc.get("type")) == "longrope":
                n = min(n, int(sc.get("original_max_position_embeddings") or n))
            self._rope = basic.rope_tables(n, self.cfg.rotary_dim, self.cfg.rope_theta, device, self.cfg.rope_scaling,
                                           model_max_pos=self.cfg.max_position_embeddings, seq_len=need)
            am = self.cfg.attention_multiplier
            if am is not None and abs(am * math.sqrt(self.cfg.head_dim) - 1.0) > 1e-9:
                # the attention kernels scale the scores by 1 / sqrt(d); a different multiplier rides on the rotation:
                # queries and keys each take sqrt(multiplier * sqrt(d)), their products the multiplier over 1 / sqrt(d)
                amp = math.sqrt(am * math.sqrt(self.cfg.head_dim))
                self._rope = ((self._rope[0] * amp).contiguous(), (self._rope[1] * amp).contiguous())
            self._rope_regime = regime
        return self._rope

    def _embedding_scale(self, dtype):
        m = self.cfg.embedding_multiplier
        if self.cfg.embedding_multiplier_rounded:       # Gemma keeps the multiplier as a tensor of the model's dtype
            return torch.tensor(m, dtype=torch.float32).to(dtype).item()
        return m

    def layer_rope(self, cos: torch.Tensor, sin: torch.Tensor) -> list:
        """One (cos, sin) pair per layer: the tables, or the identity rotation (cos 1, sin 0) for layers that apply no
        positional rotation, or (Gemma 3) tables of another base for the windowed layers. The same kernels run either
        way."""
        flags = self.cfg.no_rope_layers
        n = len(self.layers)
        if self.cfg.rope_local_theta and self.cfg.window_layers:
            local = getattr(self, "_rope_local", None)
            if local is None or local[0].shape[0] < cos.shape[0] or local[0].device != cos.device:
                local = basic.rope_tables(cos.shape[0], self.cfg.rotary_dim, self.cfg.rope_local_theta, cos.device)
                am = self.cfg.attention_multiplier
                if am is not None and abs(am * math.sqrt(self.cfg.head_dim) - 1.0) > 1e-9:
                    amp = math.sqrt(am * math.sqrt(self.cfg.head_dim))       # as for the global tables (``rope``)
                    local = ((local[0] * amp).contiguous(), (local[1] * amp).contiguous())
                self._rope_local = local
            return [local if self.cfg.window_layers[i] else (cos, sin) for i in range(n)]
        if not flags or all(flags):
            return [(cos, sin)] * n
        ident = getattr(self, "_rope_ident", None)
        if ident is None or ident[0].shape != cos.shape or ident[0].device != cos.device:
            ident = self._rope_ident = (torch.ones_like(cos), torch.zeros_like(sin))
        return [(cos, sin) if flags[i] else ident for i in range(n)]

    # ---- forward
    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        """input_ids [B, L] int64 -> final-norm hidden states [B*L, h]."""
        cfg = self.cfg
        B, L = input_ids.shape
        dev = self.embed_tokens.device
        ids = input_ids.reshape(-1).to(dev)
        pos = torch.arange(L, dtype=torch.int32, device=dev).repeat(B)
        cos, sin = self.rope(dev, L)
        pre = UNIT_PRE[0]
        if pre is not None:
            pre(self.embed_tokens, False)
        h = EmbeddingFn.apply(ids, self.embed_tokens)
        if cfg.embedding_multiplier != 1.0:
            h = h * self._embedding_scale(h.dtype)
        meta = (B, L, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps,
                bool(self.grad_checkpointing and torch.is_grad_enabled()))
        rmul = float(cfg.residual_multiplier)
        tables = self.layer_rope(cos, sin)
        meta7 = meta
        for li, (layer, (cos, sin)) in enumerate(zip(self.layers, tables)):
            meta = meta7 + (cfg.layer_window(li, L),)       # the layer's sliding window when the sequence is longer
            if pre is not None:
                pre(layer.first_param, False)
            if LAYER_WEIGHTS_PRE[0] is not None:
                LAYER_WEIGHTS_PRE[0](layer.first_param)
            if cfg.sandwich:
                from .sandwich import SandwichLayerFn
                g = lambda n: getattr(layer, n, None)
                h = SandwichLayerFn.apply(h, pos, cos, sin,
                                          meta + (2 if cfg.qk_norm_full else 3 if cfg.qk_norm_after_rope
                                                  else int(cfg.qk_norm), layer.first_param, cfg.mlp_act),
                                          layer.qkv_proj, layer.o_proj, layer.gate_up_proj, layer.down_proj,
                                          g("input_layernorm"), g("post_attention_layernorm"), g("attn_out_norm"),
                                          g("mlp_out_norm"), g("qkv_bias"), g("q_norm"), g("k_norm"))
                continue
            if cfg.num_local_experts:
                from .moe import AttnBlockFn, MoEBlockFn
                h = AttnBlockFn.apply(h, pos, cos, sin, layer.input_layernorm, layer.qkv_proj, layer.o_proj, meta,
                                      getattr(layer, "qkv_bias", None), getattr(layer, "q_norm", None),
                                      getattr(layer, "k_norm", None), rmul)
                h = MoEBlockFn.apply(h, layer.post_attention_layernorm, layer.router, layer.gate_up_proj,
                                     layer.down_proj, (cfg.rms_norm_eps, cfg.num_experts_per_tok, meta[6],
                                                       layer.input_layernorm, cfg.moe_renormalize, rmul),
                                     getattr(layer, "shared_gate_up_proj", None),
                                     getattr(layer, "shared_down_proj", None),
                                     getattr(layer, "shared_expert_gate", None))
                continue
            h = DecoderLayerFn.apply(h, pos, cos, sin, layer.input_layernorm, layer.qkv_proj, layer.o_proj,
                                     layer.post_attention_layernorm, layer.gate_up_proj, layer.down_proj, meta,
                                     getattr(layer, "qkv_bias", None), getattr(layer, "q_norm", None),
                                     getattr(layer, "k_norm", None), getattr(layer, "o_bias", None),
                                     getattr(layer, "gate_up_bias", None), getattr(layer, "down_bias", None), rmul)
        if pre is not None:
            pre(self.norm, False)
        y = FinalNormFn.apply(h, self.norm, cfg.rms_norm_eps)
        # logits = y W^T / logits_scaling: the division rides on the hidden rows, which every head (fused loss, top-K
        # collection, full logits) multiplies by the same matrix
        return y if cfg.logits_scaling == 1.0 else y * (1.0 / cfg.logits_scaling)

    @torch.no_grad()
    def hidden_states_chunked(self, input_ids: torch.Tensor, chunk_len: int) -> torch.Tensor:
        """Inference-only forward in chunks of ``chunk_len`` positions against a key / value cache - the reference's
        long-context mechanism (classes/teacher/inference_worker.py:38-48: ``max_input_len = seq_chunk_len`` with an
        ExLlamaV2 cache). Per chunk the activations are [B*chunk_len, .] instead of [B*L, .]; every layer keeps its
        rotated keys and its values for all positions seen so far ([B, L, Hkv*d] each, zero-filled beyond), and the
        chunk's queries attend to positions <= their own. Same result as ``hidden_states`` up to rounding."""
        cfg = self.cfg
        B, L = input_ids.shape
        if chunk_len <= 0 or chunk_len >= L:
            return self.hidden_states(input_ids)
        dev = self.embed_tokens.device
        H, Hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        tables = self.layer_rope(*self.rope(dev, L))
        kv = Hkv * d
        caches = [(torch.zeros((B, L, kv), dtype=self.embed_tokens.dtype, device=dev),
                   torch.zeros((B, L, kv), dtype=self.embed_tokens.dtype, device=dev)) for _ in self.layers]
        out = torch.empty((B, L, cfg.hidden_size), dtype=self.embed_tokens.dtype, device=dev)
        ids = input_ids.to(dev)
        for c0 in range(0, L, chunk_len):
            n = min(chunk_len, L - c0)
            pos = torch.arange(c0, c0 + n, dtype=torch.int32, device=dev).repeat(B)
            h = basic.embed_fwd(ids[:, c0:c0 + n].reshape(-1), self.embed_tokens)
            if cfg.embedding_multiplier != 1.0:
                h = h * self._embedding_scale(h.dtype)
            for li, (layer, (kc, vc), (cos, sin)) in enumerate(zip(self.layers, caches, tables)):
                window = cfg.layer_window(li, L)
                if LAYER_WEIGHTS_PRE[0] is not None:
                    LAYER_WEIGHTS_PRE[0](layer.first_param)
                if cfg.sandwich:
                    from .sandwich import layer_inference

                    def attend(qkv, after_rotation=None, kc=kc, vc=vc, cos=cos, sin=sin, window=window):
                        basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
                        if after_rotation is not None:
                            qkv = after_rotation(qkv)
                        kc[:, c0:c0 + n] = qkv[:, H * d:(H + Hkv) * d].reshape(B, n, kv)
                        vc[:, c0:c0 + n] = qkv[:, (H + Hkv) * d:].reshape(B, n, kv)
                        return attention.attention_fwd_cached(qkv, kc, vc, B, n, c0, H, Hkv, d, window)
                    h = layer_inference(layer, cfg, h, attend, cfg.rms_norm_eps)
                    continue
                n1, _, _ = basic.rmsnorm_fwd(h, layer.input_layernorm, cfg.rms_norm_eps)
                if not hasattr(layer, "qkv_bias") and not cfg.qk_norm and not cfg.qk_norm_full:
                    qkv = basic.linear_rope_fwd(n1, layer.qkv_proj, pos, cos, sin, H + Hkv, d)
                else:
                    qkv = basic.linear_fwd(n1, layer.qkv_proj)
                    if hasattr(layer, "qkv_bias"):
                        basic.bias_add_(qkv, layer.qkv_bias)
                    if cfg.qk_norm_full:
                        from .sandwich import _qk_full_fwd
                        qkv, _ = _qk_full_fwd(qkv, layer.q_norm, layer.k_norm, H * d, Hkv * d, cfg.rms_norm_eps)
                    elif cfg.qk_norm:
                        qkv, _ = basic.headnorm_fwd(qkv, layer.q_norm, layer.k_norm, H, Hkv, d, cfg.rms_norm_eps)
                    basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
                kc[:, c0:c0 + n] = qkv[:, H * d:(H + Hkv) * d].reshape(B, n, kv)
                vc[:, c0:c0 + n] = qkv[:, (H + Hkv) * d:].reshape(B, n, kv)
                att = attention.attention_fwd_cached(qkv, kc, vc, B, n, c0, H, Hkv, d, window)
                rm = float(cfg.residual_multiplier)
                h1 = basic.gemm(att, layer.o_proj, residual=h, alpha=rm)
                if cfg.o_bias:
                    basic.bias_add_(h1, layer.o_bias if rm == 1.0 else layer.o_bias * rm)
                n2, _, _ = basic.rmsnorm_fwd(h1, layer.post_attention_layernorm, cfg.rms_norm_eps)
                if cfg.num_local_experts:
                    from .moe import moe_mlp
                    shared = ((layer.shared_gate_up_proj, layer.shared_down_proj, getattr(layer, "shared_expert_gate", None))
                              if cfg.shared_expert_intermediate_size else None)
                    branch = moe_mlp(n2, layer.router, layer.gate_up_proj, layer.down_proj, cfg.num_experts_per_tok,
                                     cfg.moe_renormalize, shared)
                    h = h1 + (branch if rm == 1.0 else branch * rm)
                    continue
                if cfg.mlp_bias:
                    act = basic.swiglu_fwd(basic.bias_add_(basic.linear_fwd(n2, layer.gate_up_proj), layer.gate_up_bias))
                    h = basic.bias_add_(basic.gemm(act, layer.down_proj, residual=h1, alpha=rm),
                                        layer.down_bias if rm == 1.0 else layer.down_bias * rm)
                    continue
                _, act = basic.linear_swiglu_fwd(n2, layer.gate_up_proj)
                h = basic.gemm(act, layer.down_proj, residual=h1, alpha=rm)
            y, _, _ = basic.rmsnorm_fwd(h, self.norm, cfg.rms_norm_eps)
            if cfg.logits_scaling != 1.0:
                y = y * (1.0 / cfg.logits_scaling)
            out[:, c0:c0 + n] = y.reshape(B, n, -1)
        return out.reshape(B * L, -1)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Full logits [B, L, V] (collection without the fused top-K head, tests). Training never calls this."""
        B, L = input_ids.shape
        hs = self.hidden_states(input_ids)
        return LinearFn.apply(hs, self.lm_head).reshape(B, L, -1)

    # ---- HF naming
    def named_hf_parameters(self):
        """Yields (hf_name, parameter, row_slice or None) - fused tensors appear once per HF tensor they hold."""
        cfg = self.cfg
        yield "model.embed_tokens.weight", self.embed_tokens, None
        q, kv, f = cfg.q_size, cfg.kv_size, cfg.intermediate_size
        for i, l in enumerate(self.layers):
            pre = f"model.layers.{i}."
            if cfg.model_type == "gemma3_text":      # Llama's name for the norm in front of the MLP means the one behind attention
                yield pre + "input_layernorm.weight", l.input_layernorm, None
                yield pre + "self_attn.q_proj.weight", l.qkv_proj, slice(0, q)
                yield pre + "self_attn.k_proj.weight", l.qkv_proj, slice(q, q + kv)
                yield pre + "self_attn.v_proj.weight", l.qkv_proj, slice(q + kv, q + 2 * kv)
                yield pre + "self_attn.q_norm.weight", l.q_norm, None
                yield pre + "self_attn.k_norm.weight", l.k_norm, None
                yield pre + "self_attn.o_proj.weight", l.o_proj, None
                yield pre + "post_attention_layernorm.weight", l.attn_out_norm, None
                yield pre + "pre_feedforward_layernorm.weight", l.post_attention_layernorm, None
                yield pre + "mlp.gate_proj.weight", l.gate_up_proj, slice(0, f)
                yield pre + "mlp.up_proj.weight", l.gate_up_proj, slice(f, 2 * f)
                yield pre + "mlp.down_proj.weight", l.down_proj, None
                yield pre + "post_feedforward_layernorm.weight", l.mlp_out_norm, None
                continue
            if cfg.model_type in ("olmo2", "olmo3", "exaone4", "glm", "glm4"):
                glm = cfg.model_type in ("glm", "glm4")
                if glm:
                    yield pre + "input_layernorm.weight", l.input_layernorm, None
                yield pre + "self_attn.q_proj.weight", l.qkv_proj, slice(0, q)
                yield pre + "self_attn.k_proj.weight", l.qkv_proj, slice(q, q + kv)
                yield pre + "self_attn.v_proj.weight", l.qkv_proj, slice(q + kv, q + 2 * kv)
                if cfg.attention_bias:
                    yield pre + "self_attn.q_proj.bias", l.qkv_bias, slice(0, q)
                    yield pre + "self_attn.k_proj.bias", l.qkv_bias, slice(q, q + kv)
                    yield pre + "self_attn.v_proj.bias", l.qkv_bias, slice(q + kv, q + 2 * kv)
                if cfg.qk_norm_full or cfg.qk_norm:
                    yield pre + "self_attn.q_norm.weight", l.q_norm, None
                    yield pre + "self_attn.k_norm.weight", l.k_norm, None
                yield pre + "self_attn.o_proj.weight", l.o_proj, None
                if glm:      # GLM keeps Llama's name for the norm in front of the MLP and stores gate / up fused
                    if cfg.post_norm:
                        yield pre + "post_self_attn_layernorm.weight", l.attn_out_norm, None
                    yield pre + "post_attention_layernorm.weight", l.post_attention_layernorm, None
                    yield pre + "mlp.gate_up_proj.weight", l.gate_up_proj, None
                    yield pre + "mlp.down_proj.weight", l.down_proj, None
                    if cfg.post_norm:
                        yield pre + "post_mlp_layernorm.weight", l.mlp_out_norm, None
                else:        # OLMo 2 uses that name for the norm BEHIND the attention
                    yield pre + "post_attention_layernorm.weight", l.attn_out_norm, None
                    yield pre + "mlp.gate_proj.weight", l.gate_up_proj, slice(0, f)
                    yield pre + "mlp.up_proj.weight", l.gate_up_proj, slice(f, 2 * f)
                    yield pre + "mlp.down_proj.weight", l.down_proj, None
                    yield pre + "post_feedforward_layernorm.weight", l.mlp_out_norm, None
                continue
            yield pre + "input_layernorm.weight", l.input_layernorm, None
            if cfg.model_type == "phi3":     # the checkpoint stores the fused projections, in this model's own order
                yield pre + "self_attn.qkv_proj.weight", l.qkv_proj, None
                yield pre + "self_attn.o_proj.weight", l.o_proj, None
                yield pre + "post_attention_layernorm.weight", l.post_attention_layernorm, None
                yield pre + "mlp.gate_up_proj.weight", l.gate_up_proj, None
                yield pre + "mlp.down_proj.weight", l.down_proj, None
                continue
            yield pre + "self_attn.q_proj.weight", l.qkv_proj, slice(0, q)
            yield pre + "self_attn.k_proj.weight", l.qkv_proj, slice(q, q + kv)
            yield pre + "self_attn.v_proj.weight", l.qkv_proj, slice(q + kv, q + 2 * kv)
            if cfg.attention_bias:
                yield pre + "self_attn.q_proj.bias", l.qkv_bias, slice(0, q)
                yield pre + "self_attn.k_proj.bias", l.qkv_bias, slice(q, q + kv)
                yield pre + "self_attn.v_proj.bias", l.qkv_bias, slice(q + kv, q + 2 * kv)
            if cfg.qk_norm and cfg.model_type == "hunyuan_v1_dense":
                yield pre + "self_attn.query_layernorm.weight", l.q_norm, None
                yield pre + "self_attn.key_layernorm.weight", l.k_norm, None
            elif cfg.qk_norm or cfg.qk_norm_full:
                yield pre + "self_attn.q_norm.weight", l.q_norm, None
                yield pre + "self_attn.k_norm.weight", l.k_norm, None
            yield pre + "self_attn.o_proj.weight", l.o_proj, None
            if cfg.o_bias:
                yield pre + "self_attn.o_proj.bias", l.o_bias, None
            yield pre + "post_attention_layernorm.weight", l.post_attention_layernorm, None
            if cfg.mlp_bias:
                yield pre + "mlp.gate_proj.bias", l.gate_up_bias, slice(0, f)
                yield pre + "mlp.up_proj.bias", l.gate_up_bias, slice(f, 2 * f)
                yield pre + "mlp.down_proj.bias", l.down_bias, None
            if cfg.model_type in ("granitemoe", "granitemoeshared"):      # stacked tensors, in this model's own order
                yield pre + "block_sparse_moe.router.layer.weight", l.router, None
                yield pre + "block_sparse_moe.input_linear.weight", l.gate_up_proj, None
                yield pre + "block_sparse_moe.output_linear.weight", l.down_proj, None
                if cfg.shared_expert_intermediate_size:
                    yield pre + "shared_mlp.input_linear.weight", l.shared_gate_up_proj, None
                    yield pre + "shared_mlp.output_linear.weight", l.shared_down_proj, None
                continue
            if cfg.shared_expert_intermediate_size:
                fs = cfg.shared_expert_intermediate_size
                yield pre + "mlp.shared_expert.gate_proj.weight", l.shared_gate_up_proj, slice(0, fs)
                yield pre + "mlp.shared_expert.up_proj.weight", l.shared_gate_up_proj, slice(fs, 2 * fs)
                yield pre + "mlp.shared_expert.down_proj.weight", l.shared_down_proj, None
                yield pre + "mlp.shared_expert_gate.weight", l.shared_expert_gate, None
            if cfg.num_local_experts and cfg.model_type in ("qwen3_moe", "qwen2_moe", "olmoe"):
                yield pre + "mlp.gate.weight", l.router, None
                for e in range(cfg.num_local_experts):
                    ex = pre + f"mlp.experts.{e}."
                    yield ex + "gate_proj.weight", l.gate_up_proj, (e, slice(0, f))
                    yield ex + "up_proj.weight", l.gate_up_proj, (e, slice(f, 2 * f))
                    yield ex + "down_proj.weight", l.down_proj, (e,)
                continue
            if cfg.num_local_experts:      # Mixtral names: w1 = gate, w3 = up, w2 = down
                yield pre + "block_sparse_moe.gate.weight", l.router, None
                for e in range(cfg.num_local_experts):
                    ex = pre + f"block_sparse_moe.experts.{e}."
                    yield ex + "w1.weight", l.gate_up_proj, (e, slice(0, f))
                    yield ex + "w3.weight", l.gate_up_proj, (e, slice(f, 2 * f))
                    yield ex + "w2.weight", l.down_proj, (e,)
                continue
            yield pre + "mlp.gate_proj.weight", l.gate_up_proj, slice(0, f)
            yield pre + "mlp.up_proj.weight", l.gate_up_proj, slice(f, 2 * f)
            yield pre + "mlp.down_proj.weight", l.down_proj, None
        yield "model.norm.weight", self.norm, None
        if not cfg.tie_word_embeddings:
            yield "lm_head.weight", self.lm_head, None

    def _rotary_row_order(self) -> torch.Tensor:
        """Row order inside one head that turns a checkpoint whose rotary pairs are neighbours (2i, 2i+1) into this
        model's layout, where element i pairs with i + rot/2: q . k is unchanged when both are permuted alike."""
        d, rot = self.cfg.head_dim, self.cfg.rotary_dim
        return torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, d)])

    def _permute_rotary_rows(self, sd: dict, to_checkpoint: bool) -> dict:
        order = self._rotary_row_order()
        d = self.cfg.head_dim
        out = dict(sd)
        for k, v in sd.items():
            if k.endswith(("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.q_proj.bias",
                           "self_attn.k_proj.bias")):
                heads = v.reshape(v.shape[0] // d, d, *v.shape[1:])
                idx = order.to(v.device)
                if to_checkpoint:
                    t = torch.empty_like(heads)
                    t[:, idx] = heads
                else:
                    t = heads[:, idx]
                out[k] = t.reshape(v.shape)
        return out

    @staticmethod
    def _shift_norm_weights(sd: dict, by: float) -> dict:
        """Gemma stores every RMSNorm weight minus one (the module multiplies by 1 + w): this model keeps the factor."""
        return {k: (v + by if k.endswith("norm.weight") else v) for k, v in sd.items()}

    def to_hf_state_dict(self) -> dict[str, torch.Tensor]:
        sd = self._to_hf_state_dict()
        if self.cfg.rope_interleaved:
            sd = self._permute_rotary_rows(sd, to_checkpoint=True)
        if self.cfg.norm_plus_one:
            sd = self._shift_norm_weights(sd, -1.0)
        return sd

    def _to_hf_state_dict(self) -> dict[str, torch.Tensor]:
        if self.quant is None:
            return {n: (p.data if sl is None else p.data[sl]) for n, p, sl in self.named_hf_parameters()}
        # frozen low-bit matrices live packed; their parameters are views of a rotating buffer: export dequantised copies
        out, fresh = {}, {}
        for i, layer in enumerate(self.layers):
            for name, t in self.quant.dequantized(i).items():
                fresh[id(getattr(layer, name))] = t
        for n, p, sl in self.named_hf_parameters():
            src = fresh.get(id(p), p.data)
            out[n] = src if sl is None else src[sl]
        return out

    def quantize_frozen_linears(self, kind: str) -> "LlamaModel":
        """Turns the decoder layers' matrices into frozen NF4 (``"nf4"``) or int8 weights: what the reference's
        ``training_precision`` 4bit / 8bit do through bitsandbytes (classes/student/model.py:138-148). Embeddings,
        norms and the LM head stay in the compute dtype and keep training."""
        from ..ops.quant import FrozenQuantLinears
        if self.cfg.num_local_experts:
            raise NotImplementedError("frozen low-bit weights (training_precision 4bit / 8bit) are not built for "
                                      "mixture-of-experts models: use bf16")
        self.quant = FrozenQuantLinears(self, kind)
        LAYER_WEIGHTS_PRE[0] = self.quant.before_layer
        return self

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict[str, torch.Tensor], strict: bool = True) -> None:
        if self.cfg.num_local_experts and any(k.endswith("mlp.experts.gate_up_proj") for k in sd):
            sd = self._unstack_experts(sd)
        wrapped = [k for k in sd if "language_model" in k and k.endswith("embed_tokens.weight")]
        if wrapped:
            # a multimodal wrapper (Gemma 3): the language model's tensors under their plain names, the rest left out.
            # Releases of the wrapper differ in the prefix (language_model.model. / model.language_model. / ...)
            prefix = wrapped[0][: -len("embed_tokens.weight")]
            plain = {"model." + k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}
            plain.update({"lm_head.weight": v for k, v in sd.items() if k.endswith("lm_head.weight")})
            sd = plain
        if self.cfg.rope_interleaved:
            sd = self._permute_rotary_rows(sd, to_checkpoint=False)
        if self.cfg.norm_plus_one:
            sd = self._shift_norm_weights(sd, 1.0)
        seen = set()
        for n, p, sl in self.named_hf_parameters():
            if n not in sd:
                if n == "lm_head.weight" and "model.embed_tokens.weight" in sd:
                    p.copy_(sd["model.embed_tokens.weight"].to(p.dtype))
                    continue
                if strict:
                    raise KeyError(f"missing tensor {n}")
                continue
            (p if sl is None else p[sl]).copy_(sd[n].to(p.dtype))
            seen.add(n)
        extra = [k for k in sd if k not in seen and k != "lm_head.weight" and not k.endswith("rotary_emb.inv_freq")]
        if strict and extra:
            raise KeyError(f"unexpected tensors {extra[:5]}")

    def _unstack_experts(self, sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """Newer HuggingFace releases keep a Mixtral layer's experts as stacked tensors (``mlp.experts.gate_up_proj``
        [E, 2f, h], ``mlp.experts.down_proj`` [E, h, f], router ``mlp.gate.weight``); the published checkpoints - and
        this model's own names - list them per expert under ``block_sparse_moe``."""
        f = self.cfg.intermediate_size
        qwen = self.cfg.model_type in ("qwen3_moe", "qwen2_moe", "olmoe")
        block = "mlp." if qwen else "block_sparse_moe."
        gate_n, up_n, down_n = ("gate_proj", "up_proj", "down_proj") if qwen else ("w1", "w3", "w2")
        out = {}
        for k, v in sd.items():
            if k.endswith("mlp.gate.weight"):
                out[k.replace("mlp.gate.weight", block + "gate.weight")] = v
            elif k.endswith("mlp.experts.gate_up_proj"):
                pre = k[: -len("mlp.experts.gate_up_proj")] + block + "experts."
                for e in range(v.shape[0]):
                    out[f"{pre}{e}.{gate_n}.weight"] = v[e, :f]
                    out[f"{pre}{e}.{up_n}.weight"] = v[e, f:]
            elif k.endswith("mlp.experts.down_proj"):
                pre = k[: -len("mlp.experts.down_proj")] + block + "experts."
                for e in range(v.shape[0]):
                    out[f"{pre}{e}.{down_n}.weight"] = v[e]
            else:
                out[k] = v
        return out

    def apply_freeze(self, freeze_layers: list[str]) -> list[str]:
        """requires_grad=False for every parameter one of whose HF names contains a listed substring
        (reference: classes/student/model.py:214-218). A fused tensor freezes only if all its parts match."""
        by_param: dict[int, list[bool]] = {}
        params = {}
        for n, p, _ in self.named_hf_parameters():
            hit = any(s in n for s in (freeze_layers or []))
            by_param.setdefault(id(p), []).append(hit)
            params[id(p)] = (p, n)
        frozen = []
        for pid, hits in by_param.items():
            if hits and all(hits):
                params[pid][0].requires_grad = False
                frozen.append(params[pid][1])
        return frozen


def build_model(cfg: LlamaConfig, dtype=torch.bfloat16, device="cpu", seed: int | None = 0) -> LlamaModel:
    m = LlamaModel(cfg, dtype=dtype, device=device)
    if seed is not None:
        m.init_weights(seed)
    return m
