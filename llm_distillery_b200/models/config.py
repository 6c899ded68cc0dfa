"""Configuration of the decoder models: one dataclass for every family that is read (``LlamaConfig``), its mapping from
and to HuggingFace ``config.json`` files, parameter / FLOP counts, and the named presets of the benchmarks and tests.

The reference reads model configs through ``AutoConfig`` / ``AutoModelForCausalLM`` (classes/student/model.py:194-201,
classes/base_model.py:20-48). Here a config.json is mapped onto the switches of one decoder implementation
(models/llama.py with models/moe.py and models/sandwich.py): where the norms sit, which projections carry biases, how
queries and keys are normalised and rotated, whether the MLP is a mixture of experts. Variants that are not built are
refused when the config is read, not at the first forward. Keys this code does not know are carried in ``extra`` and
written back unchanged.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_hidden_layers: int = 22
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    bos_token_id: int = 1
    eos_token_id: int = 2
    model_type: str = "llama"         # llama | mistral | qwen2 (q/k/v bias) | phi3 (fused projections in the checkpoint)
                                      # | mixtral, qwen3_moe, qwen2_moe (sparse mixtures of experts, models/moe.py) | qwen3 | granite
    num_local_experts: int = 0        # > 0: every layer's MLP is that many SwiGLU experts behind a linear router
    num_experts_per_tok: int = 2
    moe_renormalize: bool = True      # router weights renormalised over the chosen experts (Mixtral; Qwen3-MoE norm_topk_prob)
    shared_expert_intermediate_size: int = 0   # > 0 (Qwen2-MoE): a dense SwiGLU expert of this width for every token,
                                               # scaled by a per-token sigmoid gate, beside the routed experts
    shared_expert_gated: bool = True           # false: the shared expert's output is added as it is (Granite MoE)
    attention_bias: bool = False      # bias on the q/k/v projections (Qwen2 family; Llama configs with attention_bias)
    o_bias: bool = False              # bias on o_proj as well (HuggingFace Llama's attention_bias = true, e.g. Granite code)
    mlp_bias: bool = False            # bias on gate / up / down projections (HuggingFace Llama's mlp_bias)
    # Granite: the embedding output, the attention scores, each branch before it joins the residual stream and the
    # logits carry fixed multipliers
    embedding_multiplier: float = 1.0
    attention_multiplier: float | None = None      # replaces 1 / sqrt(head_dim)
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0                    # logits are DIVIDED by this
    rope_scaling: dict | None = None  # HuggingFace dict; types default / linear / dynamic / llama3 / yarn / longrope (ops.basic.rope_tables)
    head_dim_override: int | None = None   # HuggingFace ``head_dim`` when it is not hidden_size / num_attention_heads
    no_rope_layers: list | None = None     # SmolLM3: one flag per layer, 1 = rotary embedding, 0 = no positional rotation
    partial_rotary_factor: float = 1.0     # < 1: only the first int(head_dim * factor) elements of a head rotate (Phi-4-mini)
    qk_norm: bool = False             # Qwen3: RMSNorm over every query and key head (one weight each) before RoPE
    qk_norm_after_rope: bool = False  # HunYuan: the per-head q/k norms act on the rotated queries and keys
    qk_norm_full: bool = False        # OLMo 2: one RMSNorm over the whole query projection, one over the key projection
    pre_norm: bool = True             # RMSNorm on the way into the attention and MLP branches (false: OLMo 2)
    post_norm: bool = False           # RMSNorm on the way out of both branches (OLMo 2, GLM-4 0414; models/sandwich.py)
    mlp_act: str = "silu"             # the gate's activation: silu (SwiGLU) or gelu_tanh (Gemma's GeGLU; PyTorch ops)
    norm_plus_one: bool = False       # checkpoint layout: RMSNorm weights are stored minus one (Gemma); converted at load / save
    rope_local_theta: float | None = None      # Gemma 3: the windowed layers rotate with this base, without scaling
    embedding_multiplier_rounded: bool = False # Gemma: the embedding multiplier is rounded to the model's dtype first
    rope_interleaved: bool = False    # checkpoint layout: rotary pairs are neighbours (GLM); rows are permuted at load / save
    sliding_window: int | None = None  # a query sees the last ``sliding_window`` positions; matters for longer sequences only
    window_layers: list | None = None  # one flag per layer, 1 = windowed; None: every layer (when sliding_window is set)
    pad_token_id: int | None = None
    extra: dict = field(default_factory=dict)   # other keys of the source config.json, written back unchanged

    @property
    def head_dim(self) -> int:
        return self.head_dim_override or self.hidden_size // self.num_attention_heads

    def layer_window(self, layer: int, seq_len: int) -> int | None:
        """The sliding window that layer's attention must apply to sequences of ``seq_len``, or None when plain causal
        attention is exact (no window, a layer that attends to everything, a sequence inside the window)."""
        w = self.sliding_window
        if not w or seq_len <= w or (self.window_layers is not None and not self.window_layers[layer]):
            return None
        return int(w)

    def check_gpu_kernels(self) -> None:
        """Raises when a shape is outside what the sm_100a kernels take, in words, before any kernel is launched."""
        problems = []
        if self.head_dim % 16:
            problems.append(f"head_dim {self.head_dim}: a multiple of 16 is needed (64 and 128 run the flash-attention "
                            "kernels, other sizes PyTorch's attention)")
        if self.rotary_dim % 16:
            problems.append(f"rotary width {self.rotary_dim}: the rotary kernel moves 16-byte vectors (a multiple of 16)")
        for name, v in (("hidden_size", self.hidden_size), ("intermediate_size", self.intermediate_size),
                        ("shared_expert_intermediate_size", self.shared_expert_intermediate_size)):
            if v % 8:
                problems.append(f"{name} {v}: rows of the GEMM operands must be multiples of 16 bytes (8 elements)")
        if problems:
            raise NotImplementedError("this model does not fit the GPU kernels - " + "; ".join(problems))

    @property
    def sandwich(self) -> bool:
        """Whether the layers take the general node of models/sandwich.py instead of the fused pre-norm layer."""
        if self.num_local_experts and self.pre_norm and not self.post_norm and not self.qk_norm_after_rope:
            return False         # experts: the two nodes of models/moe.py (their attention half takes either q/k norm)
        return (self.post_norm or not self.pre_norm or self.qk_norm_full or self.qk_norm_after_rope
                or self.mlp_act != "silu")

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_params(self) -> int:
        h, f, V, Lr = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        E = self.num_local_experts
        per_layer = h * (self.q_size + 2 * self.kv_size) + self.q_size * h + 3 * h * f * max(E, 1) + E * h + 2 * h
        if self.shared_expert_intermediate_size:
            per_layer += 3 * h * self.shared_expert_intermediate_size + (h if self.shared_expert_gated else 0)
        if self.attention_bias:
            per_layer += self.q_size + 2 * self.kv_size
        if self.qk_norm:
            per_layer += 2 * self.head_dim
        if self.qk_norm_full:
            per_layer += self.q_size + self.kv_size
        if not self.pre_norm:
            per_layer -= 2 * h
        if self.post_norm:
            per_layer += 2 * h
        if self.o_bias:
            per_layer += h
        if self.mlp_bias:
            per_layer += 2 * f + h
        return Lr * per_layer + V * h * (1 if self.tie_word_embeddings else 2) + h

    def flops_per_token_fwd(self, seq_len: int) -> float:
        h, f, V, Lr = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        mlp = 3 * h * f * (self.num_experts_per_tok if self.num_local_experts else 1) + self.num_local_experts * h
        if self.shared_expert_intermediate_size:
            mlp += 3 * h * self.shared_expert_intermediate_size + h
        lin = 2 * (Lr * (h * (self.q_size + 2 * self.kv_size) + self.q_size * h + mlp) + V * h)
        attn = Lr * 4 * self.q_size * seq_len / 2  # causal
        return lin + attn

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        extra = d.pop("extra") or {}
        for k in ("rope_scaling", "sliding_window", "pad_token_id"):
            if d[k] is None:
                d.pop(k)
        hd = d.pop("head_dim_override")
        if hd:
            d["head_dim"] = hd
        if d["partial_rotary_factor"] == 1.0:
            d.pop("partial_rotary_factor")
        nope = d.pop("no_rope_layers")
        win_layers = d.pop("window_layers")
        renorm = d.pop("moe_renormalize")
        if not self.num_local_experts:
            d.pop("num_local_experts")
            d.pop("num_experts_per_tok")
        qk = d.pop("qk_norm")
        for k in self._SWITCHES:      # implied by the model type
            d.pop(k)
        shared_f = d.pop("shared_expert_intermediate_size")
        d.pop("shared_expert_gated")
        gran = {k: d.pop(k) for k in ("embedding_multiplier", "attention_multiplier", "residual_multiplier", "logits_scaling")}
        held = dict(nope=nope, win_layers=win_layers, renorm=renorm, shared_f=shared_f, gran=gran, extra=extra)
        d.update(hidden_act="silu", torch_dtype="bfloat16")
        mt = self.model_type
        if mt in ("llama", "mistral", "qwen2", "granite") and self.attention_bias and not self.o_bias:
            mt = "qwen2"          # q/k/v bias without o_proj bias is the Qwen2 layout in HuggingFace terms
            d["model_type"] = "qwen2"
        d["architectures"] = [_ARCHITECTURES[mt]]
        _FAMILY_WRITERS.get(mt, _write_plain)(self, d, held)
        if win_layers is not None and self.sliding_window is not None and mt not in ("exaone4", "gemma3_text"):
            d["layer_types"] = ["sliding_attention" if f else "full_attention" for f in win_layers]
        d.pop("o_bias")
        d.pop("mlp_bias", None)
        if self.o_bias or self.mlp_bias:          # HuggingFace's Llama: attention_bias covers q, k, v AND o
            d.update(architectures=["LlamaForCausalLM"], model_type="llama", attention_bias=bool(self.o_bias),
                     mlp_bias=bool(self.mlp_bias))
        if self.model_type in self._MULTIPLIER_TYPES:
            d.update(architectures=[_ARCHITECTURES[self.model_type]], model_type=self.model_type, **gran)
            if d.get("attention_multiplier") is None:
                d["attention_multiplier"] = 1.0 / math.sqrt(self.head_dim)
        return {**extra, **d}

    _KNOWN_TYPES = ("llama", "mistral", "qwen2", "phi3", "mixtral", "qwen3", "qwen3_moe", "qwen2_moe", "granite",
                    "smollm3", "olmo2", "glm", "glm4", "exaone4", "helium", "ernie4_5", "seed_oss", "hunyuan_v1_dense",
                    "olmoe", "granitemoe", "granitemoeshared", "gemma", "gemma3_text", "olmo3", "ministral")
    # what HuggingFace's attention_bias puts a bias on, per family: q, k and v only / the o projection as well (built for
    # the second group, refused for every other family); families whose MLP may carry biases; families with experts
    _QKV_BIAS_TYPES = ("qwen2", "qwen2_moe", "glm", "glm4", "seed_oss", "helium")
    _QKVO_BIAS_TYPES = ("llama", "mistral", "granite")
    _MLP_BIAS_TYPES = ("llama", "mistral", "granite")
    _EXPERT_TYPES = ("mixtral", "qwen3_moe", "qwen2_moe", "olmoe", "granitemoe", "granitemoeshared")
    _MULTIPLIER_TYPES = ("granite", "granitemoe", "granitemoeshared")
    _GELU_TYPES = ("gemma", "gemma3_text")
    _SWITCHES = ("qk_norm_full", "qk_norm_after_rope", "pre_norm", "post_norm", "rope_interleaved", "mlp_act",
                 "norm_plus_one", "rope_local_theta", "embedding_multiplier_rounded")      # set by the type alone

    @classmethod
    def from_hf_dict(cls, d: dict) -> "LlamaConfig":
        d = dict(d)
        if d.get("model_type") not in cls._KNOWN_TYPES and isinstance(d.get("text_config"), dict):
            # a multimodal wrapper (gemma3, mistral3, llava ...): its language model is read, and saved, as a text model
            text = dict(d["text_config"])
            if d.get("model_type") == "gemma3":
                text["model_type"] = "gemma3_text"
            elif text.get("model_type") in cls._KNOWN_TYPES:
                missing = [k for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                       "num_attention_heads") if text.get(k) is None]
                if missing:      # such blocks list only what differs from HuggingFace's defaults for that text model
                    raise ValueError(f"the text_config of this {d.get('model_type')} checkpoint does not name {missing}")
            else:
                raise NotImplementedError(f"model_type {d.get('model_type')!r} with a {text.get('model_type')!r} language "
                                          f"model: only Llama-shaped decoders are built {cls._KNOWN_TYPES}")
            d = text
        keys = {f for f in cls.__dataclass_fields__} - {"extra"}
        kw = {k: v for k, v in d.items() if k in keys}
        mt = d.get("model_type", "llama")
        rp = d.get("rope_parameters")
        if isinstance(rp, dict):       # newer HuggingFace releases write theta and the scaling keys into one dict
            if rp.get("rope_theta") is not None and d.get("rope_theta") is None:
                kw["rope_theta"] = float(rp["rope_theta"])
            if rp.get("rope_type", rp.get("type")) not in (None, "default") and not d.get("rope_scaling"):
                kw["rope_scaling"] = {k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")}
            if rp.get("partial_rotary_factor") is not None and d.get("partial_rotary_factor") is None:
                kw["partial_rotary_factor"] = float(rp["partial_rotary_factor"])
        for k in ("bos_token_id", "eos_token_id"):
            if k in kw and kw[k] is None:
                kw.pop(k)
        if mt not in cls._KNOWN_TYPES:
            raise NotImplementedError(f"model_type {mt!r}: only Llama-shaped decoders are built {cls._KNOWN_TYPES}")
        # keys that only some families may carry
        for k in cls._SWITCHES + ("window_layers",):
            kw.pop(k, None)
        if mt not in ("smollm3", "exaone4"):
            kw.pop("no_rope_layers", None)
        if kw.get("shared_expert_intermediate_size") and mt != "qwen2_moe":
            raise NotImplementedError(f"a shared expert on model_type {mt!r} is not built (qwen2_moe is)")
        if mt == "qwen3" and d.get("num_experts"):
            raise NotImplementedError("experts in a config of model_type qwen3: the mixture-of-experts type is qwen3_moe")
        if kw.get("num_local_experts") and mt not in cls._EXPERT_TYPES:
            raise NotImplementedError(f"experts on model_type {mt!r} are not built (mixtral is)")
        if mt not in cls._MULTIPLIER_TYPES:
            for k in ("embedding_multiplier", "attention_multiplier", "residual_multiplier", "logits_scaling"):
                kw.pop(k, None)           # other families may carry such keys with another meaning
        # the family's own keys and switches
        reader = _FAMILY_READERS.get(mt)
        if reader is not None:
            reader(mt, d, kw)
        # biases
        if mt in cls._QKV_BIAS_TYPES:
            pass                           # the family's reader has set attention_bias: q, k and v only
        elif kw.get("attention_bias"):
            if mt not in cls._QKVO_BIAS_TYPES:
                raise NotImplementedError(f"{mt} with attention_bias also puts a bias on o_proj, which is not built")
            kw["o_bias"] = True            # HuggingFace's Llama puts the bias on q, k, v and o
        if d.get("mlp_bias"):
            if mt not in cls._MLP_BIAS_TYPES:
                raise NotImplementedError(f"mlp_bias on model_type {mt!r} is not built")
            kw["mlp_bias"] = True
        act = d.get("hidden_activation") or d.get("hidden_act") or ("gelu_pytorch_tanh" if mt in cls._GELU_TYPES else "silu")
        if mt in cls._GELU_TYPES:
            if act not in ("gelu_pytorch_tanh", "gelu_tanh"):
                raise NotImplementedError(f"{mt} with hidden activation {act!r} is not built (gelu_pytorch_tanh is)")
        elif act not in ("silu", "swish"):
            raise NotImplementedError(f"hidden_act {act!r}: only SwiGLU (silu) is built for model_type {mt!r}")
        # heads
        kw["partial_rotary_factor"] = float(kw.get("partial_rotary_factor") or 1.0)
        if not 0.0 < kw["partial_rotary_factor"] <= 1.0:
            raise ValueError(f"partial_rotary_factor {kw['partial_rotary_factor']} is outside (0, 1]")
        if "num_key_value_heads" not in kw or kw["num_key_value_heads"] is None:
            kw["num_key_value_heads"] = kw.get("num_attention_heads", 32)
        hd = d.get("head_dim")
        if hd is not None and hd * kw.get("num_attention_heads", 32) != kw.get("hidden_size", 2048):
            if hd % 16:
                raise NotImplementedError(f"head_dim {hd}: the rotary and attention kernels need a multiple of 16")
            kw["head_dim_override"] = int(hd)       # e.g. Mistral-Nemo: 5120 hidden, 32 heads of 128
        dense_ffn = kw.pop("_dense_intermediate_size", None)
        cfg = cls(**kw)
        if cfg.rope_scaling is not None:       # fail at load time, not at the first forward
            kind = cfg.rope_scaling.get("rope_type", cfg.rope_scaling.get("type"))
            if kind == "su":                # the name older Phi-3 configs use
                kind = "longrope"
                cfg.rope_scaling = {**{k: v for k, v in cfg.rope_scaling.items() if k not in ("type", "rope_type")},
                                    "rope_type": "longrope"}
            if kind not in (None, "default", "linear", "dynamic", "llama3", "yarn", "longrope"):
                raise NotImplementedError(f"rope_scaling type {kind!r} is not built (default, linear, dynamic, llama3, "
                                          "yarn and longrope are)")
            if kind == "longrope" and not cfg.rope_scaling.get("original_max_position_embeddings"):
                orig = d.get("original_max_position_embeddings")
                if orig:          # Phi-3 keeps it beside the dict
                    cfg.rope_scaling = dict(cfg.rope_scaling, original_max_position_embeddings=int(orig))
        generated = {"architectures", "hidden_act", "torch_dtype", "mlp_bias", "use_sliding_window", "head_dim",
                     "num_experts", "moe_intermediate_size", "norm_topk_prob", "decoder_sparse_step", "mlp_only_layers",
                     "rope_parameters", "layer_types", "hidden_activation", "query_pre_attn_scalar",
                     "rope_local_base_freq", "final_logit_softcapping", "attn_logit_softcapping"}
        cfg.extra = {k: v for k, v in d.items() if k not in keys and k not in generated}
        if dense_ffn is not None:
            cfg.extra["dense_intermediate_size"] = dense_ffn
        return cfg

    @classmethod
    def from_pretrained(cls, path: str) -> "LlamaConfig":
        with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as f:
            return cls.from_hf_dict(json.load(f))


def _whole_if_close(x: float):
    """HuggingFace's Gemma 3 config types query_pre_attn_scalar as an integer."""
    return int(round(x)) if abs(x - round(x)) < 1e-6 else x


# ---------------------------------------------------------------------------------------------- per-family readers
# Each takes (model_type, the config.json dict, the keyword arguments collected so far) and sets the family's switches.
def _window_off_unless_used(d: dict, kw: dict) -> None:
    if not d.get("use_sliding_window", False) or kw.get("sliding_window") is None:
        kw["sliding_window"] = None        # Qwen-style configs carry a window that is switched off
        return
    n_layers = int(kw.get("num_hidden_layers", 32))
    types = d.get("layer_types")
    if types is not None:
        kw["window_layers"] = [int(t == "sliding_attention") for t in types]
    elif d.get("max_window_layers") is not None:       # the first ``max_window_layers`` layers attend to everything
        kw["window_layers"] = [int(i >= int(d["max_window_layers"])) for i in range(n_layers)]
    if kw.get("window_layers") is not None and not any(kw["window_layers"]):
        kw["sliding_window"], kw["window_layers"] = None, None


def _every_layer_sparse(mt: str, d: dict) -> None:
    if int(d.get("decoder_sparse_step", 1) or 1) != 1 or d.get("mlp_only_layers"):
        raise NotImplementedError(f"{mt} with dense layers between the sparse ones is not built")


def _read_qwen2(mt, d, kw):
    kw["attention_bias"] = True
    _window_off_unless_used(d, kw)


def _read_qwen3(mt, d, kw):
    kw["qk_norm"] = True
    _window_off_unless_used(d, kw)


def _read_qwen3_moe(mt, d, kw):
    _every_layer_sparse(mt, d)
    n_exp = int(d.get("num_experts") or d.get("num_local_experts") or 0)
    if n_exp < 1 or not d.get("moe_intermediate_size"):
        raise ValueError("a qwen3_moe config needs num_experts and moe_intermediate_size")
    kw.update(num_local_experts=n_exp, intermediate_size=int(d["moe_intermediate_size"]),
              moe_renormalize=bool(d.get("norm_topk_prob", False)), qk_norm=True,
              _dense_intermediate_size=d.get("intermediate_size"))
    _window_off_unless_used(d, kw)


def _read_qwen2_moe(mt, d, kw):        # Qwen2 attention (bias on q, k, v), routed experts plus a gated shared expert
    _every_layer_sparse(mt, d)
    n_exp = int(d.get("num_experts") or d.get("num_local_experts") or 0)
    if n_exp < 1 or not d.get("moe_intermediate_size") or not d.get("shared_expert_intermediate_size"):
        raise ValueError("a qwen2_moe config needs num_experts, moe_intermediate_size and shared_expert_intermediate_size")
    if not d.get("qkv_bias", True):
        raise NotImplementedError("qwen2_moe without the q/k/v bias is not built")
    kw.update(num_local_experts=n_exp, intermediate_size=int(d["moe_intermediate_size"]),
              shared_expert_intermediate_size=int(d["shared_expert_intermediate_size"]),
              moe_renormalize=bool(d.get("norm_topk_prob", False)), attention_bias=True,
              _dense_intermediate_size=d.get("intermediate_size"))
    _window_off_unless_used(d, kw)


def _read_mixtral(mt, d, kw):
    if int(kw.get("num_local_experts") or 0) < 1:
        raise ValueError(f"a {mt} config needs num_local_experts")


def _read_granite_moe(mt, d, kw):      # Granite's multipliers around Mixtral-style experts
    _read_mixtral(mt, d, kw)
    kw.update(moe_renormalize=True, shared_expert_gated=False,
              shared_expert_intermediate_size=int(d.get("shared_intermediate_size") or 0) if mt == "granitemoeshared" else 0)


def _read_olmoe(mt, d, kw):            # Llama layers, q/k norms over the whole projections, every MLP a mixture of experts
    n_exp = int(d.get("num_experts") or d.get("num_local_experts") or 0)
    if n_exp < 1:
        raise ValueError("an olmoe config needs num_experts")
    if d.get("clip_qkv"):
        raise NotImplementedError("olmoe with clip_qkv is not built")
    kw.update(num_local_experts=n_exp, qk_norm_full=True, moe_renormalize=bool(d.get("norm_topk_prob", False)))


def _read_smollm3(mt, d, kw):          # Llama blocks; every n-th layer applies no rotary embedding
    n_layers = int(kw.get("num_hidden_layers", 32))
    flags = d.get("no_rope_layers")
    if flags is None:
        step = int(d.get("no_rope_layer_interval", 4) or 4)
        flags = [int((i + 1) % step != 0) for i in range(n_layers)]
    if len(flags) != n_layers:
        raise ValueError(f"no_rope_layers lists {len(flags)} layers, the model has {n_layers}")
    kw["no_rope_layers"] = [int(bool(v)) for v in flags]
    _window_off_unless_used(d, kw)


def _read_olmo2(mt, d, kw):            # no norms in front of the branches, norms behind them, q/k norms over all heads
    kw.update(pre_norm=False, post_norm=True, qk_norm_full=True)


def _read_ministral(mt, d, kw):        # Mistral layers; the config says which of them are windowed
    types = d.get("layer_types")
    if kw.get("sliding_window") and types is not None and "sliding_attention" in types:
        kw["window_layers"] = [int(t == "sliding_attention") for t in types]
    elif types is not None:
        kw["sliding_window"] = None


def _read_olmo3(mt, d, kw):            # OLMo 2 layers, three of every four with a sliding window
    _read_olmo2(mt, d, kw)
    n_layers = int(kw.get("num_hidden_layers", 32))
    types = d.get("layer_types") or ["sliding_attention" if (i + 1) % 4 else "full_attention" for i in range(n_layers)]
    if "sliding_window" not in d:
        kw["sliding_window"] = 4096
    if kw.get("sliding_window") and "sliding_attention" in types:
        kw["window_layers"] = [int(t == "sliding_attention") for t in types]
    else:
        kw["sliding_window"] = None


def _read_exaone4(mt, d, kw):          # OLMo 2's placement of the norms with per-head q/k norms
    kw.update(pre_norm=False, post_norm=True, qk_norm=True)
    n_layers = int(kw.get("num_hidden_layers", 32))
    window = d.get("sliding_window")
    types = d.get("layer_types")
    if types is None and window is not None:
        pat = d.get("sliding_window_pattern", 4)
        if isinstance(pat, str):         # e.g. "LLLG": local (windowed) and global layers in turn
            types = ["sliding_attention" if pat[i % len(pat)].upper() == "L" else "full_attention" for i in range(n_layers)]
        else:
            types = ["sliding_attention" if (i + 1) % int(pat) else "full_attention" for i in range(n_layers)]
    if window is not None and types and "sliding_attention" in types:
        # hybrid checkpoints: windowed layers rotate, global layers apply no rotation
        kw["no_rope_layers"] = [int(t == "sliding_attention") for t in types]
        kw["window_layers"] = list(kw["no_rope_layers"])
    else:
        kw["sliding_window"] = None
        kw.pop("no_rope_layers", None)


def _read_interleaved(mt, d, kw):      # Helium, ERNIE 4.5: rotary pairs are neighbours in the checkpoint
    kw["rope_interleaved"] = True
    if d.get("use_bias"):
        raise NotImplementedError("ernie4_5 with use_bias puts a bias on every projection, which is not built")


def _read_seed_oss(mt, d, kw):
    if d.get("attention_out_bias"):
        raise NotImplementedError("seed_oss with a bias on o_proj is not built")
    kw["attention_bias"] = bool(d.get("attention_bias", True))


def _read_glm(mt, d, kw):              # rotary pairs are neighbours in the checkpoint; half of each head rotates
    kw.update(rope_interleaved=True, post_norm=(mt == "glm4"), attention_bias=bool(d.get("attention_bias", True)))
    if kw.get("partial_rotary_factor") is None:
        kw["partial_rotary_factor"] = 0.5


def _read_hunyuan(mt, d, kw):          # Llama layers with per-head q/k norms behind the rotation
    kw.update(qk_norm=True, qk_norm_after_rope=True)


def _read_gemma(mt, d, kw):            # Llama layers with GeGLU, norm weights stored minus one, scaled embeddings
    kw.update(mlp_act="gelu_tanh", norm_plus_one=True, embedding_multiplier_rounded=True,
              embedding_multiplier=float(kw.get("hidden_size", 2048)) ** 0.5)
    for k in ("final_logit_softcapping", "attn_logit_softcapping"):
        if d.get(k):
            raise NotImplementedError(f"{mt} with {k} is not built")
    if d.get("use_bidirectional_attention"):
        raise NotImplementedError(f"{mt} with bidirectional attention is not built")


# HuggingFace's defaults for Gemma 3 text configs: published text_config blocks list only what differs from them
_GEMMA3_TEXT_DEFAULTS = dict(vocab_size=262208, hidden_size=2304, intermediate_size=9216, num_hidden_layers=26,
                             num_attention_heads=8, num_key_value_heads=4, max_position_embeddings=131072,
                             rms_norm_eps=1e-6, tie_word_embeddings=True, sliding_window=4096, head_dim=256)


def _read_gemma3_text(mt, d, kw):      # Gemma with norms behind the branches, per-head q/k norms, windowed layers
    for k, v in _GEMMA3_TEXT_DEFAULTS.items():
        if d.get(k) is None:
            d[k] = v
            if k != "head_dim":
                kw[k] = v
    _read_gemma(mt, d, kw)
    kw.update(post_norm=True, qk_norm=True)
    n_layers = int(kw.get("num_hidden_layers", 26))
    q_scalar = d.get("query_pre_attn_scalar")
    if q_scalar:
        kw["attention_multiplier"] = float(q_scalar) ** -0.5
    types = d.get("layer_types")
    if types is None:
        pat = int(d.get("sliding_window_pattern", 6) or 6)
        types = ["sliding_attention" if (i + 1) % pat else "full_attention" for i in range(n_layers)]
    if kw.get("sliding_window") is None:
        kw["sliding_window"] = int(d.get("sliding_window", 4096) or 4096)
    kw["window_layers"] = [int(t == "sliding_attention") for t in types]
    rp = d.get("rope_parameters")
    if isinstance(rp, dict) and ("full_attention" in rp or "sliding_attention" in rp):
        full, local = dict(rp.get("full_attention") or {}), dict(rp.get("sliding_attention") or {})
        kw["rope_theta"] = float(full.pop("rope_theta", d.get("rope_theta") or 1_000_000.0))
        kw["rope_local_theta"] = float(local.get("rope_theta", d.get("rope_local_base_freq") or 10_000.0))
        kw["rope_scaling"] = full if full.get("rope_type", full.get("type")) not in (None, "default") else None
        if local.get("rope_type", "default") != "default":
            raise NotImplementedError("gemma3_text with rope scaling on the windowed layers is not built")
    else:            # older configs: rope_theta, rope_local_base_freq and rope_scaling (for the global layers) side by side
        kw["rope_theta"] = float(d.get("rope_theta") or 1_000_000.0)
        kw["rope_local_theta"] = float(d.get("rope_local_base_freq") or 10_000.0)


_FAMILY_READERS = {
    "gemma": _read_gemma, "gemma3_text": _read_gemma3_text,
    "qwen2": _read_qwen2, "qwen3": _read_qwen3, "qwen3_moe": _read_qwen3_moe, "qwen2_moe": _read_qwen2_moe,
    "mixtral": _read_mixtral, "granitemoe": _read_granite_moe, "granitemoeshared": _read_granite_moe,
    "olmoe": _read_olmoe, "smollm3": _read_smollm3, "olmo2": _read_olmo2, "olmo3": _read_olmo3, "ministral": _read_ministral, "exaone4": _read_exaone4,
    "helium": _read_interleaved, "ernie4_5": _read_interleaved, "seed_oss": _read_seed_oss, "glm": _read_glm,
    "glm4": _read_glm, "hunyuan_v1_dense": _read_hunyuan,
}


# ---------------------------------------------------------------------------------------------- per-family writers
# The inverse direction: each takes (the configuration, the config.json dict so far, what was taken out of it) and puts
# the family's own keys in. ``d`` arrives with the shared keys, hidden_act = silu and the architecture name.
_ARCHITECTURES = {
    "llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM", "ministral": "MinistralForCausalLM", "qwen2": "Qwen2ForCausalLM", "phi3": "Phi3ForCausalLM",
    "mixtral": "MixtralForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
    "qwen2_moe": "Qwen2MoeForCausalLM", "granite": "GraniteForCausalLM", "granitemoe": "GraniteMoeForCausalLM",
    "granitemoeshared": "GraniteMoeSharedForCausalLM", "smollm3": "SmolLM3ForCausalLM", "olmo2": "Olmo2ForCausalLM", "olmo3": "Olmo3ForCausalLM",
    "olmoe": "OlmoeForCausalLM", "glm": "GlmForCausalLM", "glm4": "Glm4ForCausalLM", "exaone4": "Exaone4ForCausalLM",
    "helium": "HeliumForCausalLM", "ernie4_5": "Ernie4_5ForCausalLM", "seed_oss": "SeedOssForCausalLM",
    "hunyuan_v1_dense": "HunYuanDenseV1ForCausalLM", "gemma": "GemmaForCausalLM", "gemma3_text": "Gemma3ForCausalLM",
}


def _write_plain(cfg, d, held):          # llama, granite (and any type without keys of its own)
    d.update(attention_bias=False, mlp_bias=False)


def _write_granite_moe_shared(cfg, d, held):
    _write_plain(cfg, d, held)
    d["shared_intermediate_size"] = held["shared_f"]


def _write_no_attention_bias_key(cfg, d, held):      # mistral, mixtral, phi3: their configs have no such key
    d.pop("attention_bias")


def _write_ministral(cfg, d, held):      # HuggingFace's module needs the head size spelled out
    d.pop("attention_bias")
    d["head_dim"] = cfg.head_dim


def _write_qwen2(cfg, d, held):
    d.pop("attention_bias")
    d["use_sliding_window"] = cfg.sliding_window is not None


def _write_qwen3(cfg, d, held):
    d.update(use_sliding_window=cfg.sliding_window is not None, head_dim=cfg.head_dim)


def _write_qwen_moe(cfg, d, held):       # HuggingFace's names: num_experts, moe_intermediate_size, norm_topk_prob
    d.update(use_sliding_window=cfg.sliding_window is not None, num_experts=d.pop("num_local_experts"),
             moe_intermediate_size=cfg.intermediate_size, norm_topk_prob=bool(held["renorm"]), decoder_sparse_step=1,
             mlp_only_layers=[])
    d["intermediate_size"] = held["extra"].pop("dense_intermediate_size", cfg.intermediate_size)
    if cfg.model_type == "qwen3_moe":
        d["head_dim"] = cfg.head_dim
    else:
        d.pop("attention_bias")
        d.update(qkv_bias=True, shared_expert_intermediate_size=held["shared_f"])


def _write_olmoe(cfg, d, held):
    d.update(attention_bias=False, num_experts=d.pop("num_local_experts"), norm_topk_prob=bool(held["renorm"]),
             clip_qkv=None)


def _write_olmo2(cfg, d, held):
    d["attention_bias"] = False


def _write_exaone4(cfg, d, held):
    d.pop("attention_bias")
    nope = held["nope"]
    d.update(sliding_window=cfg.sliding_window,
             layer_types=["sliding_attention" if (nope and nope[i]) else "full_attention"
                          for i in range(cfg.num_hidden_layers)])


def _write_head_dim(cfg, d, held):       # hunyuan, helium, seed_oss, ernie4_5: an explicit head_dim and their bias keys
    d["head_dim"] = cfg.head_dim
    if cfg.model_type == "hunyuan_v1_dense":
        d["attention_bias"] = False
    elif cfg.model_type == "helium":
        d["mlp_bias"] = False
    elif cfg.model_type == "seed_oss":
        d.update(mlp_bias=False, attention_out_bias=False)
    else:
        d.pop("attention_bias")
        d["use_bias"] = False


def _write_glm(cfg, d, held):
    d.update(head_dim=cfg.head_dim, partial_rotary_factor=cfg.partial_rotary_factor)


def _write_smollm3(cfg, d, held):
    d.update(mlp_bias=False, use_sliding_window=cfg.sliding_window is not None,
             no_rope_layers=list(held["nope"] or [1] * cfg.num_hidden_layers))


def _write_gemma(cfg, d, held):
    d.update(hidden_act="gelu_pytorch_tanh", hidden_activation="gelu_pytorch_tanh", attention_bias=False,
             head_dim=cfg.head_dim)


def _write_gemma3_text(cfg, d, held):
    d.pop("attention_bias")
    d.pop("hidden_act")
    d.pop("rope_theta")
    d.pop("rope_scaling", None)
    am, win = held["gran"]["attention_multiplier"], held["win_layers"]
    rope_full = dict(cfg.rope_scaling or {"rope_type": "default"}, rope_theta=cfg.rope_theta)
    d.update(hidden_activation="gelu_pytorch_tanh", head_dim=cfg.head_dim,
             query_pre_attn_scalar=_whole_if_close(1.0 / am ** 2) if am else cfg.head_dim,
             layer_types=["sliding_attention" if (win is None or win[i]) and cfg.sliding_window else "full_attention"
                          for i in range(cfg.num_hidden_layers)],
             rope_parameters={"full_attention": rope_full,
                              "sliding_attention": {"rope_type": "default",
                                                    "rope_theta": cfg.rope_local_theta or cfg.rope_theta}},
             final_logit_softcapping=None, attn_logit_softcapping=None)


_FAMILY_WRITERS = {
    "granitemoeshared": _write_granite_moe_shared, "mistral": _write_no_attention_bias_key,
    "ministral": _write_ministral, "mixtral": _write_no_attention_bias_key,
    "phi3": _write_no_attention_bias_key, "qwen2": _write_qwen2, "qwen3": _write_qwen3, "qwen3_moe": _write_qwen_moe,
    "qwen2_moe": _write_qwen_moe, "olmoe": _write_olmoe, "olmo2": _write_olmo2, "olmo3": _write_olmo2, "exaone4": _write_exaone4,
    "hunyuan_v1_dense": _write_head_dim, "helium": _write_head_dim, "seed_oss": _write_head_dim,
    "ernie4_5": _write_head_dim, "glm": _write_glm, "glm4": _write_glm, "smollm3": _write_smollm3,
    "gemma": _write_gemma, "gemma3_text": _write_gemma3_text,
}


PRESETS = {
    # name: (layers, hidden, heads, kv_heads, ffn, vocab, theta, eps, tied, max_pos)
    "tinyllama-1.1b": (22, 2048, 32, 4, 5632, 32000, 10000.0, 1e-5, False, 2048),
    "llama-3.2-1b": (16, 2048, 32, 8, 8192, 128256, 500000.0, 1e-5, True, 131072),
    "llama-3-8b": (32, 4096, 32, 8, 14336, 128256, 500000.0, 1e-5, False, 8192),
    "mistral-7b": (32, 4096, 32, 8, 14336, 32000, 10000.0, 1e-5, False, 32768),
    "llama-3-70b": (80, 8192, 64, 8, 28672, 128256, 500000.0, 1e-5, False, 8192),
    # Qwen2 family: the same blocks with a bias on the q/k/v projections (attention_bias, set by preset())
    "qwen2.5-0.5b": (24, 896, 14, 2, 4864, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-1.5b": (28, 1536, 12, 2, 8960, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-7b": (28, 3584, 28, 4, 18944, 152064, 1000000.0, 1e-6, False, 32768),
    # Mixtral layout on TinyLlama's dimensions: 8 experts, 2 per token (6.4 B parameters, 1.3 B active per token)
    "tinymixtral-8x1b": (22, 2048, 32, 4, 5632, 32000, 10000.0, 1e-5, False, 2048),
    "plumbing-teacher": (2, 256, 4, 4, 688, 32000, 10000.0, 1e-6, False, 2048),
    "plumbing-student": (4, 256, 4, 4, 688, 32000, 10000.0, 1e-6, False, 2048),
}


def preset(name: str, **over) -> LlamaConfig:
    Lr, h, H, Hkv, f, V, theta, eps, tied, mp = PRESETS[name]
    cfg = LlamaConfig(vocab_size=V, hidden_size=h, intermediate_size=f, num_hidden_layers=Lr, num_attention_heads=H,
                      num_key_value_heads=Hkv, rms_norm_eps=eps, rope_theta=theta, max_position_embeddings=mp,
                      tie_word_embeddings=tied)
    if name.startswith("tinymixtral"):
        cfg.model_type, cfg.num_local_experts, cfg.num_experts_per_tok = "mixtral", 8, 2
    if name.startswith("qwen2"):
        cfg.attention_bias, cfg.model_type = True, "qwen2"
    if name.startswith("llama-3.2"):      # the published Llama 3.2 configs scale the low rope frequencies
        cfg.rope_scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}
    for k, v in over.items():
        setattr(cfg, k, v)
    return cfg
