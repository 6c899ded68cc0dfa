"""Tensor parallelism for teacher collection (kernels: csrc/comm/tp_gemm.cu, csrc/loss/topk_logprob.cu).

The reference spreads a large teacher over GPUs layer by layer (ExLlamaV2 ``load_autosplit``,
classes/teacher/inference_worker.py:46-51), which keeps one GPU busy at a time. Here every GPU holds 1/tp of every
weight matrix and the residual stream lives token-sharded between the parallel regions:

    x_shard [T/tp, h] -> RMSNorm -> (all-gather -> column-parallel GEMM)  qkv heads of this rank  -> RoPE, attention
                     -> (row-parallel GEMM -> reduce-scatter + residual)  x_shard
                     -> RMSNorm -> (all-gather -> GEMM) gate/up -> SwiGLU -> (GEMM -> reduce-scatter + residual)

Each bracket is ONE kernel launch (``TPGroup.ag_gemm`` / ``TPGroup.gemm_rs``) that moves the data over NVLink by
peer loads/stores while the tensor cores work. The LM head is vocabulary-parallel: every rank takes the top K of its
vocabulary slice plus the slice's log-sum-exp, the candidates are exchanged by peer stores, and a merge kernel
produces the exact top-K log-probs of the whole vocabulary.

On a machine without GPUs the same classes run over gloo with ``all_gather`` / ``all_reduce`` and PyTorch math, which
is what the CPU tests exercise.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.distributed as dist

from ..ops import _lib, basic, attention, topk as topk_ops
from ..ops._lib import _VP, _I, _LL

_U = ctypes.c_uint
_lib.register("b200_tp_ag_gemm", [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _LL, _I, _I, _I, _U, _VP])
_lib.register("b200_tp_gemm_rs", [_VP, _LL, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _U, _VP])
_lib.register("b200_topk_partial", [_VP, _LL, _I, _I, _I, _I, _VP, _VP, _VP, _VP])
_lib.register("b200_topk_combine", [_VP, _VP, _VP, _LL, _LL, _I, _I, _I, _VP, _VP, _VP])

ROW_BLOCK = 128   # rows per GEMM tile: slabs are whole tiles


def padded_seq_len(batch: int, seq: int, tp: int) -> int:
    """Smallest L' >= seq such that batch * L' splits into tp slabs of whole 128-row tiles."""
    unit = ROW_BLOCK * tp // math.gcd(batch, tp)
    return -(-seq // unit) * unit


class TPGroup:
    """Symmetric buffers, flags and call counters of one tensor-parallel group (all ranks of the process group)."""

    def __init__(self, device, max_tokens: int, hidden: int, topk: int = 0, group=None, dtype=torch.bfloat16):
        self.device = torch.device(device)
        self.group = group or dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.native = self.device.type == "cuda"
        self.dtype = torch.bfloat16 if self.native else dtype     # the kernels are bf16; the CPU path follows the model
        unit = ROW_BLOCK * self.world
        self.max_tokens = -(-max_tokens // unit) * unit
        self.hidden = hidden
        self.topk = topk
        self.ag_epoch = 0
        self.rs_epoch = 0
        self.bar_epoch = 0
        self._cpu_slab = None
        if not self.native:
            return
        from .p2p import SymmetricBuffer
        n = self.max_tokens * hidden
        self.xf = [SymmetricBuffer(n, torch.bfloat16, self.device, self.group) for _ in range(2)]
        self.stg = [SymmetricBuffer(n, torch.bfloat16, self.device, self.group) for _ in range(2)]
        self.ag_flags = SymmetricBuffer(64, torch.int32, self.device, self.group)
        self.rs_flags = SymmetricBuffer(64, torch.int32, self.device, self.group)
        self.sig = SymmetricBuffer(64, torch.int32, self.device, self.group)
        self.blk_count = torch.zeros(self.max_tokens // ROW_BLOCK, dtype=torch.int32, device=self.device)
        self.done_count = torch.zeros(16, dtype=torch.int32, device=self.device)
        if topk:
            w, t, k = self.world, self.max_tokens, topk
            self.cand_z = SymmetricBuffer(w * t * k, torch.float32, self.device, self.group)
            self.cand_i = SymmetricBuffer(w * t * k, torch.int32, self.device, self.group)
            self.cand_l = SymmetricBuffer(w * t, torch.float32, self.device, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # ------------------------------------------------------------------ helpers
    def tokens_per_rank(self, T: int) -> int:
        if T % (ROW_BLOCK * self.world) or T > self.max_tokens:
            raise ValueError(f"token count {T} must be a multiple of {ROW_BLOCK * self.world} and <= {self.max_tokens}")
        return T // self.world

    def slab(self, T: int, K: int) -> torch.Tensor:
        """This rank's rows [Ts, K] of the gathered buffer the NEXT ``ag_gemm`` will read: write the input there."""
        Ts = self.tokens_per_rank(T)
        if not self.native:
            self._cpu_slab = torch.empty((Ts, K), dtype=self.dtype)
            return self._cpu_slab
        if K > self.hidden:
            raise ValueError("gathered width exceeds the group's hidden size")
        buf = self.xf[self.ag_epoch & 1].tensor
        return buf[: T * K].view(T, K)[self.rank * Ts:(self.rank + 1) * Ts]

    def check(self) -> None:
        err = _lib.take_device_error()
        if err:
            raise RuntimeError(f"tensor-parallel wait timed out on rank {self.rank} (device error code {err})")

    def rendezvous(self) -> None:
        """A tiny NCCL all-reduce on the current stream, once per forward: the fused kernels' waits on peers give up
        after two seconds, and ranks can be further apart than that when a forward begins (the group's first rank also
        hands rows to the HDF5 writer, batches come from the host at different times). NCCL's wait has no such bound;
        after it the bounded waits only see the skew of a few kernels."""
        if self.native and self.world > 1:
            if getattr(self, "_rdv", None) is None:
                self._rdv = torch.zeros(1, dtype=torch.float32, device=self.device)
            dist.all_reduce(self._rdv, group=self.group)

    def barrier(self) -> None:
        if not self.native:
            dist.barrier(self.group)
            return
        self.bar_epoch += 1
        _lib.check(_lib.kernels().b200_p2p_barrier(self.sig.c_ptrs, self.rank, self.world, self.bar_epoch,
                                                   _lib.stream()), "b200_p2p_barrier")

    # ------------------------------------------------------------------ the two fused layers
    def ag_gemm(self, w: torch.Tensor, T: int, out_f32: bool = False) -> torch.Tensor:
        """[T, N] = all_gather(slabs)[T, K] @ w[N, K]^T, the slab being what was written into ``slab(T, K)``."""
        N, K = w.shape
        Ts = self.tokens_per_rank(T)
        if not self.native:
            parts = [torch.empty_like(self._cpu_slab) for _ in range(self.world)]
            dist.all_gather(parts, self._cpu_slab, group=self.group)
            y = torch.cat(parts, 0).float() @ w.float().t()
            return y if out_f32 else y.to(self.dtype)
        buf = self.xf[self.ag_epoch & 1]
        self.ag_epoch += 1
        out = torch.empty((T, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=self.device)
        _lib.check(_lib.kernels().b200_tp_ag_gemm(buf.c_ptrs, self.ag_flags.c_ptrs, _lib.ptr(w), _lib.ptr(out),
                                                  _lib.ptr(self.blk_count), T, N, K, out.stride(0), int(out_f32),
                                                  self.rank, self.world, self.ag_epoch, _lib.stream()),
                   "b200_tp_ag_gemm")
        return out

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """[T/tp, N] = this rank's rows of sum over ranks (x[T, K_local] @ w[N, K_local]^T) (+ residual)."""
        T, K = x.shape
        N = w.shape[0]
        Ts = self.tokens_per_rank(T)
        if not self.native:
            y = x.float() @ w.float().t()
            dist.all_reduce(y, group=self.group)
            y = y[self.rank * Ts:(self.rank + 1) * Ts]
            if residual is not None:
                y = y + residual.float()
            return y.to(self.dtype)
        if N > self.hidden:
            raise ValueError("gemm_rs output width exceeds the group's hidden size")
        stg = self.stg[self.rs_epoch & 1]
        self.rs_epoch += 1
        out = torch.empty((Ts, N), dtype=torch.bfloat16, device=self.device)
        _lib.check(_lib.kernels().b200_tp_gemm_rs(_lib.ptr(x), x.stride(0), _lib.ptr(w), stg.c_ptrs,
                                                  self.rs_flags.c_ptrs, _lib.ptr(residual), _lib.ptr(out),
                                                  _lib.ptr(self.done_count), T, N, K, self.rank, self.world,
                                                  self.rs_epoch, _lib.stream()), "b200_tp_gemm_rs")
        return out

    # ------------------------------------------------------------------ vocabulary-parallel top-K
    def topk_logprobs(self, logits: torch.Tensor, valid: int, id_offset: int, k: int):
        """logits fp32 [T, V_local] of this rank's vocabulary slice (first ``valid`` columns count). Returns on
        EVERY rank (fp16 log-probs [T, k], int32 ids [T, k]) of the whole vocabulary, sorted by value."""
        T = logits.shape[0]
        if not self.native:
            z = logits[:, :valid].float()
            _, i = torch.sort(z, dim=-1, descending=True, stable=True)
            i = i[:, :k]
            zs = [torch.empty((T, k)) for _ in range(self.world)]
            ids = [torch.empty((T, k), dtype=torch.int64) for _ in range(self.world)]
            ls = [torch.empty(T) for _ in range(self.world)]
            dist.all_gather(zs, torch.gather(z, 1, i).contiguous(), group=self.group)
            dist.all_gather(ids, (i + id_offset).contiguous(), group=self.group)
            dist.all_gather(ls, torch.logsumexp(z, -1), group=self.group)
            return combine_reference(torch.stack(zs), torch.stack(ids), torch.stack(ls), k)
        if k != self.topk:
            raise ValueError("TPGroup was sized for another K")
        w, tm = self.world, self.max_tokens
        zk_stride, l_stride = tm * k, tm
        z = self.cand_z.tensor[self.rank * zk_stride: self.rank * zk_stride + T * k]
        ids = self.cand_i.tensor[self.rank * zk_stride: self.rank * zk_stride + T * k]
        lse = self.cand_l.tensor[self.rank * l_stride: self.rank * l_stride + T]
        self.barrier()      # every rank has finished reading the candidates of the previous call
        _lib.check(_lib.kernels().b200_topk_partial(_lib.ptr(logits), logits.stride(0), T, valid, k, id_offset,
                                                    _lib.ptr(z), _lib.ptr(ids), _lib.ptr(lse), _lib.stream()),
                   "b200_topk_partial")
        K = _lib.kernels()
        for buf, part, n in ((self.cand_z, z, zk_stride), (self.cand_i, ids, zk_stride), (self.cand_l, lse, l_stride)):
            _lib.check(K.b200_p2p_allgather(buf.c_ptrs, _lib.ptr(part), self.rank * n * 4, part.numel() * 4, self.rank,
                                            self.world, 1, _lib.stream()), "b200_p2p_allgather")
        self.barrier()      # all candidates have landed everywhere
        out_lp = torch.empty((T, k), dtype=torch.float16, device=self.device)
        out_ix = torch.empty((T, k), dtype=torch.int32, device=self.device)
        _lib.check(K.b200_topk_combine(_lib.ptr(self.cand_z.tensor), _lib.ptr(self.cand_i.tensor),
                                       _lib.ptr(self.cand_l.tensor), zk_stride, l_stride, w, T, k, _lib.ptr(out_lp),
                                       _lib.ptr(out_ix), _lib.stream()), "b200_topk_combine")
        return out_lp, out_ix


def combine_reference(z: torch.Tensor, ids: torch.Tensor, lse: torch.Tensor, k: int):
    """PyTorch statement of the merge kernel: z, ids [parts, T, k], lse [parts, T] -> (fp16 [T, k], int32 [T, k])."""
    parts, T, _ = z.shape
    zc = z.permute(1, 0, 2).reshape(T, -1).float()
    ic = ids.permute(1, 0, 2).reshape(T, -1).long()
    g = torch.logsumexp(lse.float(), dim=0)
    # value descending, ties by lower id: sort by id first, then stable by value
    o1 = torch.argsort(ic, dim=1, stable=True)
    zc, ic = torch.gather(zc, 1, o1), torch.gather(ic, 1, o1)
    o2 = torch.argsort(zc, dim=1, descending=True, stable=True)[:, :k]
    return (torch.gather(zc, 1, o2) - g[:, None]).to(torch.float16), torch.gather(ic, 1, o2).to(torch.int32)


# ====================================================================================================== model
def shard_llama_weights(cfg, sd: dict, rank: int, tp: int, vocab: int | None = None) -> dict:
    """Slice a fused-name state dict (``LlamaModel.state_dict()`` names) for one tensor-parallel rank.

    Column-parallel: q/k/v heads and gate/up rows are split; row-parallel: o_proj / down_proj columns are split;
    the LM head is split over the (cropped) vocabulary, padded with zero rows to equal slices; embedding and norms
    are replicated. Requires heads, kv heads and the FFN width to be divisible by tp."""
    H, Hkv, d, f = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    if H % tp or Hkv % tp or f % tp:
        raise ValueError(f"tp={tp} must divide heads ({H}), kv heads ({Hkv}) and the FFN width ({f})")
    if getattr(cfg, "sandwich", False):
        raise NotImplementedError("tensor-parallel collection is built for Llama-style pre-norm layers")
    Hl, Hkvl, fl = H // tp, Hkv // tp, f // tp
    out = {"embed_tokens": sd["embed_tokens"], "norm": sd["norm"]}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        qkv = sd[p + "qkv_proj"]
        q, k, v = qkv[: H * d], qkv[H * d:(H + Hkv) * d], qkv[(H + Hkv) * d:]
        out[p + "qkv_proj"] = torch.cat([q[rank * Hl * d:(rank + 1) * Hl * d], k[rank * Hkvl * d:(rank + 1) * Hkvl * d],
                                         v[rank * Hkvl * d:(rank + 1) * Hkvl * d]], 0).contiguous()
        if p + "qkv_bias" in sd:
            bq = sd[p + "qkv_bias"]
            out[p + "qkv_bias"] = torch.cat([bq[: H * d][rank * Hl * d:(rank + 1) * Hl * d],
                                             bq[H * d:(H + Hkv) * d][rank * Hkvl * d:(rank + 1) * Hkvl * d],
                                             bq[(H + Hkv) * d:][rank * Hkvl * d:(rank + 1) * Hkvl * d]]).contiguous()
        for nm in ("q_norm", "k_norm"):
            if p + nm in sd:
                out[p + nm] = sd[p + nm]
        out[p + "o_proj"] = sd[p + "o_proj"][:, rank * Hl * d:(rank + 1) * Hl * d].contiguous()
        gu = sd[p + "gate_up_proj"]
        out[p + "gate_up_proj"] = torch.cat([gu[rank * fl:(rank + 1) * fl], gu[f + rank * fl: f + (rank + 1) * fl]],
                                            0).contiguous()
        out[p + "down_proj"] = sd[p + "down_proj"][:, rank * fl:(rank + 1) * fl].contiguous()
        out[p + "input_layernorm"] = sd[p + "input_layernorm"]
        out[p + "post_attention_layernorm"] = sd[p + "post_attention_layernorm"]
    head = sd.get("lm_head", sd["embed_tokens"])
    V = min(vocab or head.shape[0], head.shape[0])
    Vl = -(-V // tp)
    Vl = -(-Vl // 8) * 8
    lo, hi = min(rank * Vl, V), min((rank + 1) * Vl, V)
    piece = torch.zeros((Vl, head.shape[1]), dtype=head.dtype, device=head.device)
    piece[: hi - lo] = head[lo:hi]
    out["lm_head"] = piece
    out["_vocab"] = (V, Vl, lo, hi - lo)
    return out


class TPLlama:
    """Forward-only tensor-parallel Llama (teacher). ``weights`` is the output of ``shard_llama_weights`` on this
    rank's device; ``group`` a ``TPGroup`` sized for the largest batch."""

    def __init__(self, cfg, weights: dict, group: TPGroup):
        self.cfg = cfg
        self.w = weights
        self.g = group
        self.device = group.device
        self.V, self.Vl, self.v_lo, self.v_valid = weights["_vocab"]
        self._rope = None

    @classmethod
    def from_full(cls, model, group: TPGroup, vocab: int | None = None) -> "TPLlama":
        """Shard a whole ``LlamaModel`` (any device) onto this rank."""
        sd = {k: v.detach() for k, v in model.state_dict().items()}
        w = shard_llama_weights(model.cfg, sd, group.rank, group.world, vocab)
        w = {k: (v.to(group.device) if torch.is_tensor(v) else v) for k, v in w.items()}
        return cls(model.cfg, w, group)

    @classmethod
    def random_init(cls, cfg, group: TPGroup, seed: int = 0, std: float = 0.02, dtype=torch.bfloat16,
                    vocab: int | None = None) -> "TPLlama":
        """Random weights generated shard by shard on the device (benchmarks of models too large for one GPU)."""
        tp, r, dev = group.world, group.rank, group.device
        H, Hkv, d, f, h = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, cfg.hidden_size
        if H % tp or Hkv % tp or f % tp:
            raise ValueError(f"tp={tp} must divide heads ({H}), kv heads ({Hkv}) and the FFN width ({f})")
        gen = torch.Generator(device=dev).manual_seed(seed * 1000 + r)
        rep = torch.Generator(device=dev).manual_seed(seed)          # replicated tensors: same stream on every rank

        def rnd(shape, g=gen):
            return torch.empty(shape, dtype=dtype, device=dev).normal_(0.0, std, generator=g)

        w = {"embed_tokens": rnd((cfg.vocab_size, h), rep), "norm": torch.ones(h, dtype=dtype, device=dev)}
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            w[p + "qkv_proj"] = rnd(((H + 2 * Hkv) // tp * d, h))
            w[p + "o_proj"] = rnd((h, H // tp * d))
            w[p + "gate_up_proj"] = rnd((2 * f // tp, h))
            w[p + "down_proj"] = rnd((h, f // tp))
            w[p + "input_layernorm"] = torch.ones(h, dtype=dtype, device=dev)
            w[p + "post_attention_layernorm"] = torch.ones(h, dtype=dtype, device=dev)
        V = min(vocab or cfg.vocab_size, cfg.vocab_size)
        Vl = -(-(-(-V // tp)) // 8) * 8
        lo, hi = min(r * Vl, V), min((r + 1) * Vl, V)
        w["lm_head"] = rnd((Vl, h))
        w["_vocab"] = (V, Vl, lo, hi - lo)
        return cls(cfg, w, group)

    def rope(self, n: int):
        sc = getattr(self.cfg, "rope_scaling", None) or {}
        regime = None
        if sc.get("rope_type", sc.get("type")) == "longrope":    # the factor set depends on the sequence length
            regime = n > int(sc.get("original_max_position_embeddings") or self.cfg.max_position_embeddings)
        elif sc.get("rope_type", sc.get("type")) == "dynamic" and not sc.get("alpha"):
            regime = n if n > self.cfg.max_position_embeddings else False            # the base follows the length
        if regime != getattr(self, "_rope_regime", None):
            self._rope, self._rope_regime = None, regime
        if self._rope is None or self._rope[0].shape[0] < n:
            self._rope = basic.rope_tables(max(n, 2048), getattr(self.cfg, "rotary_dim", self.cfg.head_dim),
                                           self.cfg.rope_theta, self.device,
                                           getattr(self.cfg, "rope_scaling", None),
                                           model_max_pos=self.cfg.max_position_embeddings, seq_len=n)
        return self._rope

    @torch.no_grad()
    def forward_shard(self, input_ids: torch.Tensor) -> int:
        """input_ids [B, L] with B*L a multiple of 128*tp (see ``padded_seq_len``). Runs the decoder stack and leaves
        the final-norm hidden states of this rank's token slab in the group's gathered buffer, ready for the LM head.
        Returns T = B*L."""
        cfg, g, w = self.cfg, self.g, self.w
        B, L = input_ids.shape
        T = B * L
        Ts = g.tokens_per_rank(T)
        tp, r = g.world, g.rank
        Hl, Hkvl, d, h, eps = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp, cfg.head_dim, cfg.hidden_size, cfg.rms_norm_eps
        ids = input_ids.reshape(-1).to(self.device)
        pos = torch.arange(L, dtype=torch.int32, device=self.device).repeat(B)
        cos_t, sin_t = self.rope(L)
        nope = getattr(cfg, "no_rope_layers", None) or []       # 0 = the layer applies no positional rotation
        g.rendezvous()
        x = basic.embed_fwd(ids[r * Ts:(r + 1) * Ts].contiguous(), w["embed_tokens"])
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            basic.rmsnorm_fwd(x, w[p + "input_layernorm"], eps, out=g.slab(T, h))
            qkv = g.ag_gemm(w[p + "qkv_proj"], T)
            if p + "qkv_bias" in w:
                basic.bias_add_(qkv, w[p + "qkv_bias"])
            if p + "q_norm" in w:      # per-head norms act inside a head: local under head sharding
                qkv, _ = basic.headnorm_fwd(qkv, w[p + "q_norm"], w[p + "k_norm"], Hl, Hkvl, d, eps)
            if not nope or nope[i]:
                basic.rope_(qkv, pos, cos_t, sin_t, Hl + Hkvl, d)
            att, _ = attention.attention_fwd(qkv, B, L, Hl, Hkvl, d, cfg.layer_window(i, L) if hasattr(cfg, "layer_window") else None)
            x = g.gemm_rs(att, w[p + "o_proj"], residual=x)
            basic.rmsnorm_fwd(x, w[p + "post_attention_layernorm"], eps, out=g.slab(T, h))
            gu = g.ag_gemm(w[p + "gate_up_proj"], T)
            act = basic.swiglu_fwd(gu)
            x = g.gemm_rs(act, w[p + "down_proj"], residual=x)
        basic.rmsnorm_fwd(x, w["norm"], eps, out=g.slab(T, h))
        return T

    @torch.no_grad()
    def topk_logprobs(self, input_ids: torch.Tensor, k: int):
        """(fp16 log-probs [B*L, k], int32 ids [B*L, k]) of log_softmax over the (cropped) vocabulary, on every rank."""
        T = self.forward_shard(input_ids)
        logits = self.g.ag_gemm(self.w["lm_head"], T, out_f32=True)
        if self.v_valid <= 0:
            raise ValueError("a rank received an empty vocabulary slice: use fewer ranks or a larger vocabulary")
        return self.g.topk_logprobs(logits, self.v_valid, self.v_lo, k)
