"""The strongest configuration of the LIBRARIES that are installed, for the same step as the benchmark (the unmodified
reference itself is the other arm: ``baseline/reference_arm.py``). It follows the reference's op sequence
(classes/student/model.py:408-448): HuggingFace ``LlamaForCausalLM`` forward on cuBLAS + torch SDPA (the fastest
library attention on this GPU: 664 TFLOP/s forward at head dim 64 against 318 for flash_attn 2, which
``B200_BASELINE_ATTN=flash_attention_2`` selects), full-vocabulary logits -> ``[:, :, :Vc].float() / T`` -> log_softmax
-> gather at the teacher's top-K ids -> forward KL, or with ``loss="reference"`` the reference's own
``calculate_divergence`` imported from its tree and called per conversation as the reference calls it -> autograd
backward -> ``torch.optim.AdamW(fused=True)``; more than one GPU uses NCCL ``DistributedDataParallel``, or with
``shard="zero3"`` PyTorch's fully sharded data parallelism (``torch.distributed.fsdp.fully_shard`` per decoder layer,
fp32 master parameters with bf16 compute - the library counterpart of this package's full parameter sharding).
Collection runs the whole batch at once. None of this package's kernels, models or engine is on this path."""
from __future__ import annotations

import torch
import torch.nn.functional as F


class BaselineRunner:
    def __init__(self, cfg, device, world: int, temperature: float, topk: int, lr: float = 1e-5, loss: str = "kl",
                 shard: str = "ddp", grad_accum: int = 1):
        import os
        from transformers import LlamaConfig, LlamaForCausalLM
        self.loss = loss
        self.grad_accum = max(1, int(grad_accum))
        self._ref_loss = None
        if loss == "reference":
            import sys
            from . import reference_arm as ra
            ra._install_stand_ins(None if device.type != "cuda" else device.index)
            if ra.REF not in sys.path:
                sys.path.insert(0, ra.REF)
            from utils.finetuning_utils import calculate_divergence      # the reference's own function
            self._ref_loss = calculate_divergence
        hf = LlamaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                         num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                         num_key_value_heads=cfg.num_key_value_heads, rms_norm_eps=cfg.rms_norm_eps,
                         rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings,
                         tie_word_embeddings=cfg.tie_word_embeddings,
                         attn_implementation=os.environ.get("B200_BASELINE_ATTN", "sdpa"))
        torch.manual_seed(1234)
        fsdp = world > 1 and shard == "zero3"
        with torch.device(device):
            model = LlamaForCausalLM(hf).to(torch.float32 if fsdp else torch.bfloat16)
        model.train()
        self.model = model
        self.device = device
        self.T = temperature
        self.vocab = cfg.vocab_size
        if fsdp:
            from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
            mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
            for layer in model.model.layers:
                fully_shard(layer, mp_policy=mp)
            fully_shard(model, mp_policy=mp)
        elif world > 1:
            self.model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[device.index])
        self.opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.99), weight_decay=2e-8, eps=1e-8, fused=True)

    def to_device(self, hb):
        return hb.to_device(self.device)

    def _step(self, mb):
        for k in range(self.grad_accum):
            out = self._micro(mb, step=(k + 1 == self.grad_accum))
        return out

    def _micro(self, mb, step: bool):
        logits = self.model(mb.input_ids).logits[:, :, : self.vocab].float() / self.T
        B, L, V = logits.shape
        if self._ref_loss is not None:
            # classes/student/model.py:415-441: one call per conversation, losses summed, one backward
            total = None
            ids3, u3 = mb.ids.view(B, L, -1).long(), mb.logp.view(B, L, -1).float() / self.T
            none = torch.zeros(0, dtype=torch.long, device=logits.device)
            for b in range(B):
                d = self._ref_loss(logits[b], u3[b], ids3[b], mb.input_ids[b, 1:], 2, none)
                total = d["train_loss"] if total is None else total + d["train_loss"]
            (total / self.grad_accum).backward()
            if step:
                self.opt.step()
                self.opt.zero_grad(set_to_none=True)
            return total.detach()
        s_full = F.log_softmax(logits.reshape(B * L, V), dim=-1)
        s = torch.gather(s_full, 1, mb.ids.long())
        t = F.log_softmax(mb.logp.float() / self.T, dim=-1)
        if self.loss == "rkl":      # both renormalised over the teacher's top-K (the reference's reverse term)
            kl = F.kl_div(t, F.log_softmax(s, dim=-1), reduction="none", log_target=True).sum(-1)
        elif self.loss == "jsd":
            m = torch.logsumexp(torch.stack([s, t]), 0) - 0.6931471805599453
            kl = 0.5 * (F.kl_div(m, t, reduction="none", log_target=True).sum(-1)
                        + F.kl_div(m, s, reduction="none", log_target=True).sum(-1))
        else:
            kl = F.kl_div(s, t, reduction="none", log_target=True).sum(-1)      # per token
        loss = kl.reshape(B, L).mean(-1).sum()                                   # mean per conversation, summed
        (loss / self.grad_accum).backward()
        if step:
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
        return loss.detach()

    def device_step(self, db):
        return self._step(db)

    def e2e_step(self, hb):
        return self._step(hb.to_device(self.device))

    # ---- collection, restating classes/teacher/inference_worker.py:66-85 and result_processor_worker.py:27-58:
    # full forward, crop + .float(), log_softmax over the vocabulary, torch.topk, everything to the host, content
    # rows selected on the CPU
    def collect_setup(self):
        m = self.model.module if hasattr(self.model, "module") else self.model
        m.eval()
        self._teacher = m

    @torch.no_grad()
    def collect_step(self, tokens_np, convos):
        import numpy as np
        topk = int(getattr(self, "collect_topk", 200))
        ids = torch.from_numpy(tokens_np).to(self.device)
        B, L = ids.shape
        logits = self._teacher(ids).logits[:, :, : self.vocab].float()      # the whole batch at once: 2 GB of fp32
        lp = F.log_softmax(logits, dim=-1)
        v, i = torch.topk(lp, topk, dim=-1)
        vals, idx = v.to("cpu").numpy(), i.to("cpu").numpy()
        rows_v, rows_i = [], []
        for b, c in enumerate(convos):
            ci = c.content_indices()
            rows_v.append(vals[b][ci].astype(np.float16))
            rows_i.append(idx[b][ci])
        hv = torch.from_numpy(np.concatenate(rows_v))
        hi = torch.from_numpy(np.concatenate(rows_i).astype(np.int32))
        return hv, hi, [len(c.content_indices()) for c in convos]
