"""Reference-equivalent training step on the libraries that ARE installed (the literal reference cannot run here:
exllamav2 / bitsandbytes / h5py / accelerate are missing). It restates the reference's op sequence
(classes/student/model.py:408-448): HuggingFace ``LlamaForCausalLM`` forward on cuBLAS + SDPA, full-vocabulary
logits -> ``[:, :, :Vc].float() / T`` -> log_softmax -> gather at the teacher's top-K ids -> forward KL ->
autograd backward -> ``torch.optim.AdamW``; more than one GPU uses NCCL ``DistributedDataParallel``.
None of this package's kernels, models or engine is on this path."""
from __future__ import annotations

import torch
import torch.nn.functional as F


class BaselineRunner:
    def __init__(self, cfg, device, world: int, temperature: float, topk: int, lr: float = 1e-5):
        from transformers import LlamaConfig, LlamaForCausalLM
        hf = LlamaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                         num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                         num_key_value_heads=cfg.num_key_value_heads, rms_norm_eps=cfg.rms_norm_eps,
                         rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings,
                         tie_word_embeddings=cfg.tie_word_embeddings, attn_implementation="sdpa")
        torch.manual_seed(1234)
        with torch.device(device):
            model = LlamaForCausalLM(hf).to(torch.bfloat16)
        model.train()
        self.model = model
        self.device = device
        self.T = temperature
        self.vocab = cfg.vocab_size
        if world > 1:
            self.model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[device.index])
        self.opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.99), weight_decay=2e-8, eps=1e-8, fused=True)

    def to_device(self, hb):
        return hb.to_device(self.device)

    def _step(self, mb):
        logits = self.model(mb.input_ids).logits[:, :, : self.vocab].float() / self.T
        B, L, V = logits.shape
        s_full = F.log_softmax(logits.reshape(B * L, V), dim=-1)
        s = torch.gather(s_full, 1, mb.ids.long())
        t = F.log_softmax(mb.logp.float() / self.T, dim=-1)
        kl = F.kl_div(s, t, reduction="none", log_target=True).sum(-1)          # per token
        loss = kl.reshape(B, L).mean(-1).sum()                                   # mean per conversation, summed
        loss.backward()
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
        # one sequence at a time keeps the fp32 log-softmax of this arm at the size the reference itself handles
        vals, idx = [], []
        for b in range(B):
            logits = self._teacher(ids[b:b + 1]).logits[:, :, : self.vocab].float()
            lp = F.log_softmax(logits, dim=-1)
            v, i = torch.topk(lp, topk, dim=-1)
            vals.append(v[0].to("cpu").numpy())
            idx.append(i[0].to("cpu").numpy())
        rows_v, rows_i = [], []
        for b, c in enumerate(convos):
            ci = c.content_indices()
            rows_v.append(vals[b][ci].astype(np.float16))
            rows_i.append(idx[b][ci])
        hv = torch.from_numpy(np.concatenate(rows_v))
        hi = torch.from_numpy(np.concatenate(rows_i).astype(np.int32))
        return hv, hi, [len(c.content_indices()) for c in convos]
