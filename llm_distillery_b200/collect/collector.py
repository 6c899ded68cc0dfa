"""Teacher collection on device: forward -> content rows -> LM head -> log-softmax -> top-K -> pinned host.

What the reference does per batch (classes/teacher/inference_worker.py:66-85, result_processor_worker.py:27-58):
full forward, ``[:, :, :crop].float()``, log_softmax over the cropped vocabulary, ``torch.topk``, copy EVERYTHING to
the host, then keep the content positions on the CPU. Here the content rows are gathered on the device before
the LM head, so the vocabulary-sized work is done only for rows that are kept; logits exist only for one row
chunk at a time (fp32, sized to stay L2-resident) between the tcgen05 GEMM and the exact top-K kernel; fp16
log-probs + int32 ids go to pinned host memory on a copy stream, and the caller queues the next batch before it takes
delivery of this one (``submit`` / ``fetch``).
"""
from __future__ import annotations

import numpy as np
import torch

from ..data.convo import ConvoTokenized, TeacherRows
from ..ops import basic, topk as topk_ops


class TeacherCollector:
    def __init__(self, model, *, topk: int, crop_to_size: int, enable_topk: bool = True, logits_chunk_bytes: int = 96 << 20,
                 prefill_chunk_len: int = 0):
        self.model = model
        # > 0: sequences longer than this are run through the model in chunks of this many positions against a
        # key / value cache (LlamaModel.hidden_states_chunked); 0: one pass over the whole sequence
        self.prefill_chunk_len = int(prefill_chunk_len or 0)
        self.vocab = min(int(crop_to_size or model.cfg.vocab_size), model.cfg.vocab_size)
        self.K = min(int(topk), self.vocab)          # a vocabulary smaller than K: every token is kept
        self.enable_topk = bool(enable_topk)
        self.device = model.embed_tokens.device
        self.chunk_rows = max(128, (logits_chunk_bytes // (4 * self.vocab)) // 128 * 128)

    @torch.no_grad()
    def submit(self, tokens: np.ndarray, convos: list[ConvoTokenized], positions=None) -> dict:
        """Queues the whole batch - forward, LM head, top-K, copy of the kept rows to pinned host memory - and returns
        a ticket at once. The copy runs on a stream of its own behind the compute, so the caller can queue the NEXT
        batch before it ``fetch``es this one: the GPU computes batch i+1 while batch i's rows cross PCIe and are handed
        to the HDF5 writer. (Pinned buffers come from PyTorch's caching host allocator: after the first batches no
        new page-locked memory is allocated, and a buffer is reused only when every array handed out over it is gone.)
        """
        B, L = tokens.shape
        ids = torch.from_numpy(np.ascontiguousarray(tokens)).to(self.device, non_blocking=True)
        if 0 < self.prefill_chunk_len < L:
            hs = self.model.hidden_states_chunked(ids, self.prefill_chunk_len)
        else:
            hs = self.model.hidden_states(ids)
        rows, counts = [], []
        for b, c in enumerate(convos):
            ci = c.content_indices() if positions is None else np.asarray(positions[b], dtype=np.int64)
            ci = ci[ci < min(c.length, L)]
            rows.append(ci + b * L)
            counts.append(len(ci))
        rows_np = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int64)
        M = len(rows_np)
        if M == 0:
            return {"hv": None, "hi": None, "counts": counts, "event": None}
        every_row = M == B * L and bool((rows_np == np.arange(M)).all())
        if every_row:
            Hc = hs
        else:
            rows_t = torch.from_numpy(rows_np).to(self.device, non_blocking=True)
            Hc = basic.gather_rows(hs, rows_t)
        W = self.model.lm_head[: self.vocab]
        width = self.K if self.enable_topk else self.vocab
        out_v = torch.empty((M, width), dtype=torch.float16, device=self.device)
        out_i = torch.empty((M, self.K), dtype=torch.int32, device=self.device) if self.enable_topk else None
        logits = torch.empty((min(self.chunk_rows, M), self.vocab), dtype=torch.float32, device=self.device)
        for r0 in range(0, M, self.chunk_rows):
            r1 = min(M, r0 + self.chunk_rows)
            lg = logits[: r1 - r0]
            if Hc.is_cuda and Hc.dtype in (torch.bfloat16, torch.float16):
                basic.gemm(Hc[r0:r1], W, out=lg)
            else:
                lg.copy_(Hc[r0:r1].float() @ W.float().t())
            if self.enable_topk:
                v, i = topk_ops.topk_logprob(lg, self.vocab, self.K)
                out_v[r0:r1], out_i[r0:r1] = v, i
            else:
                out_v[r0:r1] = topk_ops.logprob_full(lg, self.vocab)
        return self._to_host(out_v, out_i, counts)

    def _to_host(self, out_v, out_i, counts) -> dict:
        pin = self.device.type == "cuda"
        hv = torch.empty(out_v.shape, dtype=out_v.dtype, pin_memory=pin)
        hi = torch.empty(out_i.shape, dtype=out_i.dtype, pin_memory=pin) if out_i is not None else None
        if not pin:
            hv.copy_(out_v)
            if hi is not None:
                hi.copy_(out_i)
            return {"hv": hv, "hi": hi, "counts": counts, "event": None}
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        cs = self._copy_stream
        cs.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(cs):
            hv.copy_(out_v, non_blocking=True)
            if hi is not None:
                hi.copy_(out_i, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(cs)
        out_v.record_stream(cs)          # the device rows stay allocated until the copy stream is through with them
        if out_i is not None:
            out_i.record_stream(cs)
        return {"hv": hv, "hi": hi, "counts": counts, "event": ev}

    @staticmethod
    def fetch(ticket: dict):
        """Waits for the ticket's copy (only that: later batches keep running) and returns (values, ids, counts)."""
        if ticket["event"] is not None:
            ticket["event"].synchronize()
        return ticket["hv"], ticket["hi"], ticket["counts"]

    def content_logprobs(self, tokens: np.ndarray, convos: list[ConvoTokenized], positions=None):
        """tokens [B, L] int64 (cropped to the longest member). Returns (values fp16 [M, K or Vc], ids int32 [M, K] or
        None, rows_per_convo) as host tensors; M = total content rows of the batch."""
        return self.fetch(self.submit(tokens, convos, positions))

    def rows_of(self, ticket: dict, convos: list[ConvoTokenized]) -> list[TeacherRows]:
        hv, hi, counts = self.fetch(ticket)
        out, r = [], 0
        for c, n in zip(convos, counts):
            if n == 0:
                continue
            vals = hv[r:r + n].numpy()
            idx = None if hi is None else hi[r:r + n].numpy().astype(np.int64)
            out.append(TeacherRows(c.origin_convo_id, vals, idx, c.content_sha, c.sample))
            r += n
        return out

    def collect_batch(self, tokens: np.ndarray, convos: list[ConvoTokenized], aligner=None,
                      validation: bool = False) -> list[TeacherRows]:
        if aligner is not None:
            return self._collect_aligned(tokens, convos, aligner, validation)
        return self.rows_of(self.submit(tokens, convos), convos)

    def _collect_aligned(self, tokens, convos, aligner, validation) -> list[TeacherRows]:
        """Teacher of another vocabulary: collect at the teacher positions that share a token boundary with the
        student's content rows, map the ids onto the student vocabulary, and lay the rows out in student order
        (rows without a counterpart are all -inf)."""
        if not self.enable_topk:
            raise ValueError("cross-tokenizer teachers need top-K storage (enable_topK)")
        maps = [aligner.positions_for(c, validation) for c in convos]
        wanted = [np.unique(m[m >= 0]) if m is not None else np.zeros(0, dtype=np.int64) for m in maps]
        hv, hi, counts = self.content_logprobs(tokens, convos, positions=wanted)
        out, r = [], 0
        for c, m, w, n in zip(convos, maps, wanted, counts):
            if m is None or len(m) == 0:
                r += n
                continue
            vals = np.full((len(m), self.K), -np.inf, dtype=np.float16)
            idx = np.tile(np.arange(self.K, dtype=np.int64), (len(m), 1))
            if n:
                lp, ids = aligner.remap(hv[r:r + n].to(self.device), hi[r:r + n].to(self.device), self.K)
                lp, ids = lp.cpu().numpy().astype(np.float16), ids.cpu().numpy().astype(np.int64)
                where = {int(p): j for j, p in enumerate(w[:n])}
                for row, p in enumerate(m):
                    j = where.get(int(p), -1) if p >= 0 else -1
                    if j >= 0:
                        vals[row], idx[row] = lp[j], ids[j]
                # rows whose remapped list is shorter than K keep -inf tails with placeholder ids: make the ids unique
                empty = ~np.isfinite(vals.astype(np.float32))
                idx[empty] = (np.arange(self.K, dtype=np.int64)[None, :].repeat(len(m), 0))[empty]
            r += n
            s = (aligner.student_val_convos if validation else aligner.student_convos)[c.origin_convo_id]
            out.append(TeacherRows(c.origin_convo_id, vals, idx, s.content_sha, s.sample))
        return out


class TPTeacherCollector(TeacherCollector):
    """Collector over a tensor-parallel teacher (``parallel.tp.TPLlama``): every rank of the group calls
    ``content_logprobs`` with the same batch; the vocabulary-parallel head returns the exact top-K of the whole
    vocabulary on every rank and only the group's first rank copies the content rows to the host."""

    def __init__(self, tp_model, *, topk: int, crop_to_size: int, enable_topk: bool = True):
        if not enable_topk:
            raise NotImplementedError("full-distribution storage is not offered with a tensor-parallel teacher: "
                                      "use top-K storage (enable_topK) or tp_size = 1")
        self.model = tp_model
        self.vocab = tp_model.V
        self.K = min(int(topk), int(tp_model.V))
        self.enable_topk = True
        self.device = tp_model.device
        self.is_writer = tp_model.g.rank == 0

    @torch.no_grad()
    def submit(self, tokens: np.ndarray, convos: list[ConvoTokenized], positions=None) -> dict:
        from ..parallel.tp import padded_seq_len
        B, L = tokens.shape
        Lp = padded_seq_len(B, L, self.model.g.world)
        padded = np.zeros((B, Lp), dtype=np.int64)      # causal attention: trailing padding cannot reach real rows
        padded[:, :L] = tokens
        ids = torch.from_numpy(padded).to(self.device, non_blocking=True)
        lp, ix = self.model.topk_logprobs(ids, self.K)
        rows, counts = [], []
        for b, c in enumerate(convos):
            ci = c.content_indices() if positions is None else np.asarray(positions[b], dtype=np.int64)
            ci = ci[ci < min(c.length, L)]
            rows.append(ci + b * Lp)
            counts.append(len(ci))
        rows_np = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int64)
        if len(rows_np) == 0 or not self.is_writer:
            return {"hv": None, "hi": None, "counts": counts, "event": None}
        rows_t = torch.from_numpy(rows_np).to(self.device, non_blocking=True)
        # the vocabulary-parallel head runs on every padded position and the content rows are picked afterwards: the
        # hidden states are token-sharded over the group at that point, and the head is ~1.5 % of a 70 B forward
        return self._to_host(lp[rows_t], ix[rows_t], counts)

    def collect_batch(self, tokens, convos, aligner=None, validation: bool = False):
        if self.is_writer:
            return super().collect_batch(tokens, convos, aligner=aligner, validation=validation)
        self.submit(tokens, convos)     # take part in the forward; the rows stay on the writer rank
        return []
