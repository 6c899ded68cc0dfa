"""Teacher role: collects next-token distributions for the conversations that are missing from the HDF5 store.

Reference (classes/teacher/model.py + the three worker files): a batch-creator process, N spawned inference
processes each holding an ExLlamaV2 replica, a result-processor process and the HDF5 server process, connected by
Manager queues and POSIX shared memory. Here one process per GPU does all of it: batches are planned up front
(length-sorted, cropped to the longest member, reference: batch_creator_worker.py:16-33), the model runs on the
sm_100a kernels, content rows are selected on the device, and finished conversations go straight into the
store's writer pool while the GPU computes the next batch. With several ranks, ``num_inference_workers`` becomes
the number of data-parallel replicas: rank r takes batches r, r+world, ... and rank-local stores are not shared -
each rank writes through the same HDF5 store only when it is rank 0 of its node (others send rows over the
process group).
"""
from __future__ import annotations

import math
import time

import numpy as np
import torch

from ..ckpt.hf import load_hf_model
from ..collect.collector import TeacherCollector
from ..data.convo import PARTIAL_SHA_PREFIX
from ..obs.console import progress, set_status, status
from .base_model import BaseModel


def plan_batches(dataset_chunk, batch_size: int):
    """Consecutive batches of a length-sorted chunk; every batch is cropped to its longest non-padded member."""
    out = []
    for i in range(0, len(dataset_chunk), batch_size):
        convos = dataset_chunk[i:i + batch_size]
        longest = max(c.length for c in convos)
        out.append((np.stack([c.tokenized[:longest] for c in convos]), convos))
    return out


class TeacherModel(BaseModel):
    def __init__(self, model_path: str, max_queue_size: int = 3, interactive: bool = False):
        super().__init__(model_path, student=False, interactive=interactive)
        self.max_queue_size = max_queue_size
        self.model = None
        self.dtype = torch.bfloat16
        self.tokens_collected = 0
        self.collect_seconds = 0.0
        self.chunked_prefill = "auto"       # true | false | auto (config key of the same name)
        self.prefill_max_tokens = 131072

    def prefill_chunk_len(self, batch_size: int, longest: int) -> int:
        """Positions per prefill chunk for a batch of ``batch_size`` sequences of up to ``longest`` tokens (0 = one
        pass). ``true``: the model's own ``seq_chunk_len`` as in the reference (classes/teacher/inference_worker.py:
        38-48); ``auto``: only when the batch holds more than ``prefill_max_tokens`` tokens, in chunks (multiples of
        128) that keep one pass below that."""
        mode = str(self.chunked_prefill).lower()
        if mode == "true":
            return int(self.seq_chunk_len) if 0 < int(self.seq_chunk_len or 0) < longest else 0
        if mode == "auto" and batch_size * longest > self.prefill_max_tokens > 0:
            return max(128, (self.prefill_max_tokens // max(1, batch_size)) // 128 * 128)
        return 0

    def _sort_datasets_by_len(self) -> None:
        if not self.dataset_sorted:
            self.dataset.sort(key=lambda c: c.length, reverse=True)
            self.dataset_sorted = True
        if not self.validation_dataset_sorted:
            self.validation_dataset.sort(key=lambda c: c.length, reverse=True)
            self.validation_dataset_sorted = True

    def load(self, device=None):
        if self.model is None:
            dev = torch.device(device or self.device)
            dtype = self.dtype if dev.type == "cuda" else torch.float32
            self.model = load_hf_model(self.model_path, dtype=dtype, device=dev)
            for p in self.model.parameters():
                p.requires_grad_(False)
        return self.model

    def load_tp(self, tp_group, max_tokens_hint: int | None = None):
        """Tensor-parallel load: this rank reads only its slices of the checkpoint (``ckpt.hf.load_tp_weights``)."""
        from ..ckpt.hf import load_tp_weights
        from ..parallel.tp import TPLlama
        if self.model is None:
            dev = tp_group.device
            dtype = self.dtype if dev.type == "cuda" else torch.float32
            crop = None if getattr(self, "aligner", None) is not None else (self.crop_to_size or None)
            cfg, w = load_tp_weights(self.model_path, tp_group.rank, tp_group.world, vocab=crop, dtype=dtype, device=dev)
            self.model = TPLlama(cfg, w, tp_group)
        return self.model

    def unload(self) -> None:
        self.model = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def process_chunk(self, reserve_vram_gb=None, num_inference_workers: int = 1, ids_to_collect=None,
                      data_manager=None, validation: bool = False, rank: int = 0, world: int = 1,
                      sha_by_id: dict | None = None, tp_group=None, last_teacher: bool = True) -> int:
        """Collect ``ids_to_collect`` into ``data_manager``. Returns the number of conversations written.
        ``rank`` / ``world`` index the data-parallel replicas (each takes a strided share of the batches); with
        ``tp_group`` the replica is a tensor-parallel group whose ranks all call this with the same arguments."""
        self._sort_datasets_by_len()
        wanted = set(ids_to_collect or [])
        chunk = [c for c in (self.validation_dataset if validation else self.dataset) if c.origin_convo_id in wanted]
        if not chunk:
            return 0
        aligner = getattr(self, "aligner", None)
        set_status(None, f"Loading {self.model_name[:20]}...")
        if tp_group is not None:
            from ..collect.collector import TPTeacherCollector
            model = self.load_tp(tp_group)
            collector = TPTeacherCollector(model, topk=self.topK, crop_to_size=model.V, enable_topk=self.enable_topK)
        else:
            model = self.load()
            crop = model.cfg.vocab_size if aligner is not None else self.crop_to_size   # own vocabulary when remapping
            collector = TeacherCollector(model, topk=self.topK, crop_to_size=crop, enable_topk=self.enable_topK,
                                         prefill_chunk_len=self.prefill_chunk_len(max(1, self.batch_size),
                                                                                  max(c.length for c in chunk)))
        batches = plan_batches(chunk, max(1, self.batch_size))[rank::max(1, world)]
        done = 0
        t0 = time.time()
        with progress(total=len(chunk), desc="Convos", leave=False) as bar:
            set_status(bar, "Generating...")
            hbt = getattr(self, "heartbeat", None)
            def deliver(rows, convos):
                nonlocal done
                if sha_by_id:   # the store is keyed by the STUDENT's view of the text (that is what sync compares)
                    for r in rows:
                        r.content_sha = sha_by_id.get(r.convo_id, r.content_sha)
                if not last_teacher:     # more teachers follow: the conversation is not complete yet (data/convo.py)
                    for r in rows:
                        r.content_sha = PARTIAL_SHA_PREFIX + (r.content_sha or "")
                data_manager.write_batch(rows)          # asynchronous: compression + file IO overlap the next batch
                self.tokens_collected += int(sum(c.length for c in convos))
                done += len(rows)
                bar.update(len(convos))

            # one batch deep: batch i+1 is queued on the GPU before batch i's rows are waited for, so the device
            # never idles during the copy to the host and the hand-off to the writer
            # (on CPU there is nothing to overlap: the plain per-batch call runs)
            pipelined = (aligner is None and tp_group is None and hasattr(collector, "rows_of")
                         and collector.device.type == "cuda")
            pending = None
            for tokens, convos in batches:
                if hbt is not None:      # between batches: a lost peer is noticed before the next launch
                    hbt.beat(done, "collect")
                    hbt.check()
                if pipelined:
                    ticket = collector.submit(tokens, convos)
                    if pending is not None:
                        deliver(collector.rows_of(*pending), pending[1])
                    pending = (ticket, convos)
                else:
                    deliver(collector.collect_batch(tokens, convos, aligner=aligner, validation=validation), convos)
            if pending is not None:
                deliver(collector.rows_of(*pending), pending[1])
            with status(bar, "Writing rows..."):
                data_manager.wait()
        self.collect_seconds += time.time() - t0
        return done

    def close(self) -> None:
        self.unload()
        self.dataset, self.validation_dataset = [], []
        self.dataset_len = 0
        self.dataset_sorted = self.validation_dataset_sorted = False
