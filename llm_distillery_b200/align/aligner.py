"""Cross-tokenizer alignment: use a teacher whose vocabulary differs from the student's.

The reference refuses such teachers (collect_and_finetune.py:83-101) and only offers ``crop_distr_to_size``.
Here a teacher of another vocabulary family is mapped onto the student's vocabulary in two steps:

1. *Positions.* Both models tokenise the same text; a student content row (the distribution of the token that
   starts at byte offset b) is paired with the teacher position whose next token also starts at byte b. Rows
   without a common boundary get no target from this teacher (an all ``-inf`` row: merging adds nothing, the loss
   ignores it).
2. *Mass.* A byte-level trie over the student vocabulary gives every teacher token the student token that is the
   LONGEST prefix of its byte string (what a greedy longest-match tokenizer would emit first); the walk depends
   only on the token, so it is tabulated once per tokenizer pair (``build_vocab_map``; on a GPU the whole teacher
   vocabulary is walked through the flattened trie by the ``trie_walk`` kernel, csrc/align/trie.cu). Per position the teacher's
   top-K probabilities are sent through the table, probabilities meeting on one student id are summed, the best K
   are kept (kernel ``remap_topk``; PyTorch restatement in ``ops.topk``). Total mass never grows; it is conserved
   exactly when every teacher token has an image (byte-fallback vocabularies always do).

Both models must use the same prompt-format text, so that the two token streams spell the same bytes.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import topk as topk_ops


def _gpt2_byte_decoder() -> dict[str, int]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for b, c in zip(bs, cs)}


def token_bytes(tokenizer) -> list[bytes]:
    """Byte string spelled by every token id (special / added tokens spell nothing)."""
    vocab = tokenizer.get_vocab()
    size = max(vocab.values()) + 1
    out = [b""] * size
    added = set(tokenizer.get_added_vocab().keys()) | set(getattr(tokenizer, "all_special_tokens", []))
    byte_level = any(t.startswith("Ġ") or t.startswith("Ċ") for t in vocab)
    dec = _gpt2_byte_decoder() if byte_level else None
    for tok, i in vocab.items():
        if tok in added:
            continue
        if len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            try:
                out[i] = bytes([int(tok[3:5], 16)])
                continue
            except ValueError:
                pass
        if dec is not None and all(ch in dec for ch in tok):
            out[i] = bytes(dec[ch] for ch in tok)
        else:
            out[i] = tok.replace("▁", " ").encode("utf-8")
    return out


class ByteTrie:
    """Trie over byte strings; ``longest_prefix(b)`` returns the id of the longest stored string that prefixes b."""

    def __init__(self):
        self.children: list[dict[int, int]] = [{}]
        self.value: list[int] = [-1]

    def insert(self, key: bytes, value: int) -> None:
        node = 0
        for ch in key:
            nxt = self.children[node].get(ch)
            if nxt is None:
                nxt = len(self.children)
                self.children[node][ch] = nxt
                self.children.append({})
                self.value.append(-1)
            node = nxt
        if self.value[node] < 0 or value < self.value[node]:
            self.value[node] = value      # duplicates: keep the lowest id

    def flatten(self) -> dict[str, np.ndarray]:
        """The trie as flat arrays for the walk kernel: node n owns edges ``edge_start[n] .. edge_start[n+1]-1`` sorted
        by byte; edge e leads to node ``edge_child[e]``; ``node_value[n]`` is the id stored at n (-1: none)."""
        n = len(self.children)
        counts = np.fromiter((len(c) for c in self.children), dtype=np.int32, count=n)
        start = np.zeros(n + 1, dtype=np.int32)
        np.cumsum(counts, out=start[1:])
        edge_byte = np.zeros(max(1, int(start[-1])), dtype=np.uint8)
        edge_child = np.zeros(max(1, int(start[-1])), dtype=np.int32)
        for i, c in enumerate(self.children):
            if c:
                ks = sorted(c)
                a = int(start[i])
                edge_byte[a:a + len(ks)] = ks
                edge_child[a:a + len(ks)] = [c[k] for k in ks]
        return {"edge_start": start, "edge_byte": edge_byte, "edge_child": edge_child,
                "node_value": np.asarray(self.value, dtype=np.int32)}

    def longest_prefix(self, key: bytes) -> int:
        node, best = 0, -1
        for ch in key:
            node = self.children[node].get(ch, -1)
            if node < 0:
                break
            if self.value[node] >= 0:
                best = self.value[node]
        return best


def flat_trie(student_bytes: list[bytes], student_vocab_limit: int | None = None) -> dict[str, np.ndarray]:
    """Flattened byte trie of a vocabulary (``ByteTrie.flatten`` layout), built by the native host library when it is
    there (csrc/align/trie_build.cc: same node numbering, tens of milliseconds for 128k tokens) and by the dictionary
    trie otherwise."""
    import ctypes
    from ..ops import _lib
    n = len(student_bytes) if student_vocab_limit is None else min(len(student_bytes), student_vocab_limit)
    toks = student_bytes[:n]
    try:
        lib = _lib.host()
        build = lib.b200_trie_build
    except (OSError, AttributeError):
        lib = None
    if lib is None:
        trie = ByteTrie()
        for i, b in enumerate(toks):
            if b:
                trie.insert(b, i)
        return trie.flatten()
    lens = np.fromiter((len(b) for b in toks), dtype=np.int64, count=n)
    off = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(lens, out=off[1:])
    blob = np.frombuffer(b"".join(toks) or b"\0", dtype=np.uint8)
    ids = np.arange(n, dtype=np.int32)
    vp = ctypes.c_void_p
    build.restype = vp
    build.argtypes = [vp, vp, vp, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_longlong)]
    lib.b200_trie_export.argtypes = [vp, vp, vp, vp, vp]
    lib.b200_trie_free.argtypes = [vp]
    n_nodes, n_edges = ctypes.c_int(0), ctypes.c_longlong(0)
    h = build(blob.ctypes.data, off.ctypes.data, ids.ctypes.data, n, ctypes.byref(n_nodes), ctypes.byref(n_edges))
    if not h:
        raise RuntimeError("b200_trie_build refused its arguments")
    try:
        out = {"edge_start": np.zeros(n_nodes.value + 1, dtype=np.int32),
               "edge_byte": np.zeros(max(1, n_edges.value), dtype=np.uint8),
               "edge_child": np.zeros(max(1, n_edges.value), dtype=np.int32),
               "node_value": np.zeros(n_nodes.value, dtype=np.int32)}
        if lib.b200_trie_export(h, out["edge_start"].ctypes.data, out["edge_byte"].ctypes.data,
                                out["edge_child"].ctypes.data, out["node_value"].ctypes.data) != 0:
            raise RuntimeError("b200_trie_export failed")
    finally:
        lib.b200_trie_free(h)
    return out


def vocab_map_from_bytes(teacher_bytes: list[bytes], student_bytes: list[bytes], student_vocab_limit: int | None = None,
                         device=None) -> np.ndarray:
    """int32 [teacher vocab]: the student token that is the longest byte-prefix of each teacher token (-1: none).
    On a CUDA ``device`` the whole teacher vocabulary is walked through the flattened trie by one kernel launch
    (``ops.topk.trie_walk``); otherwise token by token in Python."""
    if device is not None and torch.device(device).type == "cuda" and teacher_bytes:
        return topk_ops.trie_walk(flat_trie(student_bytes, student_vocab_limit), teacher_bytes, device)[0].cpu().numpy()
    trie = ByteTrie()
    for i, b in enumerate(student_bytes):
        if b and (student_vocab_limit is None or i < student_vocab_limit):
            trie.insert(b, i)
    return np.asarray([trie.longest_prefix(b) if b else -1 for b in teacher_bytes], dtype=np.int32)


def build_vocab_map(teacher_tokenizer, student_tokenizer, student_vocab_limit: int | None = None, device=None) -> np.ndarray:
    return vocab_map_from_bytes(token_bytes(teacher_tokenizer), token_bytes(student_tokenizer), student_vocab_limit, device)


def start_offsets(tokens: np.ndarray, length: int, tok_bytes: list[bytes]) -> np.ndarray:
    """offsets[p] = byte offset at which token p starts; offsets[length] = total bytes."""
    lens = np.fromiter((len(tok_bytes[t]) if 0 <= t < len(tok_bytes) else 0 for t in tokens[:length]), dtype=np.int64,
                       count=length)
    return np.concatenate([[0], np.cumsum(lens)])


def align_positions(student_convo, teacher_convo, student_bytes, teacher_bytes) -> np.ndarray:
    """For every student content row: the teacher position predicting a token that starts at the same byte, or -1."""
    so = start_offsets(student_convo.tokenized, student_convo.length, student_bytes)
    to = start_offsets(teacher_convo.tokenized, teacher_convo.length, teacher_bytes)
    ci = student_convo.content_indices()
    ci = ci[ci < student_convo.length]
    # teacher position p predicts token p+1, which starts at to[p+1]; zero-length (special) tokens share an offset
    # with their successor: prefer the LAST position with that boundary (the one right before real text)
    boundary_to_pos = {}
    for p in range(teacher_convo.length - 1):
        boundary_to_pos[int(to[p + 1])] = p
    out = np.full(len(ci), -1, dtype=np.int64)
    for r, p in enumerate(ci):
        if p + 1 < student_convo.length:
            out[r] = boundary_to_pos.get(int(so[p + 1]), -1)
    return out


class VocabAligner:
    def __init__(self, teacher_tokenizer, student_tokenizer, student_dataset, student_validation_dataset,
                 student_vocab_limit: int | None = None, device=None):
        self.table_np = build_vocab_map(teacher_tokenizer, student_tokenizer, student_vocab_limit, device)
        self.table = torch.from_numpy(self.table_np)
        self.student_bytes = token_bytes(student_tokenizer)
        self.teacher_bytes = token_bytes(teacher_tokenizer)
        self.student_convos = {c.origin_convo_id: c for c in student_dataset}
        self.student_val_convos = {c.origin_convo_id: c for c in student_validation_dataset}
        self.coverage = float((self.table_np >= 0).mean())

    def positions_for(self, teacher_convo, validation: bool) -> np.ndarray | None:
        s = (self.student_val_convos if validation else self.student_convos).get(teacher_convo.origin_convo_id)
        if s is None:
            return None
        return align_positions(s, teacher_convo, self.student_bytes, self.teacher_bytes)

    def remap(self, logp: torch.Tensor, ids: torch.Tensor, k_out: int):
        table = self.table.to(logp.device)
        return topk_ops.remap_topk(logp.float(), ids.int(), table, k_out)


def attach_aligners(teachers, student) -> None:
    """Give every teacher whose vocabulary differs from the student's a ``VocabAligner``."""
    from ..data.tokenize import load_tokenizer
    s_tok = load_tokenizer(student.model_path)
    for t in teachers:
        if getattr(t, "needs_alignment", False):
            t.aligner = VocabAligner(load_tokenizer(t.model_path), s_tok, student.dataset, student.validation_dataset,
                                     student_vocab_limit=student.crop_to_size or None,
                                     device=getattr(student, "device", None))
            print(f"{t.model_name}: cross-tokenizer alignment, {100 * t.aligner.coverage:.1f}% of its tokens have an "
                  f"image in the student vocabulary")
