"""OaBpeTokenizer: byte-level BPE (Source/Public/Oa/Ml/Tokenizer.h:16-58, Source/Private/Oa/Ml/Tokenizer.cpp).

Ids 0..255 are bytes; merge i creates id 256 + i.  Training picks, at every round, the most frequent adjacent pair (ties go
to the smallest (left, right) pair) and stops when no pair occurs twice.  Encoding applies the merges in rank order.  The
file format is text: the magic line, the merge count, then one "left right" line per merge.
"""
from __future__ import annotations

from collections import Counter
from typing import Sequence

from ..core.types import OaStatus, OaStatusCode

_MAGIC = "oa_bpe_v1"


class OaBpeTokenizer:
    def __init__(self, target_vocab: int = 512):
        self.TargetVocab = max(256, int(target_vocab))
        self.Merges: list[tuple[int, int]] = []

    @staticmethod
    def _apply(ids: list, pair: tuple, new_id: int) -> list:
        out, i, n = [], 0, len(ids)
        left, right = pair
        while i < n:
            if i + 1 < n and ids[i] == left and ids[i + 1] == right:
                out.append(new_id)
                i += 2
            else:
                out.append(ids[i])
                i += 1
        return out

    def Train(self, text, num_merges: int) -> None:
        self.Merges = []
        if text is None or num_merges <= 0:
            return
        ids = list(text.encode("utf-8") if isinstance(text, str) else bytes(text))
        for _ in range(min(int(num_merges), self.TargetVocab - 256)):
            if len(ids) < 2:
                break
            counts = Counter(zip(ids, ids[1:]))
            top = max(counts.values())
            if top < 2:
                break
            pair = min(p for p, c in counts.items() if c == top)
            ids = self._apply(ids, pair, 256 + len(self.Merges))
            self.Merges.append(pair)

    def Encode(self, text) -> list:
        ids = list(text.encode("utf-8") if isinstance(text, str) else bytes(text))
        for rank, pair in enumerate(self.Merges):
            ids = self._apply(ids, pair, 256 + rank)
        return ids

    def _expand(self, token: int, out: bytearray) -> None:
        if token < 0:
            return
        if token < 256:
            out.append(token)
            return
        rank = token - 256
        if rank < len(self.Merges):
            self._expand(self.Merges[rank][0], out)
            self._expand(self.Merges[rank][1], out)

    def DecodeBytes(self, tokens: Sequence[int]) -> bytes:
        out = bytearray()
        for t in tokens:
            self._expand(int(t), out)
        return bytes(out)

    def Decode(self, tokens: Sequence[int]) -> str:
        return self.DecodeBytes(tokens).decode("utf-8", errors="replace")

    def EncodePrompt(self, prompt, context_len: int) -> list:
        """The last `context_len` tokens of the prompt, left-padded with id 0."""
        toks = self.Encode(prompt)[-context_len:]
        return [0] * (context_len - len(toks)) + toks

    def VocabSize(self) -> int:
        return 256 + len(self.Merges)

    def NumMerges(self) -> int:
        return len(self.Merges)

    def Save(self, path: str) -> OaStatus:
        try:
            with open(path, "w") as f:
                f.write(f"{_MAGIC}\n{len(self.Merges)}\n")
                for left, right in self.Merges:
                    f.write(f"{left} {right}\n")
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"OaBpeTokenizer: cannot write {path}: {e}")
        return OaStatus.Ok()

    def Load(self, path: str) -> OaStatus:
        try:
            lines = open(path).read().split("\n")
        except OSError:
            return OaStatus.Error(OaStatusCode.NotFound, f"OaBpeTokenizer: cannot read {path}")
        try:
            if lines[0] != _MAGIC:
                raise ValueError("magic")
            count = int(lines[1])
            if count > 1_000_000:
                raise ValueError("count")
            merges = []
            for i in range(count):
                left, right = (int(x) for x in lines[2 + i].split())
                if not (0 <= left < 256 + i and 0 <= right < 256 + i):
                    raise ValueError("merge refers to a later token")
                merges.append((left, right))
        except (ValueError, IndexError) as e:
            return OaStatus.Error(OaStatusCode.DataLoss, f"OaBpeTokenizer: invalid file {path} ({e})")
        self.Merges = merges
        self.TargetVocab = self.VocabSize()
        return OaStatus.Ok()
