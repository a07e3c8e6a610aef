"""Text segments and images in order → one token sequence with placeholder tokens where the image embeddings go
(the reference's ``MultimodalPrompt``, ``oxidize-core/src/vision/prompt.rs:4-60``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple, Union

import torch


@dataclass
class MultimodalPrompt:
    parts: List[Union[str, torch.Tensor]] = field(default_factory=list)

    def add_text(self, text: str) -> "MultimodalPrompt":
        self.parts.append(text)
        return self

    def add_image(self, embeddings: torch.Tensor) -> "MultimodalPrompt":
        """``embeddings``: [image tokens, hidden] rows in the language model's embedding space."""
        if embeddings.ndim != 2 or embeddings.shape[0] == 0:
            raise ValueError("image embeddings must be [tokens, hidden] with at least one row")
        self.parts.append(embeddings)
        return self

    def build(self, tokenizer, placeholder_id: int, add_bos: bool = True) -> Tuple[List[int], List[int], torch.Tensor]:
        """(token ids, positions that take an embedding row instead of their token's, the rows [n, hidden])."""
        ids: List[int] = []
        positions: List[int] = []
        rows: List[torch.Tensor] = []
        first_text = True
        for p in self.parts:
            if isinstance(p, str):
                if not p:
                    continue
                toks = tokenizer.encode_with_special_tokens(p, add_bos=add_bos and first_text and not ids)
                first_text = False
                ids.extend(int(t) for t in toks)
            else:
                if rows and rows[0].shape[1] != p.shape[1]:
                    raise ValueError("all images must have the same embedding width")
                positions.extend(range(len(ids), len(ids) + p.shape[0]))
                ids.extend([placeholder_id] * p.shape[0])
                rows.append(p)
        if not ids:
            raise ValueError("empty prompt")
        return ids, positions, (torch.cat(rows, dim=0) if rows else torch.empty(0, 0))
