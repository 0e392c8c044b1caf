"""Token-embedding table stored as int8 (`src/kohakumoss/quant/embedding.py:16-60`).

A text encoder's embedding table (a quarter of a billion weights for a 150k vocabulary at 4096)
is read a few rows at a time: stored as int8 rows with one fp32 scale each (optionally rotated
by the group Hadamard, ConvRot), a lookup gathers the rows it needs, widens them and undoes the
rotation. The table may live on the host while the encoder runs on the device: `lookup` gathers
where the table is and moves only the gathered rows.
"""

from __future__ import annotations

import torch
from torch import Tensor, nn

from .formats import group_hadamard, quantize_weight_int8


class QuantEmbedding(nn.Module):
    def __init__(self, q: Tensor, scale: Tensor, rotation: int = 0, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.num_embeddings, self.embedding_dim = q.shape
        self.rotation, self.dtype = int(rotation), dtype
        self.register_buffer("q", q)
        self.register_buffer("scale", scale.float().reshape(-1))

    @classmethod
    def from_embedding(cls, emb: nn.Embedding | Tensor, rotation: int = 0, dtype: torch.dtype | None = None) -> "QuantEmbedding":
        w = emb.weight if isinstance(emb, nn.Embedding) else emb
        q, s = quantize_weight_int8(w, rotation)
        return cls(q, s, rotation, dtype or w.dtype)

    def finish(self, rows: Tensor, scales: Tensor) -> Tensor:
        """Gathered int8 rows [..., D] and their scales [...] -> embeddings."""
        x = rows.float() * scales.float().unsqueeze(-1)
        if self.rotation > 1:
            x = group_hadamard(x, self.rotation)      # the rotation is its own inverse
        return x.to(self.dtype)

    def forward(self, ids: Tensor) -> Tensor:
        return self.finish(self.q[ids], self.scale[ids])

    def lookup(self, ids: Tensor, device) -> Tensor:
        """Embeddings on `device` of ids gathered where the table lives."""
        at = ids.to(self.q.device)
        return self.finish(self.q[at].to(device, non_blocking=True), self.scale[at].to(device, non_blocking=True))

    def state(self, prefix: str) -> dict[str, Tensor]:
        out = {prefix + "weight": self.q, prefix + "weight_scale": self.scale}
        if self.rotation > 1:
            out[prefix + "rotation_group"] = torch.tensor(self.rotation, dtype=torch.int32)
        return out
