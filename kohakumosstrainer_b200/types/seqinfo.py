"""SeqInfo: layout descriptor of one packed variable-length batch, built on the host.

Layout contract (reference: `src/kohakumoss/types/seqinfo.py:28-190`): image tokens of
all samples are packed sample-major / row-major on one axis, text tokens on another; the
joint sequence of sample i is `[img_i ; txt_i]`. Positions are fp32 `[N, 4] = (r, f, h, w)`:
image tokens carry `f = text_len_i`, centred `h`, `w`; text token j carries `f = j`.
Only attention reads sample boundaries (`cu_seqlens`); everything else is per token.

The builder here is vectorised (no per-sample Python tensor ops beyond `repeat_interleave`)
and `to()` ships all fields as ONE pinned byte buffer and one async H2D copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import Tensor


@dataclass
class AttnPlan:
    """Segment boundaries of one attention call. `lengths` stays on the host so kernels
    never need a device read-back to size their grids."""

    cu_seqlens: Tensor
    max_seqlen: int
    lengths: tuple[int, ...]
    extra: dict = field(default_factory=dict)

    @property
    def total(self) -> int:
        return sum(self.lengths)


@dataclass
class SeqInfo:
    batch: int
    hw: Tensor
    text_len: Tensor
    cu_img: Tensor
    cu_txt: Tensor
    n_img: int
    n_txt: int
    seg_img: Tensor
    seg_txt: Tensor
    seg_joint: Tensor
    pos_txt: Tensor
    pos_joint: Tensor
    img_in_joint: Tensor
    txt_in_joint: Tensor
    attn_joint: AttnPlan
    attn_text: AttnPlan

    @property
    def n_joint(self) -> int:
        return self.n_img + self.n_txt

    def _tensor_fields(self) -> list[tuple[str, Tensor]]:
        out = []
        for name, value in self.__dict__.items():
            if isinstance(value, Tensor):
                out.append((name, value))
            elif isinstance(value, AttnPlan):
                out.append((name, value.cu_seqlens))
        return out

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for _, t in self._tensor_fields())

    def pin_memory(self) -> "SeqInfo":
        for name, value in list(self.__dict__.items()):
            if isinstance(value, Tensor) and value.device.type == "cpu" and not value.is_pinned():
                setattr(self, name, value.pin_memory())
            elif isinstance(value, AttnPlan) and not value.cu_seqlens.is_pinned():
                value.cu_seqlens = value.cu_seqlens.pin_memory()
        return self

    def to(self, device, non_blocking: bool = True) -> "SeqInfo":
        """Move every tensor to `device`. Host -> accelerator goes as a single staged
        byte buffer (16-byte aligned slots) and one copy; fields become views of it."""
        device = torch.device(device)
        fields = self._tensor_fields()
        moved = dict(self.__dict__)
        host = all(t.device.type == "cpu" for _, t in fields)
        if device.type == "cpu" or not host:
            new = {name: t.to(device, non_blocking=non_blocking) for name, t in fields}
        else:
            offsets, total = [], 0
            for _, t in fields:
                offsets.append(total)
                total += (t.numel() * t.element_size() + 15) // 16 * 16
            stage = torch.empty(max(total, 16), dtype=torch.uint8)
            if torch.cuda.is_available():
                stage = stage.pin_memory()
            for (name, t), off in zip(fields, offsets):
                n = t.numel() * t.element_size()
                if n:
                    stage[off : off + n] = t.contiguous().view(-1).view(torch.uint8)
            dev = stage.to(device, non_blocking=non_blocking)
            new = {}
            for (name, t), off in zip(fields, offsets):
                n = t.numel() * t.element_size()
                new[name] = dev[off : off + n].view(t.dtype).view(t.shape)
        for name, value in self.__dict__.items():
            if isinstance(value, AttnPlan):
                moved[name] = AttnPlan(new[name], value.max_seqlen, value.lengths, dict(value.extra))
            elif isinstance(value, Tensor):
                moved[name] = new[name]
        return SeqInfo(**moved)


def _cu(lengths: Tensor) -> Tensor:
    cu = torch.zeros(lengths.numel() + 1, dtype=torch.int32)
    cu[1:] = lengths.cumsum(0)
    return cu


def _plan(lengths: Tensor) -> AttnPlan:
    lens = tuple(int(v) for v in lengths.tolist())
    return AttnPlan(_cu(lengths), max(lens, default=0), lens)


def _within(lengths: Tensor) -> tuple[Tensor, Tensor]:
    """For packed segments of `lengths`: (segment id per element, index inside segment)."""
    seg = torch.repeat_interleave(torch.arange(lengths.numel()), lengths)
    starts = torch.cumsum(lengths, 0) - lengths
    inner = torch.arange(int(lengths.sum())) - starts[seg]
    return seg, inner


def build_seqinfo(
    hw: Tensor,
    text_len: Tensor,
    rope_axes: int = 4,
    img_keep: list[Tensor | None] | None = None,
) -> SeqInfo:
    """Host-side SeqInfo from latent grids `hw` [B, 2] and text lengths [B].

    `img_keep[i]` (sorted int64 indices into sample i's row-major grid, or None) keeps only
    those image tokens; kept tokens retain their original grid positions.
    """
    hw = torch.as_tensor(hw).to(torch.int64).cpu().reshape(-1, 2)
    text_len = torch.as_tensor(text_len).to(torch.int64).cpu().reshape(-1)
    batch = hw.shape[0]
    full = hw[:, 0] * hw[:, 1]
    seg_f, idx_f = _within(full)
    w_of = hw[seg_f, 1]
    ys = torch.div(idx_f, w_of, rounding_mode="floor")
    xs = idx_f - ys * w_of
    pos_img = torch.zeros(int(full.sum()), rope_axes, dtype=torch.float32)
    pos_img[:, 1] = text_len[seg_f].float()
    pos_img[:, 2] = ys.float() - (hw[seg_f, 0].float() - 1) / 2
    pos_img[:, 3] = xs.float() - (w_of.float() - 1) / 2
    if img_keep is not None and any(k is not None for k in img_keep):
        starts = torch.cumsum(full, 0) - full
        pick = [
            (torch.arange(int(full[i])) if k is None else k.to(torch.int64)) + starts[i]
            for i, k in enumerate(img_keep)
        ]
        img_lens = torch.tensor([p.numel() for p in pick], dtype=torch.int64)
        pos_img = pos_img.index_select(0, torch.cat(pick)) if pick else pos_img
    else:
        img_lens = full
    seg_i, _ = _within(img_lens)
    seg_t, idx_t = _within(text_len)
    pos_txt = torch.zeros(int(text_len.sum()), rope_axes, dtype=torch.float32)
    pos_txt[:, 1] = idx_t.float()

    joint_lens = img_lens + text_len
    joint_start = torch.cumsum(joint_lens, 0) - joint_lens
    img_start = torch.cumsum(img_lens, 0) - img_lens
    img_in_joint = torch.arange(int(img_lens.sum())) - img_start[seg_i] + joint_start[seg_i]
    txt_in_joint = idx_t + joint_start[seg_t] + img_lens[seg_t]
    n_joint = int(joint_lens.sum())
    pos_joint = torch.zeros(n_joint, rope_axes, dtype=torch.float32)
    pos_joint[img_in_joint] = pos_img
    pos_joint[txt_in_joint] = pos_txt
    seg_joint = torch.repeat_interleave(torch.arange(batch), joint_lens).to(torch.int32)

    return SeqInfo(
        batch=batch,
        hw=hw,
        text_len=text_len,
        cu_img=_cu(img_lens),
        cu_txt=_cu(text_len),
        n_img=int(img_lens.sum()),
        n_txt=int(text_len.sum()),
        seg_img=seg_i.to(torch.int32),
        seg_txt=seg_t.to(torch.int32),
        seg_joint=seg_joint,
        pos_txt=pos_txt,
        pos_joint=pos_joint,
        img_in_joint=img_in_joint,
        txt_in_joint=txt_in_joint,
        attn_joint=_plan(joint_lens),
        attn_text=_plan(text_len),
    )
