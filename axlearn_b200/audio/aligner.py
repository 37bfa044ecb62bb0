"""CTC forced alignment: the most likely frame-level path for a known label sequence.

Counterpart of axlearn/audio/aligner/ (``ctc_forced_alignment``, used by
``CTCDecoderModel.align``, axlearn/audio/decoder_asr.py:623-647).  Viterbi over the expanded label
sequence ``blank, y1, blank, y2, ..., blank``: a state may stay, advance by one, or skip a blank
between two different labels.  Batched over utterances with ragged frame and label counts.
"""

from __future__ import annotations

import dataclasses

import torch

Tensor = torch.Tensor
_NEG = -1e30


@dataclasses.dataclass
class AlignmentOutput:
    alignment: Tensor          # [B, T] label id per frame (blank where CTC emits blank; -1 on padding)
    alignment_indices: Tensor  # [B, T] index into the label sequence per frame (-1 for blank / padding)
    alignment_score: Tensor    # [B] log-probability of the best path

    def asdict(self) -> dict:
        return dataclasses.asdict(self)


def ctc_forced_alignment(*, log_pos: Tensor, log_pos_paddings: Tensor, labels: Tensor, label_paddings: Tensor,
                         blank_id: int = 0) -> AlignmentOutput:
    """``log_pos [B, T, V]`` frame log-posteriors, ``labels [B, U]``.  An utterance whose labels do
    not fit its frames gets score ``-inf`` and an all-blank alignment."""
    b, t_max, _ = log_pos.shape
    u_max = labels.shape[1]
    s_max = 2 * u_max + 1
    dev = log_pos.device
    frames = (~log_pos_paddings.bool()).sum(-1)
    num_labels = (~label_paddings.bool()).sum(-1)
    ext = torch.full((b, s_max), blank_id, dtype=torch.long, device=dev)
    ext[:, 1::2] = labels.clamp_min(0).long()
    state = torch.arange(s_max, device=dev)[None]
    live_state = state < (2 * num_labels + 1)[:, None]
    # Skipping the blank between labels u-1 and u is allowed when they differ.
    can_skip = torch.zeros(b, s_max, dtype=torch.bool, device=dev)
    can_skip[:, 3::2] = ext[:, 3::2] != ext[:, 1:-2:2]
    emit = torch.gather(log_pos.float(), 2, ext[:, None, :].expand(-1, t_max, -1))       # [B, T, S]

    score = torch.full((b, s_max), _NEG, device=dev)
    score[:, 0] = emit[:, 0, 0]
    if s_max > 1:
        score[:, 1] = torch.where(num_labels > 0, emit[:, 0, 1], torch.full_like(emit[:, 0, 1], _NEG))
    back = torch.zeros(b, t_max, s_max, dtype=torch.long, device=dev)                    # 0 stay, 1 advance, 2 skip
    for t in range(1, t_max):
        stay = score
        adv = torch.cat([score.new_full((b, 1), _NEG), score[:, :-1]], dim=1)
        skip = torch.cat([score.new_full((b, 2), _NEG), score[:, :-2]], dim=1)
        skip = torch.where(can_skip, skip, torch.full_like(skip, _NEG))
        cand = torch.stack([stay, adv, skip], dim=-1)
        best, arg = cand.max(dim=-1)
        new = torch.where(live_state, best + emit[:, t], torch.full_like(best, _NEG))
        active = (t < frames)[:, None]
        score = torch.where(active, new, score)
        back[:, t] = torch.where(active, arg, torch.zeros_like(arg))
    # The path ends in the last blank or the last label.
    last = 2 * num_labels
    rows = torch.arange(b, device=dev)
    end_blank = score[rows, last]
    end_label = torch.where(num_labels > 0, score[rows, (last - 1).clamp_min(0)], torch.full_like(end_blank, _NEG))
    final_score = torch.maximum(end_blank, end_label)
    cur = torch.where(end_label > end_blank, last - 1, last)
    path = torch.zeros(b, t_max, dtype=torch.long, device=dev)
    for t in range(t_max - 1, -1, -1):
        inside = t < frames
        path[:, t] = torch.where(inside, cur, torch.zeros_like(cur))
        step = back[rows, t, cur]
        cur = torch.where(inside & (t > 0), cur - step, cur)
    ok = final_score > _NEG / 2
    frame_live = torch.arange(t_max, device=dev)[None] < frames[:, None]
    is_label = (path % 2 == 1) & ok[:, None]
    alignment = torch.where(is_label, torch.gather(ext, 1, path), torch.full_like(path, blank_id))
    alignment = torch.where(frame_live, alignment, torch.full_like(alignment, -1))
    indices = torch.where(is_label & frame_live, path // 2, torch.full_like(path, -1))
    return AlignmentOutput(alignment=alignment, alignment_indices=indices,
                           alignment_score=torch.where(ok, final_score, torch.full_like(final_score, float("-inf"))))
