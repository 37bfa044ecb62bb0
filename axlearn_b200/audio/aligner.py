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


def alignment_to_segments(alignment: Tensor, blank_id: int) -> Tensor:
    """``[B, T]`` frame labels (negative = padding) -> ``[B, T, 2]`` segments: row ``l`` holds the
    start frame (inclusive) and end frame (exclusive) of the l-th emitted label, ``-1`` beyond the
    last label.  A label's segment runs to the start of the next label (trailing blanks belong to
    it); the last one runs to the number of frames (axlearn/audio/aligner/ctc_aligner.py:611)."""
    b, t = alignment.shape
    dev = alignment.device
    prev = torch.cat([alignment.new_full((b, 1), -1), alignment[:, :-1]], dim=1)
    starts_here = (alignment != prev) & (alignment != blank_id) & (alignment >= 0)
    frame = torch.arange(t, device=dev)[None].expand(b, -1)
    starts = torch.where(starts_here, frame, torch.full_like(frame, t + 1)).sort(dim=-1).values
    starts = torch.where(starts == t + 1, torch.full_like(starts, -1), starts)
    ends = torch.cat([starts[:, 1:], starts.new_full((b, 1), -1)], dim=1)
    count = (starts >= 0).sum(-1)
    frames = (alignment >= 0).sum(-1)
    rows = torch.arange(b, device=dev)
    has = count > 0
    last = (count - 1).clamp_min(0)
    ends[rows[has], last[has]] = frames[has]
    return torch.stack([starts, ends], dim=-1)


class CtcAligner:
    """Forced alignment of ONE utterance on the host (numpy in, numpy out): the offline tool form of
    ``ctc_forced_alignment`` (axlearn/audio/aligner/ctc_aligner.py:31-188)."""

    def __init__(self, vocab_size: int, blank_id: int = 0):
        if blank_id != 0:
            raise ValueError("Only blank_id == 0 is supported.")
        self.blank_id = blank_id
        self.vocab_size = vocab_size

    def _check_input(self, log_posterior, ground_truth) -> None:
        import numpy as np

        if log_posterior.ndim != 2:
            raise ValueError(f"Expecting log_posterior is a 2-D tensor, but got {log_posterior.shape}.")
        if log_posterior.shape[1] != self.vocab_size:
            raise ValueError(f"Expecting vocab_size to be {self.vocab_size}, but got {log_posterior.shape[1]}.")
        if ground_truth.ndim != 1:
            raise ValueError(f"Expecting ground_truth is a 1-D tensor, but got {ground_truth.shape}.")
        if ground_truth.dtype != np.int32:
            raise ValueError(f"Ground_truth must have a int32 dtype, got {ground_truth.dtype}")
        if ground_truth.size and (ground_truth.max() >= self.vocab_size or ground_truth.min() < 0):
            raise ValueError(f"Ground truth label must be in range [0, {self.vocab_size}), "
                             f"but we got [{ground_truth.min()}, {ground_truth.max()}].")

    def align(self, log_posterior, ground_truth):
        """``log_posterior [T, V]``, ``ground_truth [W]`` int32 -> ``[T]`` int32 frame labels, or
        None when the labels do not fit the frames."""
        import numpy as np

        self._check_input(log_posterior, ground_truth)
        t, w = log_posterior.shape[0], ground_truth.shape[0]
        out = ctc_forced_alignment(
            log_pos=torch.from_numpy(np.asarray(log_posterior, dtype=np.float32))[None],
            log_pos_paddings=torch.zeros(1, t, dtype=torch.bool),
            labels=torch.from_numpy(ground_truth.astype(np.int64))[None].reshape(1, w),
            label_paddings=torch.zeros(1, w, dtype=torch.bool), blank_id=self.blank_id)
        if not torch.isfinite(out.alignment_score[0]):
            return None
        return out.alignment[0].numpy().astype(np.int32)

    def alignment_to_boundary(self, alignment, ground_truth):
        """``[2, W]``: row 0 the first frame of every label, row 1 the frame after its last one (a
        label's span includes the blanks that follow it)."""
        import numpy as np

        ext = np.concatenate([alignment, np.array([self.blank_id], dtype=np.int32)])
        shifted = np.roll(ext, 1)
        mask = (shifted != ext) & (ext != self.blank_id)
        if not np.array_equal(ext[mask], ground_truth):
            raise ValueError(f"{alignment} is not a valid alignment for {ground_truth}")
        start = np.where(mask)[0].astype(np.int32)
        end = np.roll(start, -1)
        if end.size:
            end[-1] = alignment.shape[0]
        return np.stack([start, end], axis=0)
