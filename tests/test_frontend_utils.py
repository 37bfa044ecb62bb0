"""Audio frontend helpers (vectors: axlearn/audio/frontend_utils_test.py:50-120)."""

import numpy as np
import pytest
import torch

from axlearn_b200.audio import frontend_utils as fu


@pytest.mark.parametrize("seq_len,frame_size,hop_size,expected", [(0, 5, 2, 0), (1, 5, 2, 1), (7, 5, 2, 2), (8, 5, 2, 3), (9, 5, 2, 3)])
def test_num_frames(seq_len, frame_size, hop_size, expected):
    assert fu.num_frames(seq_len, frame_size=frame_size, hop_size=hop_size) == expected
    assert fu.num_frames(torch.tensor([seq_len]), frame_size=frame_size, hop_size=hop_size).tolist() == [expected]
    with pytest.raises(ValueError):
        fu.num_frames(-1, frame_size=5, hop_size=2)


def test_frame_keeps_a_partial_frame():
    frames = fu.frame(torch.arange(20)[None], frame_size=15, hop_size=10)
    assert frames.tolist() == [[list(range(15)), list(range(10, 20)) + [0] * 5]]
    assert fu.frame(torch.zeros(2, 3, 0), frame_size=4, hop_size=2).shape == (2, 3, 0, 4)


@pytest.mark.parametrize("frame_size,hop,seq_len", [(25, 10, 3600), (27, 13, 3600), (25, 25, 3600), (400, 160, 3600)])
def test_frame_against_index_arithmetic(frame_size, hop, seq_len):
    x = torch.randn(3, seq_len)
    n = fu.num_frames(seq_len, frame_size=frame_size, hop_size=hop)
    padded = torch.nn.functional.pad(x, (0, n * hop + frame_size))
    idx = hop * torch.arange(n)[:, None] + torch.arange(frame_size)[None]
    torch.testing.assert_close(fu.frame(x, frame_size=frame_size, hop_size=hop), padded[:, idx])
    lengths = torch.tensor([seq_len, seq_len // 2, 7])
    paddings = (torch.arange(seq_len)[None] >= lengths[:, None]).long()
    out = fu.frame_paddings(paddings, frame_size=frame_size, hop_size=hop)
    assert out.shape == (3, n)
    # A frame is valid only if it lies wholly inside the sequence.
    want = (idx[None, :, -1] >= lengths[:, None]).long()
    assert out.tolist() == want.tolist()


@pytest.mark.parametrize("hop_size,expected", [(1, [[1, 1, 1, 1, 1, 1]]), (2, [[1, 1, 1, 1]])])
def test_frame_paddings_simple(hop_size, expected):
    paddings = torch.tensor([[1, 1, 1, 1, 0, 0, 0, 0, 1, 1]])
    assert fu.frame_paddings(paddings, frame_size=5, hop_size=hop_size).tolist() == expected
    with pytest.raises(ValueError):
        fu.frame_paddings(paddings, frame_size=2, hop_size=3)


def test_units_windows_and_scales():
    assert fu.ms_to_samples(25, sample_rate=16000) == 400 and fu.ms_to_samples(2.5, sample_rate=16000) == 40
    with pytest.raises(ValueError):
        fu.ms_to_samples(0.01, sample_rate=16000)
    assert fu.next_power_of_2(400) == 512 and fu.next_power_of_2(512) == 512
    hz = np.array([0.0, 125.0, 3800.0, 7600.0])
    mel = fu.hertz_to_warped_scale(hz, freq_scale=fu.FrequencyScale.MEL_LN)
    np.testing.assert_allclose(fu.warped_to_hertz_scale(mel, freq_scale=fu.FrequencyScale.MEL_LN), hz, atol=1e-9)
    np.testing.assert_allclose(mel[1], 1127.0 * np.log(1 + 125 / 700))
    # Periodic windows are what torch calls periodic; symmetric ones what numpy computes.
    for n in (400, 401):
        torch.testing.assert_close(fu.window_coffs(n, window_type=fu.WindowType.HANN).float(),
                                   torch.hann_window(n, periodic=n % 2 == 0), atol=1e-6, rtol=0)
        torch.testing.assert_close(fu.window_coffs(n, window_type=fu.WindowType.HAMMING, periodic=False).float(),
                                   torch.hamming_window(n, periodic=False), atol=1e-6, rtol=0)
    x = torch.randn(2, 7, 400)
    torch.testing.assert_close(fu.windowing(x, window_type=fu.WindowType.HANN), x * torch.hann_window(400), atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(fu.pre_emphasis(x, coeff=0.97), x[..., 1:] - 0.97 * x[..., :-1])


def test_log_mel_pipeline_matches_direct_computation():
    torch.manual_seed(0)
    audio = torch.randn(2, 1600).to(torch.bfloat16)
    frames = fu.windowing(fu.frame(audio.float(), frame_size=400, hop_size=160), window_type=fu.WindowType.HANN)
    spec = fu.magnitude_spectrogram(fu.fft(512)(frames), dtype=torch.float32)
    assert spec.shape == (2, fu.num_frames(1600, frame_size=400, hop_size=160), 257)
    assert fu.cast_for_rfft(audio).dtype == torch.float32 and fu.cast_for_rfft(audio.double()).dtype == torch.float64
    w = fu.linear_to_mel_weight_matrix(num_filters=80, num_spectrogram_bins=257, sample_rate=16000,
                                       lower_edge_hertz=125.0, upper_edge_hertz=7600.0)
    out = fu.linear_to_log_mel_spectrogram(spec, weight_matrix=w, mel_floor=1.0)
    torch.testing.assert_close(out, torch.log(torch.clamp(spec @ w, min=1.0)))
    assert out.min() >= 0.0
    tiny = torch.zeros(3)
    assert torch.isfinite(fu.linear_to_log_spectrogram(tiny)).all()
