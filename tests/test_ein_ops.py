import pytest
import torch

from axlearn_b200.common.ein_ops import rearrange, repeat


def test_rearrange_and_repeat_match_einops():
    einops = pytest.importorskip("einops")
    x = torch.randn(2, 6, 12)
    for pattern, kw in [("b t (n h) -> b n t h", dict(n=3)), ("b t d -> (b t) d", {}), ("b t d -> b d t", {}),
                        ("b (t two) d -> b t (two d)", dict(two=2)), ("b t d -> b 1 t d", {})]:
        assert torch.equal(rearrange(x, pattern, **kw), einops.rearrange(x, pattern, **kw)), pattern
    for pattern, kw in [("b t d -> b t k d", dict(k=3)), ("b t d -> b (t r) d", dict(r=2)), ("b t d -> (k b) t d", dict(k=2))]:
        assert torch.equal(repeat(x, pattern, **kw), einops.repeat(x, pattern, **kw)), pattern
    y = torch.randn(4, 1, 5)
    assert torch.equal(rearrange(y, "b 1 d -> b d"), y[:, 0])
    with pytest.raises(ValueError):
        rearrange(x, "b t d -> b t")
    with pytest.raises(ValueError):
        rearrange(x, "b t (n h) -> b n t h")
    with pytest.raises(ValueError):
        repeat(x, "b t d -> b t k d")
