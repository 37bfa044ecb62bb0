import pytest
import torch

from axlearn_b200.common.gradient_accumulation import split_batch, with_minibatch_steps


def test_accumulated_gradients_equal_full_batch_gradients():
    torch.manual_seed(0)
    w = torch.randn(5, 3, requires_grad=True)
    batch = {"x": torch.randn(8, 5), "y": torch.randn(8, 3), "scale": torch.tensor(2.0)}

    def loss_fn(b):
        err = (b["x"] @ w - b["y"]) * b["scale"]
        return err.pow(2).mean(), {"abs": err.abs().mean(), "per_row": err.abs().mean(-1)}

    loss, _ = loss_fn(batch)
    loss.backward()
    want, w.grad = w.grad.clone(), None
    acc_loss, aux = with_minibatch_steps(loss_fn, steps=4)(batch)
    torch.testing.assert_close(w.grad, want)
    torch.testing.assert_close(acc_loss, loss.detach())
    assert set(aux) == {"abs"}
    assert len(split_batch(batch, 2)) == 2 and split_batch(batch, 2)[1]["x"].shape == (4, 5)
    with pytest.raises(ValueError):
        split_batch(batch, 3)
