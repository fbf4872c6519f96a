"""PinnedFeed: batches arrive intact and in order while kernels of the previous step are still running."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_batches_arrive_in_order_and_intact(cuda):
    from graphcuda_b200 import PinnedFeed
    n = 1 << 20
    host = [(torch.full((n,), float(k)).pin_memory(), torch.full((17,), k, dtype=torch.int64).pin_memory())
            for k in range(6)]
    feed = PinnedFeed(cuda, like=list(host[0]))
    sums = []
    feed.submit(host[0])
    for k in range(6):
        x, y = feed.take()
        if k + 1 < 6:
            feed.submit(host[k + 1])
        # a long-running consumer: the next copy must not overwrite this slot before release()
        acc = x.clone()
        for _ in range(20):
            acc = acc * 1.0 + 0.0
        sums.append((acc.sum(), y.sum()))
        feed.release()
    torch.cuda.synchronize()
    assert [float(a) for a, _ in sums] == [float(k) * n for k in range(6)]
    assert [int(b) for _, b in sums] == [17 * k for k in range(6)]


def test_misuse_is_reported(cuda):
    from graphcuda_b200 import PinnedFeed
    h = torch.zeros(8).pin_memory()
    feed = PinnedFeed(cuda, like=[h])
    with pytest.raises(RuntimeError):
        feed.take()
    feed.submit([h])
    feed.submit([h])
    with pytest.raises(RuntimeError):
        feed.submit([h])  # both slots busy
    feed.take()
    with pytest.raises(ValueError):
        feed.release() or feed.submit([torch.zeros(9).pin_memory()])
    with pytest.raises(ValueError):
        PinnedFeed(cuda, like=[h], depth=1)
