"""dmoe.HostPipeline: results come back in order and equal the unpipelined step, with the host
buffers of consecutive batches reused in turn."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_sequential_steps():
    from stk_b200 import dmoe
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 64, generator=g).to(dev)

    def step(x, scale):
        return (x @ w) * scale.float()

    batches = [(torch.randn(512, 256, generator=g).pin_memory(),
                torch.full((1,), i + 1, dtype=torch.int32).pin_memory()) for i in range(7)]
    expected = [step(x.to(dev), s.to(dev)).cpu() for x, s in batches]
    pipe = dmoe.HostPipeline(step, dev)
    got = []
    for batch in batches:
        done = pipe.submit(*batch)
        if done is not None:
            pipe.wait(done)
            got.append(done.clone())
    got.append(pipe.flush().clone())
    assert len(got) == len(expected)
    for i, (a, b) in enumerate(zip(got, expected)):
        assert torch.equal(a, b), f"batch {i}"
    assert pipe.flush() is None


def test_read_back_by_kernel():
    from stk_b200 import dmoe
    for shape, dtype in [((8,), torch.int64), ((2, 5), torch.int32), ((3,), torch.int16), ((0,), torch.int64)]:
        t = torch.arange(int(torch.tensor(shape).prod()) if shape != (0,) else 0, device="cuda").to(dtype).view(shape)
        got = dmoe.read_back(t)
        assert not got.is_cuda and got.dtype == dtype and torch.equal(got, t.cpu())
