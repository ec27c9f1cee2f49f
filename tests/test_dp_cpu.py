"""World-size-2 gloo test of the bucketed gradient averager (host logic of the data-parallel path)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from sparseattention_b200.dp import BucketedGradAverager
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 8))
    avg = BucketedGradAverager(model.parameters(), bucket_bytes=1024)      # several small buckets
    assert len(avg.buckets) >= 2
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    gen = torch.Generator().manual_seed(100 + rank)
    for step in range(3):
        x = torch.randn(4, 16, generator=gen)
        avg.zero_grad()
        model(x).pow(2).mean().backward()
        avg.finish()
        opt.step()
    flat = torch.cat([p.detach().flatten() for p in model.parameters()])
    gflat = torch.cat([p.grad.flatten() for p in model.parameters()])
    out[rank] = (flat, gflat)
    dist.destroy_process_group()


def _reference(world):
    """Same training on one process with the mean of the per-rank gradients."""
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 8))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    gens = [torch.Generator().manual_seed(100 + r) for r in range(world)]
    for step in range(3):
        grads = None
        for r in range(world):
            x = torch.randn(4, 16, generator=gens[r])
            model.zero_grad()
            model(x).pow(2).mean().backward()
            g = [p.grad.clone() for p in model.parameters()]
            grads = g if grads is None else [a + b for a, b in zip(grads, g)]
        for p, g in zip(model.parameters(), grads):
            p.grad = g / world
        opt.step()
    return (torch.cat([p.detach().flatten() for p in model.parameters()]),
            torch.cat([p.grad.flatten() for p in model.parameters()]))


def test_bucketed_grad_average_gloo_world2():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    want_p, want_g = _reference(world)
    for r in range(world):
        got_p, got_g = out[r]
        assert torch.allclose(got_p, want_p, atol=1e-6), r
        assert torch.allclose(got_g, want_g, atol=1e-6), r


class _Tied(nn.Module):
    """A parameter used twice in one forward (as the LM's embedding / head matrix is)."""

    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(12, 8)
        self.mid = nn.Linear(8, 8)

    def forward(self, ids):
        return self.mid(self.emb(ids)) @ self.emb.weight.t()


def _tied_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from sparseattention_b200.dp import BucketedGradAverager
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(1)
    model = _Tied()
    avg = BucketedGradAverager(model.parameters(), bucket_bytes=128)
    gen = torch.Generator().manual_seed(7 + rank)
    for step in range(2):
        ids = torch.randint(0, 12, (5,), generator=gen)
        avg.zero_grad()
        model(ids).pow(2).mean().backward()
        avg.finish()
    out[rank] = torch.cat([p.grad.flatten() for p in model.parameters()])
    dist.destroy_process_group()


def test_bucketed_grad_average_with_a_tied_parameter():
    world = 2
    port = 31500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_tied_worker, args=(world, port, out), nprocs=world, join=True)
    torch.manual_seed(1)
    model = _Tied()
    gens = [torch.Generator().manual_seed(7 + r) for r in range(world)]
    want = None
    for step in range(2):
        want = None
        for r in range(world):
            ids = torch.randint(0, 12, (5,), generator=gens[r])
            model.zero_grad()
            model(ids).pow(2).mean().backward()
            g = torch.cat([p.grad.flatten() for p in model.parameters()])
            want = g if want is None else want + g
        want = want / world
    for r in range(world):
        assert torch.allclose(out[r], want, atol=1e-6), r


def test_zipf_tokens_shape_and_skew():
    sys.path.insert(0, ROOT)
    from sparseattention_b200.lm import zipf_tokens
    t = zipf_tokens(4, 1000, 50257, seed=1)
    assert t.shape == (4, 1000) and int(t.min()) >= 0 and int(t.max()) < 50257
    # rank 1 (id 0) is the most frequent token by a wide margin under s = 1.1
    counts = torch.bincount(t.flatten(), minlength=10)
    assert counts[0] > counts[1] > counts[4]
    assert torch.equal(t, zipf_tokens(4, 1000, 50257, seed=1))
