"""One-launch dense optimizer and the peer-memory gradient all-reduce against plain fp32 torch."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["adagrad", "sgd", "adam"])
def test_fused_dense_optimizer_matches_torch(kind):
    from torchrec_b200.optim.fused_dense import FusedDenseOptimizer

    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(13, 512), torch.nn.Linear(512, 257), torch.nn.Linear(257, 1)).cuda()
    ref = copy.deepcopy(m)
    opt = FusedDenseOptimizer(m.parameters(), kind, lr=0.05, eps=1e-8 if kind == "adam" else 1e-10)
    ropt = {"adagrad": lambda p: torch.optim.Adagrad(p, lr=0.05), "sgd": lambda p: torch.optim.SGD(p, lr=0.05),
            "adam": lambda p: torch.optim.Adam(p, lr=0.05)}[kind](ref.parameters())
    for _ in range(3):
        x = torch.randn(64, 13, device="cuda")
        opt.zero_grad()
        ropt.zero_grad()
        m(x).square().mean().backward()
        ref(x).square().mean().backward()
        opt.step()
        ropt.step()
    b = opt.buffer
    for i, (p, q) in enumerate(zip(m.parameters(), ref.parameters())):
        torch.testing.assert_close(p, q, rtol=1e-3, atol=1e-4 if kind == "adam" else 2e-5)  # the kernel is built with fast-math square roots and divisions
        torch.testing.assert_close(b.w16_view(i).float(), q.detach(), rtol=1e-2, atol=1e-2)
        if p.dim() == 2:
            torch.testing.assert_close(b.wT16_view(i).float(), q.detach().t(), rtol=1e-2, atol=1e-2)
    assert all(p.grad.data_ptr() == b.grad.data_ptr() + 4 * off for p, off in zip(b.params, b.offsets))


@pytest.mark.parametrize("world,n", [(2, 1000), (4, 1_000_003), (8, 4096)])
def test_peer_allreduce_virtual_ranks(world, n):
    """Virtual ranks on one GPU: every rank signals first, then the reduce kernels run one after the other (none waits)."""
    from torchrec_b200.distributed.peer_memory import EmulatedPeerGroup

    dev = torch.device("cuda:0")
    emu = EmulatedPeerGroup(world, dev)
    npad = (n + 63) // 64 * 64
    views = [emu.view(r) for r in range(world)]
    bufs = [v.alloc_shared((npad,), torch.float32) for v in views]
    flags = [v.new_flags(2) for v in views]
    counters = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
    torch.manual_seed(1)
    for step in range(2):
        data = [torch.randn(npad, device=dev) for _ in range(world)]
        for (local, _), d in zip(bufs, data):
            local.copy_(d)
        want = torch.stack(data).sum(0) / world
        for f in flags:
            f.signal(0)
        for r, v in enumerate(views):
            torch.ops.trb200.peer_allreduce(bufs[r][1], npad, 1.0 / world, flags[r].ptrs, r, 0, 1, flags[r].epochs, counters[r], False, v.wait_cycles, v.err)
        for f in flags:
            f.wait(1)
        torch.cuda.synchronize()
        for r, v in enumerate(views):
            v.check_error()
            torch.testing.assert_close(bufs[r][0], want, rtol=1e-5, atol=1e-6)
