"""Quantised embedding collectives on two gloo ranks: the byte containers (FP8, INT8, MX4) change the size of what travels, so the
split sizes of the all-to-all must follow the encoded chunks.  Values and gradients are compared with the unquantised
collective within the format's precision (cf. ``torchrec/distributed/tests/test_comm.py``)."""
import pytest
import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

_TOL = {"fp16": 2e-3, "int8": 0.03, "fp8": 0.15, "mx4": 0.6}


def _codecs(name):
    from torchrec_b200.distributed.fbgemm_qcomm_codec import CommType, QCommsConfig, get_qcomm_codecs

    ct = CommType(name)
    return get_qcomm_codecs(QCommsConfig(forward_precision=ct, backward_precision=ct))


def _pooled(rank, world_size, name):
    from torchrec_b200.distributed import comm_ops

    with MultiProcessContext(rank, world_size, "gloo", timeout_s=60) as ctx:
        torch.manual_seed(10 + rank)
        batch = [3, 5]          # uneven batch per rank
        dims = [48, 80]         # 48 is not a multiple of the MX4 block: chunks are padded per destination
        x = torch.randn(sum(batch), dims[rank], requires_grad=True)
        xq = x.detach().clone().requires_grad_(True)
        want = comm_ops.alltoall_pooled(x, batch, dims, group=ctx.pg).wait()
        got = comm_ops.alltoall_pooled(xq, batch, dims, group=ctx.pg, codecs=_codecs(name)).wait()
        assert got.shape == want.shape == (batch[rank], sum(dims))
        torch.testing.assert_close(got, want.detach(), rtol=0, atol=_TOL[name] * float(want.abs().max()))
        g = torch.randn_like(want)
        want.backward(g)
        got.backward(g)
        torch.testing.assert_close(xq.grad, x.grad, rtol=0, atol=_TOL[name] * float(x.grad.abs().max()) + 1e-6)


def _sequence(rank, world_size, name):
    from torchrec_b200.distributed import comm_ops

    with MultiProcessContext(rank, world_size, "gloo", timeout_s=60) as ctx:
        torch.manual_seed(20 + rank)
        D = 40
        # rank r looked up rows for ids it received: in_rows[r][s] rows go back to source s
        rows_back = [[2, 4], [3, 1]]
        sends = rows_back[rank]
        recvs = [rows_back[s][rank] for s in range(world_size)]
        x = torch.randn(sum(sends), D, requires_grad=True)
        xq = x.detach().clone().requires_grad_(True)
        lengths = torch.tensor(sends)

        def run(t, codecs):
            return comm_ops.alltoall_sequence(t, None, None, lengths, input_splits=recvs, output_splits=sends, group=ctx.pg, codecs=codecs).wait()

        want, got = run(x, None), run(xq, _codecs(name))
        assert got.shape == want.shape == (sum(recvs), D)
        torch.testing.assert_close(got, want.detach(), rtol=0, atol=_TOL[name] * float(want.abs().max()))
        g = torch.randn_like(want)
        want.backward(g)
        got.backward(g)
        torch.testing.assert_close(xq.grad, x.grad, rtol=0, atol=_TOL[name] * float(x.grad.abs().max()) + 1e-6)


@pytest.mark.parametrize("name", ["fp16", "int8", "fp8", "mx4"])
def test_pooled_all_to_all_with_codecs(name):
    run_multi_process(_pooled, world_size=2, name=name)


@pytest.mark.parametrize("name", ["int8", "mx4"])
def test_sequence_all_to_all_with_codecs(name):
    run_multi_process(_sequence, world_size=2, name=name)


def test_mx4_container_size_and_values():
    from torchrec_b200.distributed.fbgemm_qcomm_codec import Mx4Codec

    codec = Mx4Codec(32)
    x = torch.tensor([0.0, 0.5, -1.0, 1.5, 2.0, -3.0, 4.0, 6.0] * 4 + [100.0] + [0.0] * 31)
    ctx = codec.create_context()
    q = codec.encode(x, ctx)
    assert q.numel() == 2 * 17 == codec.calc_quantized_size(x.numel())  # 4.25 bits per value
    # every representable magnitude at block exponent 0 survives exactly; a block is scaled by a power of two
    torch.testing.assert_close(codec.decode(q, ctx)[:32], x[:32], rtol=0, atol=0)
    assert abs(float(codec.decode(q, ctx)[32]) - 96.0) < 1e-6  # 100 -> 6 * 2^4


def _functional_forms(rank, world_size):
    from torchrec_b200.distributed import comm_ops as co

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        x = (torch.arange(8, dtype=torch.float32).view(4, 2) + 10 * rank).requires_grad_(True)
        gathered = co.all_gather_into_tensor(x, 0, ctx.pg)
        assert gathered.shape == (8, 2) and torch.equal(gathered[4 * rank: 4 * rank + 4].detach(), x.detach())
        gathered.sum().backward()
        assert torch.equal(x.grad, torch.full((4, 2), float(world_size)))  # the gradient comes back through a reduce-scatter
        y = torch.ones(4, 3, requires_grad=True)
        scattered = co.reduce_scatter_tensor(y, 0, ctx.pg)
        assert torch.equal(scattered.detach(), torch.full((2, 3), float(world_size)))
        scattered.sum().backward()
        assert torch.equal(y.grad, torch.ones(4, 3))
        pooled = co.all2all_pooled_sync(ctx.pg, co.All2AllPooledInfo([2, 2], [3, 3], None, None), torch.full((4, 3), float(rank + 1)))
        assert pooled.shape == (2, 6) and torch.equal(pooled[:, :3], torch.ones(2, 3)) and torch.equal(pooled[:, 3:], torch.full((2, 3), 2.0))
        flat = torch.arange(10, dtype=torch.float32)  # rank 0 keeps feature batches (1, 2) x dims (2, 1) = 4 values, rank 1 gets (2, 2) = 6
        part = co.reduce_scatter_v_per_feature_pooled(flat, [[1, 2], [2, 2]], [2, 1], ctx.pg).wait()
        want = flat[:4] * world_size if rank == 0 else flat[4:] * world_size
        assert torch.equal(part, want)
        # dense rows grouped by destination: rank r sends r + 1 rows to rank 0 and 2 rows to rank 1
        from torchrec_b200.distributed.dist_data import TensorAllToAll, TensorValuesAllToAll

        rows = torch.arange((rank + 3) * 2, dtype=torch.float32).view(rank + 3, 2) + 100 * rank
        got = TensorAllToAll(ctx.pg)(rows, torch.tensor([rank + 1, 2])).wait().wait()
        from_0 = torch.arange(6, dtype=torch.float32).view(3, 2)
        from_1 = torch.arange(8, dtype=torch.float32).view(4, 2) + 100
        want = torch.cat([from_0[:1], from_1[:2]]) if rank == 0 else torch.cat([from_0[1:], from_1[2:]])
        assert torch.equal(got, want)
        direct = TensorValuesAllToAll(ctx.pg)(rows, [rank + 1, 2], [1, 2] if rank == 0 else [2, 2]).wait()
        assert torch.equal(direct, want)


def test_blocking_and_functional_collective_forms():
    run_multi_process(_functional_forms, world_size=2)
