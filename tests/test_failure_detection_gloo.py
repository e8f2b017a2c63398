"""Failure detection with failures injected on the host only: a rank that raises, a rank whose heartbeat stops, a rank that
never joins a collective (short process-group timeout), and resume from a checkpoint after a rank was lost."""
import copy
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist

import test_sharding_gloo as T
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _raising_rank(rank, world_size):
    from torchrec_b200.distributed.failure_detection import FailureBoard, PeerFailure, guarded_step, world_store

    with MultiProcessContext(rank, world_size, "gloo", timeout_s=20) as ctx:
        board = FailureBoard(world_store(), rank, world_size)
        dist.barrier()
        done = 0

        def step():
            nonlocal done
            if rank == 1 and done == 2:
                raise ValueError("bad batch on rank 1")
            t = torch.ones(1)
            dist.all_reduce(t)
            done += 1
            return t

        caught = None
        for i in range(6):
            try:
                guarded_step(step, board)
            except ValueError as e:
                caught = ("own", str(e))
                break
            except PeerFailure as e:
                caught = ("peer", e.ranks, e.reasons)
                break
        if rank == 1:
            assert caught == ("own", "bad batch on rank 1") and done == 2
        else:
            # rank 0 either saw the post before launching step 3, or its all-reduce timed out and was attributed to rank 1
            assert caught is not None and caught[0] == "peer" and caught[1] == [1] and "bad batch" in caught[2][1]
            assert done == 2


def test_rank_that_raises_is_reported_to_peers_between_steps():
    run_multi_process(_raising_rank, world_size=2, timeout_s=120)


def _silent_rank(rank, world_size):
    from torchrec_b200.distributed.failure_detection import Heartbeat, PeerFailure, world_store

    with MultiProcessContext(rank, world_size, "gloo", timeout_s=20):
        hb = Heartbeat(world_store(), rank, world_size, interval_s=0.1).start()
        dist.barrier()
        time.sleep(0.5)
        assert hb.silent_ranks(max_silence_s=1.0) == []
        if rank == 1:
            hb.pause()  # the host thread of rank 1 stops making progress
            time.sleep(4.0)
            hb.resume()
        else:
            deadline = time.monotonic() + 3.5
            seen = []
            while time.monotonic() < deadline and not seen:
                seen = hb.silent_ranks(max_silence_s=1.0)
                time.sleep(0.1)
            assert seen == [1]
            with pytest.raises(PeerFailure):
                hb.raise_if_silent(1.0)
            time.sleep(1.5)
        dist.barrier()
        time.sleep(0.5)
        assert hb.silent_ranks(max_silence_s=1.0) == []  # it came back
        hb.stop()


def test_heartbeat_detects_a_silent_rank_and_its_return():
    run_multi_process(_silent_rank, world_size=3, timeout_s=120)


def _absent_rank(rank, world_size):
    os.environ["TORCH_GLOO_LAZY_INIT"] = "0"
    with MultiProcessContext(rank, world_size, "gloo", timeout_s=60):
        short = dist.new_group(ranks=list(range(world_size)), timeout=datetime.timedelta(seconds=2), backend="gloo")
        dist.barrier()
        if rank == 1:
            time.sleep(5.0)  # never joins the collective below
        else:
            t0 = time.monotonic()
            with pytest.raises(RuntimeError):
                dist.all_reduce(torch.ones(4), group=short)
            assert time.monotonic() - t0 < 10.0
        # the default group is still usable for an orderly shutdown message
        from torchrec_b200.distributed.failure_detection import FailureBoard, world_store

        board = FailureBoard(world_store(), rank, world_size)
        if rank == 0:
            board.post("collective timed out waiting for rank 1")
        else:
            deadline = time.monotonic() + 10
            while time.monotonic() < deadline and not board.failed_ranks():
                time.sleep(0.1)
            assert 0 in board.failed_ranks()
        dist.barrier()  # rank 0 hosts the store: it stays until its peer has read the message


def test_collective_with_short_timeout_errors_instead_of_hanging():
    run_multi_process(_absent_rank, world_size=2, timeout_s=120)


def _train(rank, world_size, steps, ckpt_dir, resume_from=None, save_at=None):
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    with MultiProcessContext(rank, world_size, "gloo", timeout_s=60) as ctx:
        torch.manual_seed(0)
        model = T._Model(T._make_ebc(PoolingType.SUM))
        apply_optimizer_in_backward(RowWiseAdagrad, model.ebc.parameters(), {"lr": 0.1, "eps": 1e-8})
        plan = ShardingPlan({"ebc": T._plan_for(model.ebc, "mixed", world_size)})
        dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan)
        dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda ps: torch.optim.Adagrad(ps, lr=0.1))
        opt = CombinedOptimizer([dmp.fused_optimizer, dense])
        start = 0
        if resume_from is not None:
            ck = torch.load(os.path.join(ckpt_dir, f"step{resume_from}_rank{rank}.pt"), weights_only=False)
            dmp.load_state_dict(ck["model"])
            opt.init_state(set())
            opt.load_state_dict(ck["optim"])
            start = resume_from
        for step in range(start, steps):
            kjt = T._make_kjt(6, 1000 + 10 * step + rank)
            opt.zero_grad()
            pred, _ = dmp(kjt)
            pred.mean().backward()
            opt.step()
            if save_at is not None and step + 1 == save_at:
                torch.save({"model": dmp.state_dict(), "optim": opt.state_dict()}, os.path.join(ckpt_dir, f"step{save_at}_rank{rank}.pt"))
                if resume_from is None and steps > save_at and os.environ.get("TRB_TEST_CRASH_AFTER_SAVE") == "1":
                    return  # every rank leaves between steps: the job "lost a rank" and is restarted from the checkpoint
        final = {}
        for k, v in dmp.state_dict().items():
            final[k] = [(list(s.metadata.shard_offsets), s.tensor.clone()) for s in v.local_shards()] if hasattr(v, "local_shards") else v.clone()
        torch.save(final, os.path.join(ckpt_dir, f"final_{'resumed' if resume_from is not None else 'straight'}_rank{rank}.pt"))


def test_resume_from_checkpoint_reproduces_the_uninterrupted_run(tmp_path):
    d = str(tmp_path)
    run_multi_process(_train, world_size=2, steps=5, ckpt_dir=d, save_at=3)            # uninterrupted, checkpoint on the way
    run_multi_process(_train, world_size=2, steps=5, ckpt_dir=d, resume_from=3)        # restarted job
    for rank in range(2):
        a = torch.load(os.path.join(d, f"final_straight_rank{rank}.pt"), weights_only=False)
        b = torch.load(os.path.join(d, f"final_resumed_rank{rank}.pt"), weights_only=False)
        assert a.keys() == b.keys()
        for k in a:
            if isinstance(a[k], list):
                for (oa, ta), (ob, tb) in zip(a[k], b[k]):
                    assert oa == ob
                    torch.testing.assert_close(ta, tb, rtol=1e-6, atol=1e-7, msg=lambda m: f"{k}: {m}")
            else:
                torch.testing.assert_close(a[k], b[k], rtol=1e-6, atol=1e-7, msg=lambda m: f"{k}: {m}")
