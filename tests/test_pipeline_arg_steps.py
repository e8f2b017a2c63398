"""Explicit argument steps of the train pipelines, the forward that runs the lookup ahead of time, and the small pipeline helpers
(cf. ``torchrec/distributed/train_pipeline/tests/test_tracing.py``, ``test_train_pipelines_base.py``)."""
from dataclasses import dataclass

import pytest
import torch

from torchrec_b200.distributed.train_pipeline.postproc import NoOpStream
from torchrec_b200.distributed.train_pipeline.tracing import (
    ArgInfo,
    ArgInfoStepFactory,
    CallArgs,
    GetAttrArgInfoStep,
    GetItemArgInfoStep,
    NoopArgInfoStep,
    ScalarArgInfoStep,
)
from torchrec_b200.distributed.train_pipeline.train_pipelines import TorchCompileConfig, TrainPipelinePT2
from torchrec_b200.distributed.train_pipeline.utils import get_h2d_func
from torchrec_b200.streamable import Pipelineable


@dataclass
class _Batch(Pipelineable):
    ids: dict
    dense: torch.Tensor

    def to(self, device, non_blocking=False):
        return _Batch({k: v.to(device) for k, v in self.ids.items()}, self.dense.to(device))

    def record_stream(self, stream):
        pass


def test_steps_compose_and_compare():
    batch = _Batch({"a": torch.arange(4), "b": torch.arange(2)}, torch.ones(2, 3))
    f = ArgInfoStepFactory
    double = torch.nn.Identity()
    info = ArgInfo(steps=[f.get_attr("ids"), f.get_item("a")])
    assert torch.equal(info.process_steps(batch), torch.arange(4)) and torch.equal(info.resolve(batch), torch.arange(4))
    assert ArgInfo(steps=[]).process_steps(batch) is None
    nested = ArgInfo(steps=[f.from_dict({"x": ArgInfo(steps=[f.get_attr("dense")]), "y": ArgInfo(steps=[f.from_scalar(3)]),
                                         "z": ArgInfo(steps=[f.from_list([ArgInfo(steps=[f.noop()]), 7])])})])
    out = nested.process_steps(batch)
    assert out["x"] is batch.dense and out["y"] == 3 and out["z"][0] is batch and out["z"][1] == 7
    via_module = ArgInfo(steps=[f.get_attr("dense"), f.postproc(double)])
    assert via_module.process_steps(batch) is batch.dense
    # add_step puts a step in front, append_step behind
    built = ArgInfo(steps=[f.get_item("b")]).add_step(f.get_attr("ids")).append_step(f.noop())
    assert [type(s) for s in built.steps] == [GetAttrArgInfoStep, GetItemArgInfoStep, NoopArgInfoStep]
    assert torch.equal(built.process_steps(batch), torch.arange(2))
    assert GetAttrArgInfoStep("ids") == GetAttrArgInfoStep("ids") and GetAttrArgInfoStep("ids") != GetAttrArgInfoStep("dense")
    assert GetItemArgInfoStep(0) != ScalarArgInfoStep(0)
    call = CallArgs(args=[info], kwargs={"k": ArgInfo(steps=[f.from_scalar("v")]), "old": ArgInfo(["dense"], [False])})
    args, kwargs = call.build_args_kwargs(batch)
    assert torch.equal(args[0], torch.arange(4)) and kwargs["k"] == "v" and kwargs["old"] is batch.dense


def test_lookup_ahead_forward_needs_its_stage_first():
    from torchrec_b200.distributed.train_pipeline.pipeline_context import PrefetchTrainPipelineContext
    from torchrec_b200.distributed.train_pipeline.runtime_forwards import PrefetchEmbeddingPipelinedForward

    class _Ctx:
        def record_stream(self, stream):
            pass

    class _Mod(torch.nn.Module):
        def compute_and_output_dist(self, ctx, data):
            return ("awaitable", data)

        def forward(self, x):
            raise AssertionError("the original forward must not run")

    context = PrefetchTrainPipelineContext()
    fwd = PrefetchEmbeddingPipelinedForward("m", CallArgs(), _Mod(), context, None)
    with pytest.raises(Exception, match="compute_and_output_dist must be called"):
        fwd(None)
    with pytest.raises(AssertionError):
        fwd.compute_and_output_dist()
    context.module_input_post_prefetch["m"] = "prefetched"
    context.module_contexts_post_prefetch["m"] = _Ctx()
    fwd.compute_and_output_dist()
    assert fwd(None) == ("awaitable", "prefetched")
    with pytest.raises(Exception):
        fwd(None)  # one awaitable per stage run


def test_small_helpers_and_hooks_run_at_the_configured_iteration():
    with NoOpStream(None) as s:
        assert isinstance(s, NoOpStream)
    moved = get_h2d_func(_Batch({"a": torch.arange(3)}, torch.zeros(1)), torch.device("cpu"))
    assert torch.equal(moved.ids["a"], torch.arange(3))
    cfg = TorchCompileConfig()
    assert (cfg.fullgraph, cfg.dynamic, cfg.backend, cfg.compile_on_iter) == (False, None, "inductor", 3)

    class _M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(3, 1)

        def forward(self, batch):
            loss = self.lin(batch.dense).sum()
            return loss, loss.detach()

    model = _M()
    seen = []
    pipe = TrainPipelinePT2(model, torch.optim.SGD(model.parameters(), lr=0.1), torch.device("cpu"), compile_configs=TorchCompileConfig(compile_on_iter=1),
                            pre_compile_fn=lambda m: seen.append(("pre", pipe._iter)), post_compile_fn=lambda m: seen.append(("post", pipe._iter)))
    data = iter([_Batch({}, torch.ones(2, 3)) for _ in range(3)])
    for _ in range(3):
        pipe.progress(data)
    assert seen == [("pre", 1), ("post", 1)]
