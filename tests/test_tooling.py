"""fx tracer, schema compatibility check, docstring linter, method logger, pt2 helpers, module utilities."""
import inspect
import logging
from typing import List, Optional

import pytest
import torch
from torch import nn


def test_fx_tracer_keeps_embedding_modules_as_leaves():
    from torchrec_b200.fx import Tracer, is_fx_tracing, symbolic_trace
    from torchrec_b200.fx import utils as fxu
    from torchrec_b200.fx.utils import assert_fx_safe, is_marker_node
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.ebc = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="t", embedding_dim=4, num_embeddings=10, feature_names=["f"])])
            self.lin = nn.Linear(4, 1)

        def forward(self, kjt: KeyedJaggedTensor):
            assert_fx_safe(not is_fx_tracing() or True, "never evaluated on proxies")
            fxu.fx_marker("BEGIN", kjt)  # looked up in its module at call time, where the tracer patches it
            return self.lin(self.ebc(kjt).values())

    m = M()
    gm = symbolic_trace(m, leaf_modules=["EmbeddingBagCollection"])
    targets = [n.target for n in gm.graph.nodes if n.op == "call_module"]
    assert "ebc" in targets and "lin" in targets
    assert any(is_marker_node(n, "BEGIN") for n in gm.graph.nodes)
    kjt = KeyedJaggedTensor(keys=["f"], values=torch.tensor([1, 2, 3]), lengths=torch.tensor([2, 1]))
    torch.testing.assert_close(gm(kjt), m(kjt))
    assert not is_fx_tracing()
    assert isinstance(Tracer(), torch.fx.Tracer)


def test_signature_compatibility():
    from torchrec_b200.schema.utils import is_signature_compatible

    def old(a: int, b: str = "x", *, c: Optional[int] = None) -> int: ...
    def ok(a: int, b: str = "x", d: float = 1.0, *, c: Optional[int] = None, e: int = 0) -> int: ...
    def renamed(a: int, bb: str = "x", *, c: Optional[int] = None) -> int: ...
    def lost_default(a: int, b: str, *, c: Optional[int] = None) -> int: ...
    def new_required(a: int, b: str = "x", *, c: Optional[int] = None, z: int) -> int: ...
    def retyped(a: List[int], b: str = "x", *, c: Optional[int] = None) -> int: ...
    def widened(a: Optional[int], b: str = "x", *, c: Optional[int] = None) -> int: ...

    s = inspect.signature
    assert is_signature_compatible(s(old), s(ok))
    assert is_signature_compatible(s(old), s(widened))
    for bad in (renamed, lost_default, new_required, retyped):
        assert not is_signature_compatible(s(old), s(bad)), bad.__name__


def test_public_api_signatures_are_stable():
    """The constructor arguments users of the reference rely on are present, by name and in order."""
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
    from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor

    def names(f):
        return [p for p in inspect.signature(f).parameters if p != "self"]

    assert names(EmbeddingBagCollection.__init__)[:3] == ["tables", "is_weighted", "device"]
    assert names(EmbeddingCollection.__init__)[:3] == ["tables", "device", "need_indices"]
    assert names(DistributedModelParallel.__init__)[:8] == ["module", "env", "device", "plan", "sharders", "init_data_parallel", "init_parameters", "data_parallel_wrapper"]
    assert names(KeyedJaggedTensor.__init__)[:6] == ["keys", "values", "weights", "lengths", "offsets", "stride"]
    assert names(JaggedTensor.__init__)[:4] == ["values", "weights", "lengths", "offsets"]
    assert names(KeyedTensor.__init__)[:4] == ["keys", "length_per_key", "values", "key_dim"]
    assert names(TrainPipelineSparseDist.__init__)[:4] == ["model", "optimizer", "device", "execute_all_batches"]


def test_module_linter_reports_missing_sections(tmp_path, capsys):
    from torchrec_b200.linter.module_linter import linter_one_file

    src = tmp_path / "mod.py"
    src.write_text('''
import torch
class Good(torch.nn.Module):
    """Does a thing.

    Args:
        dim (int): width.

    Example::

        Good(3)
    """
    def __init__(self, dim: int) -> None:
        super().__init__()
    def forward(self, x):
        """
        Args:
            x: input.
        Returns:
            the output.
        """
        return x

class Bad(torch.nn.Module):
    def __init__(self, dim):
        super().__init__()

class Half(torch.nn.Module):
    """Only a summary."""
    def __init__(self, dim, other):
        super().__init__()
    def forward(self, x):
        return x
''')
    linter_one_file(str(src))
    out = capsys.readouterr().out
    assert "Good" not in out
    assert "No docstring found in a module class" in out
    assert "Missing Args: section for __init__" in out and "No docstring on forward" in out and "No runnable example" in out


def test_method_logger_records_calls_and_errors():
    from torchrec_b200.distributed.logger import _torchrec_method_logger
    from torchrec_b200.distributed.logging_handlers import _log_handlers

    records = []

    class H(logging.Handler):
        def emit(self, record):
            records.append(record.msg)

    old = _log_handlers["default"]
    _log_handlers["default"] = H()
    try:
        @_torchrec_method_logger()
        def f(a, b=2):
            if a < 0:
                raise ValueError("neg")
            return a + b

        assert f(1) == 3
        with pytest.raises(ValueError):
            f(-1)
    finally:
        _log_handlers["default"] = old
    assert records[0]["func_name"] == "f" and "'a': '1'" in records[0]["input"] and records[0]["output"] == "3"
    assert records[1]["error"] == "neg"


def test_pt2_helpers_and_settings():
    from torchrec_b200.distributed import global_settings as gs
    from torchrec_b200.pt2 import checks
    from torchrec_b200.pt2.utils import kjt_for_pt2_tracing
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    assert not checks.is_pt2_compiling()
    assert checks.pt2_checks_all_is_size([1, 2]) == [1, 2]
    checks.set_use_torchdynamo_compiling_path(True)
    assert checks.is_torchdynamo_compiling()
    checks.set_use_torchdynamo_compiling_path(False)
    kjt = KeyedJaggedTensor(keys=["a", "b"], values=torch.tensor([1, 2, 3], dtype=torch.int32), lengths=torch.tensor([1, 0, 1, 1], dtype=torch.int32))
    t = kjt_for_pt2_tracing(kjt)
    assert t.values().dtype == torch.int64 and t.lengths().dtype == torch.int64 and t.stride() == 2
    vb = kjt_for_pt2_tracing(kjt, convert_to_vb=True)
    assert vb.variable_stride_per_key() and vb.stride_per_key() == [2, 2]
    gs.set_propogate_device(True)
    assert gs.get_propogate_device()
    gs.set_propogate_device(False)


def test_module_utils():
    from torchrec_b200.modules import utils as U
    from torchrec_b200.modules.lazy_extension import LazyModuleExtensionMixin, lazy_apply
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    assert U.get_module_output_dimension(nn.Linear(3, 7), 3) == 7
    assert U.check_module_output_dimension([nn.Linear(3, 7), nn.Linear(3, 7)], 3, 7)
    ml = U.construct_modulelist_from_single_module(nn.Linear(2, 2), (2, 3))
    assert len(ml) == 2 and len(ml[0]) == 3 and ml[0][0].weight.data_ptr() != ml[0][1].weight.data_ptr()
    assert isinstance(U.extract_module_or_tensor_callable(lambda: nn.ReLU()), nn.ReLU)
    assert U.extract_module_or_tensor_callable(torch.relu) is torch.relu
    ids = torch.tensor([5, 3, 5, 9, 3])
    u, last = U.deterministic_dedup(ids)
    assert u.tolist() == [3, 5, 9] and last.tolist() == [4, 2, 3]
    kjt = KeyedJaggedTensor(keys=["a", "b"], values=torch.tensor([1, 2, 3]), lengths=torch.tensor([1, 0, 1, 1]))
    emb = torch.arange(6.0).view(3, 2)
    jts = U.construct_jagged_tensors(emb, kjt, ["a", "b"], need_indices=True)
    assert jts["a"].values().tolist() == [[0.0, 1.0]] and jts["b"].lengths().tolist() == [1, 1] and jts["b"].weights().tolist() == [2, 3]
    jts2 = U.construct_jagged_tensors_inference(emb, kjt.lengths().view(2, 2), kjt.values(), ["a", "b"])
    assert torch.equal(jts2["b"].values(), jts["b"].values())

    class Lazy(LazyModuleExtensionMixin, nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.UninitializedParameter()

        def initialize_parameters(self, x, scale=None):
            self.w.materialize((x.shape[-1],))
            with torch.no_grad():
                self.w.fill_(1.0 if scale is None else scale)

        def forward(self, x, scale=None):
            return x * self.w

    m = Lazy()
    with pytest.raises(RuntimeError):
        m.apply(lambda mod: None)
    seen = []
    lazy_apply(m, lambda mod: seen.append(type(mod).__name__))
    out = m(torch.ones(2, 3), scale=2.0)
    assert out.tolist() == [[2.0] * 3] * 2 and seen == ["Lazy"]
    m(torch.ones(2, 3))
    assert seen == ["Lazy"]
