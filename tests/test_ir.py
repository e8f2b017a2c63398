"""Export round trip: encapsulate -> ``torch.export`` -> unflatten -> decapsulate gives back working embedding modules."""
import copy

import torch
from torch import nn

from torchrec_b200.ir.serializer import JsonSerializer
from torchrec_b200.ir.utils import decapsulate_ir_modules, encapsulate_ir_modules, mark_dynamic_kjt
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.feature_processor_ import PositionWeightedModuleCollection
from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection
from torchrec_b200.modules.regroup import KTRegroupAsDict
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class _Model(nn.Module):
    def __init__(self):
        super().__init__()
        t1 = EmbeddingBagConfig(name="t1", embedding_dim=8, num_embeddings=20, feature_names=["f1"])
        t2 = EmbeddingBagConfig(name="t2", embedding_dim=4, num_embeddings=30, feature_names=["f2", "f3"])
        self.ebc = EmbeddingBagCollection(tables=[t1, t2])
        self.fpebc = FeatureProcessedEmbeddingBagCollection(
            EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="t3", embedding_dim=4, num_embeddings=10, feature_names=["f1"])], is_weighted=True),
            PositionWeightedModuleCollection({"f1": 6}))
        self.regroup = KTRegroupAsDict(groups=[["f1", "f3"], ["f2"]], keys=["a", "b"])
        self.lin = nn.Linear(12 + 4 + 4, 1)

    def forward(self, kjt: KeyedJaggedTensor):
        kt = self.ebc(kjt)
        fp = self.fpebc(KeyedJaggedTensor(keys=["f1"], values=kjt["f1"].values(), lengths=kjt["f1"].lengths()))
        d = self.regroup([kt])
        return self.lin(torch.cat([d["a"], d["b"], fp.values()], dim=1))


def _kjt():
    return KeyedJaggedTensor(keys=["f1", "f2", "f3"], values=torch.tensor([1, 2, 3, 4, 5, 6, 7, 8, 9]), lengths=torch.tensor([2, 1, 0, 3, 1, 2]))


def test_encapsulate_records_metadata_and_swaps_forward():
    m = _Model()
    m2, fqns = encapsulate_ir_modules(copy.deepcopy(m), JsonSerializer)
    assert set(fqns) == {"ebc", "fpebc", "fpebc._feature_processors", "fpebc._embedding_bag_collection", "regroup"}
    out = m2(_kjt())  # opaque ops produce tensors of the right shape
    assert out.shape == (2, 1)
    back = decapsulate_ir_modules(m2, JsonSerializer)
    assert isinstance(back.ebc, EmbeddingBagCollection) and isinstance(back.regroup, KTRegroupAsDict)
    assert [c.name for c in back.ebc.embedding_bag_configs()] == ["t1", "t2"]
    assert isinstance(back.fpebc, FeatureProcessedEmbeddingBagCollection)


def test_export_round_trip_matches_eager():
    torch.manual_seed(0)
    m = _Model()
    kjt = _kjt()
    ref = m(kjt)
    enc, fqns = encapsulate_ir_modules(copy.deepcopy(m), JsonSerializer)
    shapes = mark_dynamic_kjt(kjt)
    ep = torch.export.export(enc, (kjt,), {}, dynamic_shapes=shapes, strict=False, preserve_module_call_signature=tuple(fqns))
    assert any("trb200_ir.emb_lookup" in str(n.target) for n in ep.graph.nodes)
    un = torch.export.unflatten(ep)
    dec = decapsulate_ir_modules(un, JsonSerializer)
    dec.load_state_dict(m.state_dict(), strict=False)
    torch.testing.assert_close(dec(kjt), ref)
    # another batch with a different number of ids
    kjt2 = KeyedJaggedTensor(keys=["f1", "f2", "f3"], values=torch.arange(1, 8), lengths=torch.tensor([1, 1, 2, 1, 1, 1]))
    torch.testing.assert_close(dec(kjt2), m(kjt2))


def test_copy_nodes_of_a_graph_module_are_pointed_at_the_serving_device():
    import torch.fx

    from torchrec_b200.ir import utils as ir_utils

    graph = torch.fx.Graph()
    x = graph.placeholder("x")
    copy = graph.call_function(torch.ops.aten._to_copy.default, (x,), {"dtype": torch.float64, "device": torch.device("cpu")})
    copy.name = "_to_copy"
    other = graph.call_function(torch.add, (copy, 1))
    graph.output(other)
    gm = torch.fx.GraphModule(torch.nn.Module(), graph)
    ir_utils.move_to_copy_nodes_to_device(gm, torch.device("meta"))
    node = next(n for n in gm.graph.nodes if n.name == "_to_copy")
    assert node.kwargs == {"dtype": torch.float64, "device": torch.device("meta")}
    gm.recompile()
    assert gm(torch.ones(2)).device.type == "meta"
    # the eager bodies and the shape-only bodies of the export placeholders are reachable by name
    out = ir_utils.ir_emb_lookup_impl([torch.ones(1)], 4, [3, 5])
    assert [tuple(t.shape) for t in out] == [(4, 3), (4, 5)]
    assert callable(ir_utils.ir_emb_lookup_fake) and callable(ir_utils.ir_kt_regroup_fake) and callable(ir_utils.ir_dynamic_batch_emb_lookup_fake)
