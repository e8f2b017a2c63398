"""Prediction service end to end on the host: factory -> quantized predict module -> gRPC server -> client; packaging round trip."""
import torch

from torchrec_b200.inference import predictor_pb as pb
from torchrec_b200.inference.client import PredictorClient, create_request
from torchrec_b200.inference.dlrm_predict import DLRMModelConfig, DLRMPredictFactory
from torchrec_b200.inference.server import PredictorServicer, decode_request, serve
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _config():
    return DLRMModelConfig(dense_arch_layer_sizes=[16, 8], dense_in_features=4, embedding_dim=8, id_list_features_keys=["a", "b", "c"],
                           num_embeddings_per_feature=[50, 60, 70], over_arch_layer_sizes=[16, 1])


def _inputs(B=5, seed=0):
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(0, 4, (3 * B,), generator=g)
    kjt = KeyedJaggedTensor(keys=["a", "b", "c"], values=torch.randint(0, 50, (int(lengths.sum()),), generator=g), lengths=lengths)
    return torch.rand(B, 4, generator=g), kjt


def test_request_wire_format_round_trip():
    dense, kjt = _inputs()
    req = create_request(dense, kjt)
    again = pb.PredictionRequest.FromString(req.SerializeToString())
    t = decode_request(again)
    assert again.batch_size == 5 and again.id_list_features.num_features == 3
    torch.testing.assert_close(t["float_features"], dense)
    assert torch.equal(t["id_list_features.lengths"], kjt.lengths().int()) and torch.equal(t["id_list_features.values"], kjt.values().int())
    resp = pb.PredictionResponse()
    resp.predictions["default"].data.extend([0.5, 0.25])
    assert list(pb.PredictionResponse.FromString(resp.SerializeToString()).predictions["default"].data) == [0.5, 0.25]


def test_grpc_predict_matches_direct_call():
    torch.manual_seed(0)
    factory = DLRMPredictFactory(_config(), quantize=True, device="cpu")
    module = factory.create_predict_module()
    assert "quant" in type(module.predict_module.sparse_arch.embedding_bag_collection).__module__
    servicer = PredictorServicer(module, torch.device("cpu"), id_list_feature_names=factory.model_inputs_data()["id_list_features"])
    server = serve(servicer, "127.0.0.1:0")
    try:
        client = PredictorClient(f"127.0.0.1:{server.bound_port}")
        for seed in range(3):
            dense, kjt = _inputs(B=4 + seed, seed=seed)
            got = client.predict(create_request(dense, kjt))["default"]
            with torch.no_grad():
                want = module({"float_features": dense, "id_list_features": kjt})["default"]
            torch.testing.assert_close(got, want.float(), rtol=1e-5, atol=1e-6)
            assert ((got > 0) & (got < 1)).all()
        client.close()
    finally:
        server.stop(0)
    assert factory.result_metadata() == "dict_of_tensor" and "float_features" in factory.batching_metadata_json()


def test_package_and_load_predict_factory(tmp_path):
    from torchrec_b200.inference.dlrm_packager import main
    from torchrec_b200.inference.model_packager import load_predict_factory

    out = tmp_path / "dlrm.pt"
    main(["--output_path", str(out)])
    factory = load_predict_factory(str(out))
    assert type(factory).__name__ == "DLRMPredictFactory"
    assert factory.model_config.dense_in_features == 13
