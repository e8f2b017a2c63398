"""Inference fixtures: quantized test model, device placement, weight specs, plain-tensor wrappers."""
import torch


def test_quantized_sharded_model_matches_quantized_model():
    from torchrec_b200.distributed.quant_state import sharded_tbes_weights_spec
    from torchrec_b200.distributed.test_utils.infer_utils import (
        KJTInputWrapper, TorchTypesModelInputWrapper, assert_close, assert_weight_spec, create_test_model, model_input_to_forward_args,
        model_input_to_forward_args_kjt, prep_inputs, shard_qebc,
    )

    cpu = torch.device("cpu")
    mi = create_test_model(num_embeddings=64, emb_dim=16, world_size=2, batch_size=4, dense_device=cpu, sparse_device=cpu, num_features=3,
                           num_weighted_features=1, quant_state_dict_split_scale_bias=True)
    sharded = shard_qebc(mi, "table_wise", cpu, world_size=2)
    inputs = prep_inputs(mi, world_size=1, batch_size=4, count=3)
    for x in inputs:
        with torch.no_grad():
            assert_close(mi.quant_model(x), sharded(x))
    # quantization error against the float model stays small
    with torch.no_grad():
        torch.testing.assert_close(mi.quant_model(inputs[0]), mi.model(inputs[0]), rtol=0.05, atol=0.02)

    spec = sharded_tbes_weights_spec(sharded)
    assert_weight_spec(spec, [[((0, 0, 64, 16), "rank:0/cpu")], [((0, 0, 64, 16), "rank:1/cpu")], [((0, 0, 64, 16), "rank:0/cpu")]],
                       "sparse.ebc", "embedding_bags", ["table_0", "table_1", "table_2"], "table_wise")

    wrapped = TorchTypesModelInputWrapper(mi.quant_model)
    with torch.no_grad():
        assert_close(mi.quant_model(inputs[1]), wrapped(*model_input_to_forward_args(inputs[1])))
        kjt_out = KJTInputWrapper(mi.quant_model.sparse.ebc)(*model_input_to_forward_args_kjt(inputs[1]))
        assert_close(mi.quant_model.sparse.ebc(inputs[1].idlist_features), kjt_out)
