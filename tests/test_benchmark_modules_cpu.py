"""CPU smoke runs of the module / operator benchmarks (tiny shapes)."""
import torch


def test_benchmark_inference_forms():
    from torchrec_b200.distributed.benchmark.benchmark_inference import main

    res = main(["--module", "both", "--forms", "float,quant,quant_sharded", "--world_size", "2", "--row_cap", "500", "--num_tables", "3",
                "--batch_size", "8", "--iters", "2", "--warmup", "1", "--device", "cpu"])
    assert [r.short_name for r in res] == ["ebc-float", "ebc-quant", "ebc-quant_sharded", "ec-float", "ec-quant", "ec-quant_sharded"]
    assert all(r.gpu_elapsed_time.numel() == 2 for r in res)


def test_benchmark_tbe_operator_and_wrappers():
    from torchrec_b200.distributed.benchmark.benchmark_split_table_batched_embeddings import TBEBenchConfig, op_bench
    from torchrec_b200.distributed.benchmark.embedding_collection_wrappers import ModuleForm, benchmark_ebc_module, get_tables

    res = op_bench(TBEBenchConfig(num_tables=2, num_embeddings=200, embedding_dim=8, batch_size=16, pooling=2, num_iters=2, warmup_iters=1, device="cpu"))
    assert res.gpu_elapsed_time.numel() == 2
    res = op_bench(TBEBenchConfig(num_tables=2, num_embeddings=200, embedding_dim=8, batch_size=16, pooling=2, train=False, num_iters=2, warmup_iters=1, device="cpu"))
    assert "fwd" in res.short_name
    tables = get_tables([(100, 8), (50, 8)], is_pooled=True)
    r = benchmark_ebc_module(tables, ModuleForm.FLOAT, batch_size=8, pooling=2, num_iters=2, warmup_iters=1, device=torch.device("cpu"), train=True)
    assert r.short_name == "ebc-float-train"


def test_benchmark_post_a2a_variants_agree():
    from torchrec_b200.distributed.benchmark import benchmark_set_sharding_context_post_a2a as m
    from torchrec_b200.distributed.embedding import EmbeddingCollectionContext
    from torchrec_b200.distributed.embedding_sharding import _set_sharding_context_post_a2a
    from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    kjt = KeyedJaggedTensor(keys=["a", "b"], values=torch.arange(5), lengths=torch.tensor([1, 1, 1, 2]), stride_per_key_per_rank=[[1, 1], [2, 0]])
    out = []
    for fn in (_set_sharding_context_post_a2a, m._set_sharding_context_post_a2a_zip):
        ctx = EmbeddingCollectionContext(sharding_contexts=[SequenceShardingContext(batch_size_per_rank_per_feature=[])])
        fn([kjt], ctx)
        out.append(ctx.sharding_contexts[0].batch_size_per_rank_per_feature)
    assert out[0] == out[1] == [[1, 2], [1, 0]]
    m.main(["--num_list", "5", "--num_keys", "4"])


def test_benchmark_zch_collision_rates():
    from torchrec_b200.distributed.benchmark.benchmark_zch.benchmark_zch import main

    common = ["--num_tables", "2", "--zch_size", "1000", "--distinct_ids", "700", "--batch_size", "128", "--train_batches", "6", "--eval_batches", "2",
              "--embedding_dim", "8", "--pooling", "2", "--device", "cpu", "--warmup_batches", "1"]
    zch = main(["--zch_method", "mpzch"] + common)
    mod = main(["--zch_method", "none"] + common)
    assert zch["distinct_lookups"] == mod["distinct_lookups"] > 0
    # zero-collision hashing keeps distinct ids apart where a plain modulo does not
    assert zch["collision_rate"] * 3 < mod["collision_rate"]
    assert 0.0 <= zch["auc"] <= 1.0 and zch["train_qps"] > 0


def test_top_level_ebc_benchmark_runs():
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "ebc_benchmarks.py")
    spec = importlib.util.spec_from_file_location("ebc_benchmarks_main", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.get_shrunk_dlrm_num_embeddings(128)[0] == 45833188 // 128 and mod.get_shrunk_dlrm_num_embeddings(128)[1] == 36746
    e, es, f, fs, speedup = mod.get_ebc_comparison(mod._tables([50, 20], dim=8), torch.device("cpu"), epochs=2, batch_size=8, num_batches=2)
    assert e > 0 and f > 0 and speedup > 0


def test_count_dataset_distributions():
    from torchrec_b200.distributed.benchmark.benchmark_zch.count_dataset_distributions import count_distributions, main
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    kjt = KeyedJaggedTensor(keys=["a"], values=torch.tensor([7, 7, 7, 7, 7, 7, 1, 2, 3, 4]), lengths=torch.tensor([10]))
    r = count_distributions([kjt], top_k=1)["a"]
    assert r["lookups"] == 10 and r["distinct_ids"] == 5 and abs(r["top_1_share"] - 0.6) < 1e-9 and r["ids_for_50pct"] == 1 and r["ids_for_90pct"] == 4
    res = main(["--num_batches", "2", "--batch_size", "64", "--distinct_ids", "50"])
    assert set(res) == {"f0", "f1"} and res["f0"]["lookups"] == 128
