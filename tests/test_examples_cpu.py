"""The example scripts run end to end on CPU with tiny settings (each in its own process, as a user would start them)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = {
    "golden_training": (["examples/golden_training/train_dlrm.py", "--num_embeddings", "500", "--embedding_dim", "16", "--num_tables", "3", "--batch_size", "32",
                         "--num_iterations", "4"], 29611),
    "binary_dataloader": (["examples/binary_dataloader/train_from_binary.py", "--num_rows", "256", "--batch_size", "64", "--hash_size", "100", "--embedding_dim", "16"], 29612),
    "bert4rec": (["examples/bert4rec/bert4rec_main.py", "--vocab_size", "300", "--max_len", "8", "--emb_dim", "16", "--nhead", "2", "--num_layers", "1", "--batch_size", "8",
                  "--num_negatives", "16", "--num_iterations", "2", "--sharding", "table_wise"], 29613),
    "zch": (["examples/zch/main.py", "--zch_size", "256", "--distinct_ids", "150", "--batch_size", "32", "--num_iterations", "3"], 29614),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_example_runs(name):
    args, port = CASES[name]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
