"""Train and evaluate a small DLRM whose sparse ids come from a huge raw id space through a managed-collision module, and report
throughput (samples/s), collision rate of the remapping, and AUC / normalized entropy on held-out batches.

    python -m torchrec_b200.distributed.benchmark.benchmark_zch.benchmark_zch --zch_method mpzch
    python -m torchrec_b200.distributed.benchmark.benchmark_zch.benchmark_zch --zch_method none      # modulo-hash baseline

Labels depend on the *raw* ids (a hidden per-id propensity), so rows shared by several ids hurt AUC/NE measurably.
Counterpart of ``torchrec/distributed/benchmark/benchmark_zch/benchmark_zch.py``."""
from __future__ import annotations

import json
import time
from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.distributed.benchmark.benchmark_zch.arguments import parse_args
from torchrec_b200.distributed.benchmark.benchmark_zch.benchmark_zch_utils import BenchmarkMCProbe, ZipfIdStream
from torchrec_b200.metrics.auc import compute_auc
from torchrec_b200.metrics.ne import compute_cross_entropy, compute_ne
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.mc_adapter import McEmbeddingBagCollectionAdapter
from torchrec_b200.modules.mlp import MLP
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class _ModuloEBC(nn.Module):
    """Baseline: fold raw ids into the table with a modulo."""

    def __init__(self, tables: List[EmbeddingBagConfig], device: torch.device) -> None:
        super().__init__()
        self.ebc = EmbeddingBagCollection(tables=tables, device=device)
        self._rows = tables[0].num_embeddings
        self.remapped_ids: Optional[KeyedJaggedTensor] = None

    def forward(self, kjt: KeyedJaggedTensor):
        self.remapped_ids = KeyedJaggedTensor(keys=kjt.keys(), values=kjt.values() % self._rows, lengths=kjt.lengths())
        return self.ebc(self.remapped_ids)


class _Net(nn.Module):
    def __init__(self, sparse: nn.Module, num_tables: int, dim: int, num_dense: int, device: torch.device) -> None:
        super().__init__()
        self.sparse = sparse
        self.dense = MLP(num_dense, [64, dim], device=device)
        self.over = MLP(dim * (num_tables + 1), [128], device=device)
        self.over_last = nn.Linear(128, 1, device=device)

    def forward(self, dense: torch.Tensor, kjt: KeyedJaggedTensor) -> torch.Tensor:
        pooled = self.sparse(kjt)
        return self.over_last(self.over(torch.cat([self.dense(dense).float(), pooled.values().float()], dim=1)).float()).squeeze(-1)


def _make_batch(args, stream: ZipfIdStream, propensity: List[Dict[int, float]], gen: torch.Generator, device: torch.device):
    B, F, L = args.batch_size, args.num_tables, args.pooling
    values, logit = [], torch.zeros(B)
    for f in range(F):
        raw = stream.draw(f, B * L)
        values.append(raw)
        # hidden per-raw-id effect: a fixed pseudo-random number in [-1, 1] derived from the id
        eff = ((raw * 2654435761 % 1000003).double() / 1000003.0 * 2 - 1).float()
        logit += eff.view(B, L).mean(1)
    dense = torch.randn(B, args.num_float_features, generator=gen)
    label = (torch.rand(B, generator=gen) < torch.sigmoid(2.0 * logit + 0.3 * dense[:, 0])).float()
    kjt = KeyedJaggedTensor(keys=[f"f{i}" for i in range(F)], values=torch.cat(values), lengths=torch.full((F * B,), L, dtype=torch.int64))
    return dense.to(device), kjt.to(device), label.to(device)


def run(args) -> Dict[str, float]:
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    torch.manual_seed(args.seed)
    gen = torch.Generator().manual_seed(args.seed + 1)
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=args.embedding_dim, num_embeddings=args.zch_size, feature_names=[f"f{i}"]) for i in range(args.num_tables)]
    if args.zch_method == "none":
        sparse: nn.Module = _ModuloEBC(tables, device)
    else:
        sparse = McEmbeddingBagCollectionAdapter(tables, input_hash_size=args.input_hash_size, device=device, world_size=1, eviction_interval=args.eviction_interval,
                                                 zch_method=args.zch_method, mpzch_num_buckets=args.mpzch_num_buckets, mpzch_max_probe=args.mpzch_max_probe)
        sparse.mc_embedding_bag_collection._return_remapped_features = True  # the probe needs the rows the ids landed on
        emb = sparse.mc_embedding_bag_collection._embedding_module
        if any(p.is_meta for p in emb.parameters()):
            emb.to_empty(device=device)
            for p in emb.parameters():
                nn.init.uniform_(p, -0.05, 0.05)
    model = _Net(sparse, args.num_tables, args.embedding_dim, args.num_float_features, device)
    opt = torch.optim.Adagrad([p for p in model.parameters() if p.requires_grad], lr=args.lr)
    stream = ZipfIdStream(args.num_tables, args.distinct_ids, args.zipf_alpha, args.input_hash_size, args.seed)
    probe = BenchmarkMCProbe([t.name for t in tables], args.zch_size, device)

    def step(train: bool) -> Tuple[torch.Tensor, torch.Tensor]:
        dense, kjt, label = _make_batch(args, stream, [], gen, device)
        logits = model(dense, kjt)
        remapped = sparse.remapped_ids
        if remapped is not None:
            raw_d, rem_d = kjt.to_dict(), remapped.to_dict()
            for i, t in enumerate(tables):
                probe.record(t.name, raw_d[f"f{i}"].values(), rem_d[f"f{i}"].values())
        if train:
            opt.zero_grad()
            nn.functional.binary_cross_entropy_with_logits(logits, label).backward()
            opt.step()
        return logits.detach(), label

    model.train()
    for _ in range(args.warmup_batches):
        step(True)
    if device.type == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.train_batches):
        step(True)
    if device.type == "cuda":
        torch.cuda.synchronize()
    train_s = time.perf_counter() - t0
    model.eval()
    preds, labels = [], []
    with torch.no_grad():
        for _ in range(args.eval_batches):
            lg, lb = step(False)
            preds.append(torch.sigmoid(lg))
            labels.append(lb)
    p, y = torch.cat(preds).double().unsqueeze(0), torch.cat(labels).double().unsqueeze(0)
    w = torch.ones_like(p)
    ce = compute_cross_entropy(y, p, w, 1e-12).sum(-1)
    ne = compute_ne(ce, w.sum(-1), (y * w).sum(-1), ((1 - y) * w).sum(-1), 1e-12)
    out = {"zch_method": args.zch_method, "train_qps": args.train_batches * args.batch_size / train_s, "auc": float(compute_auc(1, p, y, w)[0]), "ne": float(ne[0])}
    out.update(probe.summary())
    return out


def main(argv=None) -> Dict[str, float]:
    args = parse_args(argv)
    res = run(args)
    print(json.dumps(res))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(res, f)
    return res


if __name__ == "__main__":
    main()
