"""Multi-rank check run under torchrun: data-parallel embedding gather (producer-side peer stores) and sharded
search with the peer-memory top-k merge must match single-rank references."""
import os, sys
import torch, torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import antfly_b200  # first: sets the multicast-off defaults before NCCL or the symmetric allocator start
from antfly_b200.parallel.launch import install_exit_guards, finish_ranks
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ["LOCAL_RANK"])
install_exit_guards(local, watchdog_s=150)
torch.cuda.set_device(local); dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
from antfly_b200 import _native as N
from antfly_b200.index.flat import FlatIndex, recall_at_k
from antfly_b200.index.sharded import ShardedFlatIndex
from antfly_b200.models.bert import BertConfig, BertModel, pack_sequences
from antfly_b200.parallel.dp_embed import DpEmbedder

cfg = BertConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512, vocab_size=1000)
model = BertModel.random_init(cfg, device=dev, seed=0)  # same seed: replicated weights
g = torch.Generator().manual_seed(5)
all_seqs = [torch.randint(5, 1000, (int(n),), generator=g).tolist() for n in torch.randint(4, 60, (8 * world,), generator=g)]
mine = all_seqs[rank * 8:(rank + 1) * 8]
dp = DpEmbedder(model, rank, world, max_local_batch=64)
ok = True
for it in range(2):
    got = dp.embed(pack_sequences(mine).to(dev)).clone()
    ref = model.embed(pack_sequences(all_seqs).to(dev))
    err = float((got - ref).abs().max())
    ok = ok and err < 2e-3
    print(f"rank {rank}: dp gather err={err:.2e}", flush=True)

gd = torch.Generator(device=dev).manual_seed(11)  # same data on every rank, each keeps its shard
x = torch.nn.functional.normalize(torch.randn(4000 * world, 64, generator=gd, device=dev), dim=-1)
q = torch.nn.functional.normalize(torch.randn(33, 64, generator=gd, device=dev), dim=-1)
sh = ShardedFlatIndex(x[rank * 4000:(rank + 1) * 4000], "cosine", rank, world, 4000, max_queries=64, max_k=32)
for it in range(2):
    res = sh.search(q, 20)
    full = FlatIndex(x, metric="cosine").search(q, 20)
    same = recall_at_k(res.ids, full.ids, 20)
    ok = ok and same > 0.999 and bool(torch.allclose(res.distances, full.distances, atol=1e-3))
    print(f"rank {rank}: sharded search agreement={same:.4f}", flush=True)
# sharded IVF: jointly trained centroids, local list scans, the same pushed merge
from antfly_b200.index.ivf import IVFIndex
from antfly_b200.index.sharded import ShardedIVFIndex
siv = ShardedIVFIndex(x[rank * 4000:(rank + 1) * 4000], 32, "cosine", rank, world, 4000, max_queries=64, max_k=32)
for it in range(2):
    res = siv.search(q, 20, nprobe=32)             # all lists probed: must equal the exact search
    full = FlatIndex(x, metric="cosine").search(q, 20)
    same = recall_at_k(res.ids, full.ids, 20)
    ok = ok and same > 0.999
    print(f"rank {rank}: sharded ivf (all lists) agreement={same:.4f}", flush=True)
st = N.status()
print(f"rank {rank}: DP_SHARDED_CHECK {'OK' if ok and st == 0 else 'FAILED'} status={st}", flush=True)
finish_ranks()
