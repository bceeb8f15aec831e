"""Multi-GPU host logic on CPU: the request partition is balanced and identical on every rank, and two gloo ranks that
each run the (oracle) decode of their own shard reassemble exactly the single-process result."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import synth
from horizon_kernels_b200.sharding import kv_bytes, partition_requests


def test_partition_is_balanced_and_complete():
    rng = np.random.default_rng(0)
    lens = np.exp(rng.uniform(np.log(128), np.log(32768), 2048)).astype(int).tolist()
    for n in (1, 2, 4, 8):
        shards = partition_requests(lens, n)
        assert sorted(i for s in shards for i in s) == list(range(len(lens)))
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.01 * sum(lens) / n + max(lens)
        assert shards == partition_requests(lens, n)
    assert kv_bytes(16, 2, 256) == 16 * 2 * 288


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, q):
    from oracle import kvfp4 as O
    from horizon_kernels_b200.sharding import gather_outputs
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lens = [40, 300, 17, 129, 64, 7]
    KVH, G, D, PS = 2, 4, 128, 16
    c = synth.paged_case(77, lens, KVH, G, D, PS, outliers=True)
    lay = O.Layout.slots(PS, KVH, D)
    cache = np.zeros(c["NP"] * 2 * KVH * PS * 72, np.uint8)
    gk = np.full(KVH, 0.05, np.float32)
    gv = np.full(KVH, 0.01, np.float32)
    O.write(c["key"], c["val"], cache, lay, c["slots"], gk, gv, True)
    mine = partition_requests(lens, world)[rank]
    sl = c["seq_lens"][mine]
    qsl = np.arange(len(mine) + 1, dtype=np.int32)
    out, _ = O.attention(c["q"][mine], cache, lay, c["bt"][mine], sl, qsl, KVH, D ** -0.5, gk, gv)
    full = gather_outputs(torch.from_numpy(out), mine, len(lens))
    if rank == 0:
        ref, _ = O.attention(c["q"], cache, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, D ** -0.5, gk, gv)
        q.put(bool(np.array_equal(full.numpy(), ref)))
    dist.destroy_process_group()


def test_two_gloo_ranks_reassemble_the_batch():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    ok = q.get(timeout=120)
    for p in ps:
        p.join(60)
    assert ok and all(p.exitcode == 0 for p in ps)
