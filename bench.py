"""Benchmark of the NVFP4 KV-cache decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c2|c0]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one layer-step of a decode batch through the plugin surface (HorizonFp4Impl): quantize-on-write of the
step's new K/V token of every request, then paged split-K decode + combine over the whole cached context.
Default workload ("c1"): batch 64, 32 query heads / 8 kv heads, head_dim 128, context lengths uniform in
[1024, 8192], page size 16, pages scattered in a 600,000-slot cache, K with 4 outlier channels per head scaled by 20.
All data is synthetic and seeded. With N > 1 every rank runs its own batch of the same shape (requests are
independent: weak scaling, no collective on the timed path; NCCL only gathers the outputs for validation).

Prints ONE JSON line (rank 0). Keys beyond the common contract:
  roofline      the decode kernel alone, timed with CUDA events: algorithmic FP4 cache bytes / duration vs measured peak
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch path to C) on a bounded sample of the same batch
  e2e           the same step with HOST inputs: pinned-memory H2D copies of the step's inputs and a D2H read of the
                output inside the timed region
  parity        max-abs / mean-abs / relative-L2 error of the GPU output against the oracle on that sample
"""
import argparse
import json
import math
import os
import sys
import threading
import time
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("HORIZON_KVFP4_STANDALONE", "1")     # the plugin classes without importing vLLM

WORKLOADS = {
    # name: (B, HQ, KVH, D, PS, pool pages, length law)
    "c0": dict(B=4, HQ=32, KVH=8, D=128, PS=16, pool=1024, law=("const", 2048)),
    "c1": dict(B=64, HQ=32, KVH=8, D=128, PS=16, pool=37500, law=("uniform", 1024, 8192)),
    "c2": dict(B=8, HQ=64, KVH=8, D=128, PS=16, pool=8 * 8192 * 2 + 16, law=("const", 131072)),
    # hybrid batch sharded by request over the GPUs (strong scaling): one batch (6.9 GB of cache reads at N = 1) in a
    # page pool of up to 150 GB per GPU
    "c4": dict(B=2048, HQ=16, KVH=2, D=256, PS=16, pool=int(150e9) // (2 * 2 * 16 * 144), law=("loguniform", 128, 32768),
               sharded=True, n_batches=1),
}
METRIC = "decode_attn_tokens_per_s"


def draw_lens(cfg, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    law = cfg["law"]
    if law[0] == "const":
        return [law[1]] * cfg["B"]
    if law[0] == "loguniform":
        return [int(round(math.exp(x))) for x in rng.uniform(math.log(law[1]), math.log(law[2]), cfg["B"])]
    return [int(x) for x in rng.integers(law[1], law[2] + 1, cfg["B"])]


# --------------------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """samples SM clock and throttle reasons of one GPU with NVML while the GPU is under the benchmark's load"""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.stop, self.max_mhz, self.thread = index, [], set(), False, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self.stop:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop = True
        if self.thread is not None:
            self.thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------------------- workload
def build_batches(cfg, seed, device, n_batches=2, rows=None, lens_seed=None):
    """n_batches decode batches over disjoint pages of one cache pool, written by the CUDA write kernel. `rows` keeps
    only these requests of every batch (the shard of one rank); lens_seed fixes the length draw across ranks."""
    import torch
    from horizon_kernels_b200 import kernels as K
    from horizon_kernels_b200 import layout as Lt
    HQ, KVH, D, PS = cfg["HQ"], cfg["KVH"], cfg["D"], cfg["PS"]
    B = cfg["B"] if rows is None else len(rows)
    g = torch.Generator(device=device).manual_seed(seed)
    page_b = 2 * KVH * PS * Lt.slot_bytes(D)
    free_b, _ = torch.cuda.mem_get_info(device)
    n_pool = min(cfg["pool"], int((free_b - (24 << 30)) // page_b)) if cfg.get("sharded") else cfg["pool"]
    pool = torch.empty((n_pool, 2 * KVH, PS, Lt.slot_bytes(D)), dtype=torch.uint8, device=device)
    perm = torch.randperm(n_pool, generator=g, device=device).to(torch.int32)
    ch = torch.tensor([3, D // 4 + 3, D // 2 + 3, 3 * D // 4 + 3], device=device)
    # global scales amax / (6 * 448): K ~ N(0,1) with x20 outlier channels, V ~ N(0,1); fixed from the distribution's
    # range so that every batch and rank shares them (5.5 sigma)
    gk = torch.full((KVH,), 20.0 * 5.5 / (6 * 448), device=device)
    gv = torch.full((KVH,), 5.5 / (6 * 448), device=device)
    flat, strides = Lt.flat_views(*Lt.slot_views(pool, KVH, D))
    batches, used = [], 0
    for bi in range(n_batches):
        # (a rank whose draw does not fit what is left of the pool draws again: the pool size is the configuration's)
        for attempt in range(256):
            lens = draw_lens(cfg, (seed if lens_seed is None else lens_seed) * 131 + bi + 7919 * attempt)
            if rows is not None:
                lens = [lens[r] for r in rows]
            pages = [(L + PS - 1) // PS for L in lens]
            tot = sum(pages)
            if used + tot <= n_pool or lens_seed is not None:
                break
        if used + tot > n_pool:
            raise RuntimeError("page pool too small for the batches")
        mine = perm[used:used + tot]
        used += tot
        MP = max(pages)
        bt = torch.zeros((B, MP), dtype=torch.int32, device=device)
        o = 0
        for b, n in enumerate(pages):
            bt[b, :n] = mine[o:o + n]
            o += n
        CH = 8192
        for i in range(0, tot, CH):
            pgs = mine[i:i + CH].long()
            n = pgs.numel() * PS
            k = torch.randn(n, KVH, D, generator=g, device=device)
            k[:, :, ch] *= 20.0
            v = torch.randn(n, KVH, D, generator=g, device=device)
            sl = (pgs[:, None] * PS + torch.arange(PS, device=device)[None, :]).reshape(-1)
            K.write(k.to(torch.bfloat16), v.to(torch.bfloat16), flat, strides, PS, sl, gk, gv, True)
            del k, v
        lens_t = torch.tensor(lens, dtype=torch.int32, device=device)
        last = lens_t.long() - 1
        slot_new = bt[torch.arange(B, device=device), (last // PS)].long() * PS + last % PS
        k_new = torch.randn(B, KVH, D, generator=g, device=device)
        k_new[:, :, ch] *= 20.0
        batches.append(SimpleNamespace(
            lens=lens, seq_lens=lens_t, bt=bt, qsl=torch.arange(B + 1, dtype=torch.int32, device=device),
            q=torch.randn(B, HQ, D, generator=g, device=device).to(torch.bfloat16),
            k_new=k_new.to(torch.bfloat16), v_new=torch.randn(B, KVH, D, generator=g, device=device).to(torch.bfloat16),
            slot_new=slot_new.to(torch.int64), out=torch.zeros(B, HQ, D, dtype=torch.bfloat16, device=device)))
    return pool, (flat, strides), gk, gv, batches


def cam_of(bt):
    """what vLLM hands the metadata builder for a pure decode step"""
    B = bt.seq_lens.shape[0]
    return SimpleNamespace(num_reqs=B, num_actual_tokens=B, query_start_loc=bt.qsl, query_start_loc_cpu=bt.qsl_cpu,
                           seq_lens=bt.seq_lens, block_table_tensor=bt.bt, slot_mapping=bt.slot_new,
                           seq_lens_cpu_upper_bound=None)


def algorithmic_bytes(cfg, lens):
    """FP4 cache bytes one decode launch must read: sum(L) * KVH * D * 1.125 (K and V codes plus block scales)"""
    return sum(lens) * cfg["KVH"] * cfg["D"] * 1.125


# ------------------------------------------------------------------------------------------------ CPU oracle legs
def oracle_sample(cfg, host_pool, bt_np, lens, q_bits, gk, gv, rows, threads=None):
    """fp64 attention of the oracle for the requests `rows` of a batch; returns (out rows, seconds, threads)"""
    import numpy as np
    from oracle import kvfp4 as O
    if threads:
        O.set_num_threads(threads)
    KVH, D, PS = cfg["KVH"], cfg["D"], cfg["PS"]
    lay = O.Layout.slots(PS, KVH, D)
    sl = np.array([lens[r] for r in rows], np.int32)
    qsl = np.arange(len(rows) + 1, dtype=np.int32)
    t0 = time.perf_counter()
    out, _ = O.attention(q_bits[rows], host_pool, lay, bt_np[rows], sl, qsl, KVH, float(D) ** -0.5, gk, gv, float(gv[0]))
    return out, time.perf_counter() - t0, O.num_threads()


def run_reference(args, cfg):
    """the CPU arm: the oracle port on all host cores, each step a bounded sample of the default batch (the cache of
    the sampled requests is quantised by the oracle's own writer; no GPU is used)"""
    import numpy as np
    from oracle import kvfp4 as O
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth
    KVH, D, PS, HQ = cfg["KVH"], cfg["D"], cfg["PS"], cfg["HQ"]
    lens_all = draw_lens(cfg, args.seed * 131)
    O.set_num_threads(len(os.sched_getaffinity(0)))        # every host core (torchrun would pin OpenMP to one thread)
    cores = O.num_threads()
    # sample size: requests whose contexts add up to about 40k tokens (a step of a few seconds on ~8 cores)
    rows, tok = [], 0
    for i, L in enumerate(lens_all):
        rows.append(i)
        tok += L
        if tok >= args.ref_tokens:
            break
    lens = [lens_all[r] for r in rows]
    c = synth.paged_case(args.seed + 7, lens, KVH, HQ // KVH, D, PS, outliers=True)
    gk = np.full(KVH, 20.0 * 5.5 / (6 * 448), np.float32)
    gv = np.full(KVH, 5.5 / (6 * 448), np.float32)
    lay = O.Layout.slots(PS, KVH, D)
    cache = np.zeros(c["NP"] * 2 * KVH * PS * (D // 2 + D // 16), np.uint8)
    O.write(c["key"], c["val"], cache, lay, c["slots"], gk, gv, True)
    last = np.array([int(c["bt"][b, (L - 1) // PS]) * PS + (L - 1) % PS for b, L in enumerate(lens)], np.int64)
    first_tok = np.cumsum([0] + lens[:-1])
    k_new = c["key"][first_tok + np.array(lens) - 1]
    v_new = c["val"][first_tok + np.array(lens) - 1]

    def step():
        O.write(k_new, v_new, cache, lay, last, gk, gv, True)
        O.attention(c["q"], cache, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, float(D) ** -0.5, gk, gv, float(gv[0]))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    # throughput of the whole batch at this rate: requests per second scaled by the sample's share of the cached tokens
    value = len(rows) / dt        # the sample's requests follow the batch's length law: its requests / s is the batch's
    sample = f"{len(rows)} of {cfg['B']} requests ({sum(lens)} of {sum(lens_all)} cached tokens) per step"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": args.workload, **{k: cfg[k] for k in ("B", "HQ", "KVH", "D", "PS")},
                       "context": list(cfg["law"]), "sample": sample},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=20261125)
    ap.add_argument("--ref-tokens", type=int, default=150000, help="cached tokens per step of the CPU arm's sample")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the cpu_baseline leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline / parity leg")
    ap.add_argument("--shard", default=None, help="R/N: on one GPU, run only shard R of N of a sharded workload (c4)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        if rank == 0:
            run_reference(args, cfg)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from horizon_kernels_b200 import backend as BE
    from horizon_kernels_b200 import kernels as K
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    B, HQ, KVH, D, PS = cfg["B"], cfg["HQ"], cfg["KVH"], cfg["D"], cfg["PS"]
    NBT = cfg.get("n_batches", 2)
    if cfg.get("sharded"):
        # one batch for the whole job, partitioned by cached tokens; every rank builds only its own requests
        from horizon_kernels_b200.sharding import partition_requests
        lens_all = draw_lens(cfg, args.seed * 131)
        shard_r, shard_n = (int(x) for x in args.shard.split("/")) if (args.shard and world == 1) else (rank, world)
        rows = partition_requests(lens_all, shard_n)[shard_r]
        pool, (flat, strides), gk, gv, batches = build_batches(cfg, args.seed + 1000 * rank, device, NBT, rows, args.seed)
        B = len(rows)
    else:
        # weak scaling: every rank gets the same context lengths (the same work) on its own pages and data
        pool, (flat, strides), gk, gv, batches = build_batches(cfg, args.seed + 1000 * rank, device, NBT, None, args.seed)
    for bt in batches:
        bt.qsl_cpu = bt.qsl.cpu()
    impl = BE.HorizonFp4Impl(HQ, D, float(D) ** -0.5, num_kv_heads=KVH, kv_cache_dtype="nvfp4", max_num_seqs=max(B, 1))
    builder = BE.HorizonFp4Builder()
    layer = SimpleNamespace(_k_scale_float=float(gk[0]), _v_scale_float=float(gv[0]), layer_name="layers.0.attn")
    metas = [builder.build(0, cam_of(bt)) for bt in batches]

    def step(i):
        bt, m = batches[i % len(batches)], metas[i % len(batches)]
        impl.do_kv_cache_update(layer, bt.k_new, bt.v_new, pool, bt.slot_new)
        impl.forward(layer, bt.q, bt.k_new, bt.v_new, pool, m, bt.out)

    # ---- CUDA graphs of one step per batch (the surface allocates nothing and never synchronises)
    for i in range(len(batches)):
        step(i)
    torch.cuda.synchronize()
    graphs = []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(len(batches)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                step(i)
            graphs.append(g)
        # a serving engine captures all layers of a model in one graph: CHAIN consecutive steps (alternating batches)
        # in one graph, so that a step's launches follow the previous step's without a graph boundary in between
        CHAIN = 5 * NBT
        chain_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(chain_graph, stream=side):
            for i in range(CHAIN):
                step(i)
    torch.cuda.synchronize()

    def replay_steps(n, first=0):
        i = first
        while n - (i - first) >= CHAIN and i % NBT == 0:
            chain_graph.replay()
            i += CHAIN
        while i - first < n:
            graphs[i % NBT].replay()
            i += 1

    # graphs holding only the decode launch, for the roofline timing of that kernel
    v_scale = float(gv[0])

    def decode_only(i):
        bt, m = batches[i % NBT], metas[i % NBT]
        v = impl._cache_views(pool)
        K.decode_ragged(bt.q, v["flat"], v["strides"], PS, m.block_table, m.seq_lens, m.query_start_loc, impl.scale,
                        v_scale, gk, gv, 1, bt.out, impl._state(device)["ws"], _combine=False)
    dgraph = torch.cuda.CUDAGraph()                  # args.steps launches back to back, alternating batches
    with torch.cuda.stream(side):
        with torch.cuda.graph(dgraph, stream=side):
            for i in range(max(args.steps, 1)):
                decode_only(i)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with sampler:
        # the GPU is kept under the same load before and after the timed steps so that the 20 ms clock samples see it
        t_end = time.perf_counter() + 0.6
        i = 0
        while time.perf_counter() < t_end:
            graphs[i % NBT].replay()
            i += 1
        for i in range(args.warmup):
            graphs[i % NBT].replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        replay_steps(args.steps)
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)

        # ---- the decode kernel alone (roofline): graphs holding only that launch, CUDA events around K replays
        torch.cuda.synchronize()
        dgraph.replay()                                  # warm-up: the same args.steps launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        dgraph.replay()
        b.record()
        b.synchronize()
        dec_ms = [a.elapsed_time(b) / max(args.steps, 1)]

        # ---- end to end: host inputs -> one pinned H2D copy -> write + decode + combine (graph) -> D2H of the output.
        # The step's inputs (query, new K/V rows, slot ids, context lengths, query offsets, block tables) sit back to
        # back in one pinned host buffer and one device buffer, so a step is one H2D copy, one graph launch over views
        # of the device buffer, one D2H copy and a stream synchronize: what a serving engine's model runner does.
        def packed(bt):
            parts = dict(q=bt.q, k=bt.k_new, v=bt.v_new, slot=bt.slot_new, sl=bt.seq_lens, qsl=bt.qsl, bt=bt.bt)
            offs, n = {}, 0
            for name, t in parts.items():
                offs[name] = n
                n += (t.numel() * t.element_size() + 255) // 256 * 256
            host = torch.empty(n, dtype=torch.uint8).pin_memory()
            dev = torch.empty(n, dtype=torch.uint8, device=device)
            hv, dv = {}, {}
            for name, t in parts.items():
                nb = t.numel() * t.element_size()
                hv[name] = host[offs[name]:offs[name] + nb].view(t.dtype).view(t.shape)
                dv[name] = dev[offs[name]:offs[name] + nb].view(t.dtype).view(t.shape)
                hv[name].copy_(t.cpu())
            return SimpleNamespace(host=host, dev=dev, h=hv, d=SimpleNamespace(**dv), nbytes=sum(
                t.numel() * t.element_size() for t in parts.values()))
        packs = [packed(bt) for bt in batches]
        for pk, bt in zip(packs, batches):
            pk.out_dev = torch.empty_like(bt.out)
            pk.out_host = torch.empty_like(bt.out, device="cpu").pin_memory()
            pk.dev.copy_(pk.host)
            cam = SimpleNamespace(num_reqs=B, num_actual_tokens=B, query_start_loc=pk.d.qsl,
                                  query_start_loc_cpu=pk.h["qsl"], seq_lens=pk.d.sl, block_table_tensor=pk.d.bt,
                                  slot_mapping=pk.d.slot, seq_lens_cpu_upper_bound=None)
            pk.meta = builder.build(0, cam)
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            for pk in packs:
                impl.do_kv_cache_update(layer, pk.d.k, pk.d.v, pool, pk.d.slot)
                impl.forward(layer, pk.d.q, pk.d.k, pk.d.v, pool, pk.meta, pk.out_dev)
                pk.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(pk.graph, stream=side):
                    impl.do_kv_cache_update(layer, pk.d.k, pk.d.v, pool, pk.d.slot)
                    impl.forward(layer, pk.d.q, pk.d.k, pk.d.v, pool, pk.meta, pk.out_dev)
        torch.cuda.synchronize()
        h2d = packs[0].nbytes
        d2h = packs[0].out_host.numel() * packs[0].out_host.element_size()

        def e2e_step(i):
            pk = packs[i % NBT]
            pk.dev.copy_(pk.host, non_blocking=True)
            pk.graph.replay()
            pk.out_host.copy_(pk.out_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()       # the caller reads the result
        for i in range(args.warmup):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        barrier()
        e2e_s = time.perf_counter() - t0
        t_end = time.perf_counter() + 0.4
        i = 0
        while time.perf_counter() < t_end:
            graphs[i % NBT].replay()
            i += 1
        torch.cuda.synchronize()
    clocks = sampler.summary()

    # ---- max over ranks
    times = torch.tensor([ms_total, e2e_s * 1e3, sum(dec_ms) / len(dec_ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, dec_ms_avg = (float(x) for x in times.cpu())
    ms_step = ms_total / args.steps
    n_req = (B if args.shard else cfg["B"]) if cfg.get("sharded") else B * world   # requests of the whole job per step
    value = n_req / (ms_step * 1e-3)
    e2e_value = n_req / (e2e_ms / args.steps * 1e-3)

    # ---- validation: outputs gathered with NCCL (the only collective), checked on rank 0
    for i in range(NBT):
        step(i)
    torch.cuda.synchronize()
    status = K.workspace_status(impl._state(device)["ws"])
    finite = bool(torch.isfinite(batches[0].out.float()).all())
    # the end-to-end path (host buffers) and the device-resident path compute the same step: bit-identical outputs
    e2e_equal = bool(torch.equal(packs[0].out_host, batches[0].out.cpu()))
    if world > 1:
        if cfg.get("sharded"):
            from horizon_kernels_b200.sharding import gather_outputs
            full = gather_outputs(batches[0].out, rows, cfg["B"])            # request order of the whole batch
            finite = bool(torch.isfinite(full.float()).all()) and full.shape[0] == cfg["B"]
        else:
            outs = [torch.empty_like(batches[0].out) for _ in range(world)]
            dist.all_gather(outs, batches[0].out)
            finite = all(bool(torch.isfinite(o.float()).all()) for o in outs)
        st = torch.tensor([status], device=device)
        dist.all_reduce(st, op=dist.ReduceOp.MIN)
        status = int(st)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    alg = algorithmic_bytes(cfg, [L for bt in batches for L in bt.lens]) / NBT      # rank 0's launch
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    achieved = alg / (dec_ms_avg * 1e-3) / 1e9
    # DRAM traffic of one decode launch of this workload from the ncu capture summarised in profiles/ (read + written
    # bytes), scaled by the algorithmic bytes of this run's batches
    traffic = alg * TRAFFIC_RATIO.get(args.workload, float("nan")) if args.workload in TRAFFIC_RATIO else None
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if cfg.get("sharded") else "weak",
            "vs_baseline": None, "dtype": "f16 mma over e2m1 x e4m3 dequantised values, fp32 softmax and accumulation",
            "data": "synthetic",
            "config": {"workload": args.workload, **{k: cfg[k] for k in ("B", "HQ", "KVH", "D", "PS")},
                       "context": list(cfg["law"]), "pool_pages": int(pool.shape[0]), "per_gpu_batch": B,
                       "step": "quantize-on-write of 1 new token per request + paged decode + combine, one layer",
                       "l2": ("two batches on disjoint pages alternate, each reads more cache bytes than the L2 holds"
                              if NBT > 1 else "one batch whose cache reads per GPU exceed the L2 several times"),
                       "timing": ("CUDA graphs of the plugin calls (5 steps per batch chained in one graph, like the layers "
                                  "of a model), CUDA events around the K steps, max over ranks; roofline: K decode "
                                  "launches back to back in one graph, CUDA events around it, divided by K"),
                       "clocks": "NVML sampled every 20 ms while the same step loops before, during and after the timed steps"},
            "tokens_per_s_per_gpu": value / world,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_src, "kernel": "hkv::decode_kernel",
                         "algorithmic_bytes_per_launch": alg, "kernel_ms": dec_ms_avg,
                         "frac_of_nominal_8tbs": achieved / 8000.0},
            "step_hbm_gbs": alg / (ms_step * 1e-3) / 1e9,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": 3 * args.steps, "clocks": clocks, "device_status": status, "outputs_finite": finite,
            "e2e_output_equal": e2e_equal}

    if world == 1 and not args.no_cpu:
        # ---- CPU baseline and parity on a bounded sample of batch 0 (the oracle is the checker, never the product)
        bt = batches[0]
        host_pool = pool.cpu().numpy().reshape(-1)
        bt_np, q_bits = bt.bt.cpu().numpy(), bt.q.cpu().view(torch.int16).numpy().view(np.uint16)
        gk_np, gv_np = gk.cpu().numpy(), gv.cpu().numpy()
        O_threads = len(os.sched_getaffinity(0))
        order = sorted(range(B), key=lambda r: bt.lens[r])
        _, t1, cores = oracle_sample(cfg, host_pool, bt_np, bt.lens, q_bits, gk_np, gv_np, order[:1], O_threads)
        rate = bt.lens[order[0]] / max(t1, 1e-6)                         # cached tokens per second, first estimate
        rows, tok = [], 0
        for r in range(B):
            if tok + bt.lens[r] > rate * args.cpu_seconds and rows:
                break
            rows.append(r)
            tok += bt.lens[r]
        ref, secs, cores = oracle_sample(cfg, host_pool, bt_np, bt.lens, q_bits, gk_np, gv_np, rows, O_threads)
        got = bt.out[rows].float().cpu().numpy().astype(np.float64)
        d = np.abs(got - ref)
        line["cpu_baseline"] = {"value": len(rows) / secs, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"{len(rows)} of {B} requests of the same batch ({tok} of {sum(bt.lens)} cached "
                                          f"tokens), decode only, {secs:.1f} s"}
        line["parity"] = {"max_abs": float(d.max()), "mean_abs": float(d.mean()),
                          "rel_l2": float(np.linalg.norm(got - ref) / np.linalg.norm(ref)), "requests": len(rows),
                          "against": "CPU oracle (fp64 attention over the same cache bytes)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + written) per algorithmic byte of one decode launch, from the ncu captures summarised under
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum over sum(L) * KVH * D * 1.125)
TRAFFIC_RATIO = {"c1": (330.123 + 4.825) / 328.42, "c2": (1209.754 + 4.464) / 1207.960}

if __name__ == "__main__":
    main()
