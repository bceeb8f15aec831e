"""Benchmark of the NVFP4 KV-cache decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4|c1|c2|c0]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one layer-step of a decode batch through the plugin surface (HorizonFp4Impl): quantize-on-write of the
step's new K/V token of every request, then the paged split-K decode (split sequences are merged inside that launch)
over the whole cached context.

Default workload ("c4", the hybrid batch of the task's configuration list, its largest single-GPU case): batch 2048,
16 query heads / 2 kv heads, head_dim 256, context lengths log-uniform in [128, 32768], page size 16, pages scattered
over a pool of up to 150 GB per GPU. With N > 1 the 2048 requests of ONE batch are partitioned over the ranks by cached
tokens (strong scaling); nothing is exchanged on the timed path and NCCL only gathers the outputs afterwards, where
rank 0 checks rows owned by every rank against the CPU oracle. The other workloads ("c1": batch 64, 32 / 8 heads,
head_dim 128, contexts uniform in [1024, 8192]; "c2": batch 8, 64 / 8 heads, 131072 tokens each; "c0") run as
independent replicas per rank (weak scaling). All data is synthetic and seeded.

Prints ONE JSON line (rank 0). Keys beyond the common contract:
  roofline        the decode kernel of the timed workload alone: algorithmic FP4 cache bytes / CUDA-event duration
                  against the measured copy peak; median, min and max over repeats, back to back and launch by launch
  roofline_c1/c2  the same for the decode kernel on configurations 1 and 2 (rank 0, before the timed workload)
  step_samples    per-step time of every replay unit inside the timed region (median / min / max)
  cpu_baseline    the CPU oracle (a C port of the reference's PyTorch path) on a bounded sample of the same batch
  e2e             the same step with HOST inputs: pinned-memory H2D copies of the step's inputs and a D2H read of the
                  output inside the timed region, with a breakdown of its parts
  parity          max-abs / mean-abs / relative-L2 error of the GPU output against the oracle: requests of every rank
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
REPEATS = 11                      # replays behind every median of the kernel-only figures
# DRAM bytes (read + written) per algorithmic byte of one decode launch, from the ncu captures summarised under
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum over sum(L) * KVH * D * 1.125); c4's capture is one rank's
# share of the batch at 8 GPUs (same length law), and traffic grows in proportion to the cached tokens
TRAFFIC_RATIO = {"c1": (296.768 + 5.083) / 297.3, "c2": (1210.028 + 3.940) / 1207.960,
                 "c4": (565.765 + 5.784) / 560.241}


def draw_lens(cfg, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    law = cfg["law"]
    if law[0] == "const":
        return [law[1]] * cfg["B"]
    if law[0] == "loguniform":
        return [int(round(math.exp(x))) for x in rng.uniform(math.log(law[1]), math.log(law[2]), cfg["B"])]
    return [int(x) for x in rng.integers(law[1], law[2] + 1, cfg["B"])]


def stats(xs):
    s = sorted(xs)
    return {"median": s[len(s) // 2], "min": s[0], "max": s[-1], "n": len(s)}


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


def setup_workload(name, device, seed, rank, world, shard=None):
    """builds the batches of a workload on this rank and the plugin objects that run a step of it"""
    import torch
    from horizon_kernels_b200 import backend as BE
    cfg = WORKLOADS[name]
    NBT = cfg.get("n_batches", 2)
    rows = None
    if cfg.get("sharded"):
        # one batch for the whole job, partitioned by cached tokens; every rank builds only its own requests
        from horizon_kernels_b200.sharding import partition_requests
        lens_all = draw_lens(cfg, seed * 131)
        shard_r, shard_n = (int(x) for x in shard.split("/")) if (shard and world == 1) else (rank, world)
        rows = partition_requests(lens_all, shard_n)[shard_r]
        pool, (flat, strides), gk, gv, batches = build_batches(cfg, seed + 1000 * rank, device, NBT, rows, seed)
    else:
        # weak scaling: every rank gets the same context lengths (the same work) on its own pages and data
        pool, (flat, strides), gk, gv, batches = build_batches(cfg, seed + 1000 * rank, device, NBT, None, seed)
    B = len(batches[0].lens)
    for bt in batches:
        bt.qsl_cpu = bt.qsl.cpu()
    impl = BE.HorizonFp4Impl(cfg["HQ"], cfg["D"], float(cfg["D"]) ** -0.5, num_kv_heads=cfg["KVH"],
                             kv_cache_dtype="nvfp4", max_num_seqs=max(B, 1))
    builder = BE.HorizonFp4Builder()
    layer = SimpleNamespace(_k_scale_float=float(gk[0]), _v_scale_float=float(gv[0]), layer_name="layers.0.attn")
    w = SimpleNamespace(name=name, cfg=cfg, NBT=NBT, rows=rows, B=B, pool=pool, flat=flat, strides=strides, gk=gk,
                        gv=gv, batches=batches, impl=impl, builder=builder, layer=layer, device=device,
                        metas=[builder.build(0, cam_of(bt)) for bt in batches], side=torch.cuda.Stream(),
                        v_scale=float(gv[0]))

    def step(i):
        bt, m = w.batches[i % NBT], w.metas[i % NBT]
        impl.do_kv_cache_update(layer, bt.k_new, bt.v_new, pool, bt.slot_new)
        impl.forward(layer, bt.q, bt.k_new, bt.v_new, pool, m, bt.out)
    w.step = step
    for i in range(NBT):                                # first calls outside capture: workspace, per-device set-up
        step(i)
    torch.cuda.synchronize()
    return w


def decode_only(w, i):
    """the decode launch of step i alone (split sequences are merged inside it)"""
    from horizon_kernels_b200 import kernels as K
    bt, m = w.batches[i % w.NBT], w.metas[i % w.NBT]
    v = w.impl._cache_views(w.pool)
    K.decode_ragged(bt.q, v["flat"], v["strides"], w.cfg["PS"], m.block_table, m.seq_lens, m.query_start_loc,
                    w.impl.scale, w.v_scale, w.gk, w.gv, 1, bt.out, w.impl._state(w.device)["ws"])


def time_decode_kernel(w, launches, local, seconds=0.35):
    """the decode kernel alone, timed with CUDA events on the launching stream:
      back to back  `launches` launches (alternating batches) in one graph, events around a replay, / launches; with
                    programmatic dependent launch the prologue of launch k + 1 overlaps the tail of launch k, as it
                    does between the layers of a model
      isolated      one launch per graph, captured with the early-metadata option off, events around each replay:
                    nothing overlaps, and the event pair's own overhead is inside the figure
    REPEATS replays each, medians with min / max; the SM clock is sampled while the same graphs keep the GPU loaded."""
    import torch
    from horizon_kernels_b200 import kernels as K
    launches = max(1, launches)
    with torch.cuda.stream(w.side):
        dgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(dgraph, stream=w.side):
            for i in range(launches):
                decode_only(w, i)
        K.set_option(K.OPT_EARLY_METADATA, 0)
        singles = []
        for i in range(w.NBT):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=w.side):
                decode_only(w, i)
            singles.append(g)
        K.set_option(K.OPT_EARLY_METADATA, 0 if os.environ.get("HORIZON_KVFP4_EARLY_META", "1") == "0" else 1)
    torch.cuda.synchronize()

    def timed(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        return a.elapsed_time(b)
    sampler = ClockSampler(local)
    with sampler:
        t_end = time.perf_counter() + seconds          # load before the samples, so that the clocks are the loaded ones
        while time.perf_counter() < t_end:
            dgraph.replay()
        torch.cuda.synchronize()
        b2b = [timed(dgraph.replay) / launches for _ in range(REPEATS)]
        iso = [timed(singles[i % w.NBT].replay) for i in range(REPEATS * w.NBT)]
        t_end = time.perf_counter() + 0.1
        while time.perf_counter() < t_end:
            dgraph.replay()
        torch.cuda.synchronize()
    return {"back_to_back_ms": stats(b2b), "isolated_ms": stats(iso), "launches_per_replay": launches,
            "clocks": sampler.summary(), "b2b_samples": b2b, "iso_samples": iso, "clock_samples": list(sampler.samples)}


def merge_timings(a, b):
    """two legs of time_decode_kernel (before and after the timed steps) as one record: under the power cap the SM clock
    wanders by 10 to 15 % over seconds, so the kernel is sampled on both sides of the region it is compared with"""
    b2b, iso, clk = a["b2b_samples"] + b["b2b_samples"], a["iso_samples"] + b["iso_samples"], sorted(
        a["clock_samples"] + b["clock_samples"])
    return {"back_to_back_ms": stats(b2b), "isolated_ms": stats(iso), "launches_per_replay": a["launches_per_replay"],
            "clocks": {"sm_mhz": clk[len(clk) // 2] if clk else None, "sm_max_mhz": a["clocks"]["sm_max_mhz"],
                       "reasons": sorted(set(a["clocks"]["reasons"]) | set(b["clocks"]["reasons"])), "samples": len(clk)},
            "b2b_samples": b2b, "iso_samples": iso, "clock_samples": clk}


def roofline_record(w, t, peak, peak_src):
    alg = algorithmic_bytes(w.cfg, [L for bt in w.batches for L in bt.lens]) / w.NBT      # this rank's launch
    ms, iso = t["back_to_back_ms"]["median"], t["isolated_ms"]["median"]
    achieved = alg / (ms * 1e-3) / 1e9
    ratio = TRAFFIC_RATIO.get(w.name)
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": alg * ratio if ratio else None, "peak_source": peak_src, "kernel": "hkv::decode_kernel",
            "workload": w.name, "algorithmic_bytes_per_launch": alg, "kernel_ms": ms,
            "kernel_ms_min": t["back_to_back_ms"]["min"], "kernel_ms_max": t["back_to_back_ms"]["max"],
            "repeats": t["back_to_back_ms"]["n"], "launches_per_replay": t["launches_per_replay"],
            "kernel_ms_samples": [round(x, 5) for x in t["b2b_samples"]],
            "frac_of_nominal_8tbs": achieved / 8000.0,
            "isolated_kernel_ms": iso, "isolated_kernel_ms_min": t["isolated_ms"]["min"],
            "isolated_kernel_ms_max": t["isolated_ms"]["max"], "frac_isolated": alg / (iso * 1e-3) / 1e9 / peak,
            "sm_mhz": t["clocks"]["sm_mhz"], "clock_reasons": t["clocks"]["reasons"]}


# ------------------------------------------------------------------------------------------------ CPU oracle legs
def extract_requests(w, bt, rows):
    """the cache pages of the requests `rows` of a batch as a compact host pool (pages renumbered from 0) with its
    block table: what the CPU oracle needs, without copying a 150 GB pool to the host"""
    import numpy as np
    import torch
    PS = w.cfg["PS"]
    n_pages = [(bt.lens[r] + PS - 1) // PS for r in rows]
    ids = torch.cat([bt.bt[r, :n] for r, n in zip(rows, n_pages)]).long() if rows else torch.zeros(0, dtype=torch.long)
    sub = w.pool[ids].cpu().numpy().reshape(-1)
    btc = np.zeros((len(rows), max(n_pages) if rows else 1), np.int32)
    o = 0
    for i, n in enumerate(n_pages):
        btc[i, :n] = np.arange(o, o + n)
        o += n
    return sub, btc


def oracle_rows(w, bt, rows, threads=None):
    """fp64 attention of the oracle for the requests `rows` of a batch; returns (out rows, seconds, threads)"""
    import numpy as np
    import torch
    from oracle import kvfp4 as O
    if threads:
        O.set_num_threads(threads)
    cfg = w.cfg
    KVH, D, PS = cfg["KVH"], cfg["D"], cfg["PS"]
    host_pool, btc = extract_requests(w, bt, rows)
    q_bits = bt.q[rows].cpu().view(torch.int16).numpy().view(np.uint16)
    gk, gv = w.gk.cpu().numpy(), w.gv.cpu().numpy()
    sl = np.array([bt.lens[r] for r in rows], np.int32)
    qsl = np.arange(len(rows) + 1, dtype=np.int32)
    t0 = time.perf_counter()
    out, _ = O.attention(q_bits, host_pool, O.Layout.slots(PS, KVH, D), btc, sl, qsl, KVH, float(D) ** -0.5, gk, gv,
                         float(gv[0]))
    return out, time.perf_counter() - t0, O.num_threads()


def error_record(got, ref, n_req, extra=None):
    import numpy as np
    d = np.abs(got - ref)
    rec = {"max_abs": float(d.max()), "mean_abs": float(d.mean()),
           "rel_l2": float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-300)), "requests": n_req,
           "against": "CPU oracle (fp64 attention over the same cache bytes)",
           "within_tolerance": bool(d.max() <= 2e-2 and d.mean() <= 2e-3)}
    if extra:
        rec.update(extra)
    return rec


def run_reference(args, cfg):
    """the CPU arm: the reference's own PyTorch implementation of the path (kv_fp4_ref.py, byte-compiled into
    oracle/_ref by oracle/build_ref.py) on all host cores when it is there, else the C port of it; each step a bounded
    sample of the default batch: write of the step's new tokens + fp64 attention over the sampled requests' cache.
    The sampled cache is quantised by the oracle's writer beforehand; no GPU is used."""
    import numpy as np
    from oracle import build_ref
    from oracle import kvfp4 as O
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth
    KVH, D, PS, HQ = cfg["KVH"], cfg["D"], cfg["PS"], cfg["HQ"]
    lens_all = draw_lens(cfg, args.seed * 131)
    cores = len(os.sched_getaffinity(0))
    O.set_num_threads(cores)                           # every host core (torchrun would pin OpenMP to one thread)
    # sample: requests in batch order until their contexts add up to --ref-tokens cached tokens
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
    last = np.array([int(c["bt"][b, (L - 1) // PS]) * PS + (L - 1) % PS for b, L in enumerate(lens)], np.int64)
    first_tok = np.cumsum([0] + lens[:-1])
    k_new = c["key"][first_tok + np.array(lens) - 1]
    v_new = c["val"][first_tok + np.array(lens) - 1]
    sm = float(D) ** -0.5
    REF = None if args.ref_port else build_ref.load()
    if REF is not None:
        import torch
        torch.set_num_threads(cores)
        kind = "reference"
        lay = O.Layout.region(PS, KVH, D)               # the page layout of the reference's torch oracle
        cache = np.zeros(c["NP"] * 2 * KVH * PS * (D // 2 + D // 16), np.uint8)
        O.write(c["key"], c["val"], cache, lay, c["slots"], gk, gv, True)
        views = REF.split_views(torch.from_numpy(cache).view(c["NP"], 2 * KVH, PS, D // 2 + D // 16), KVH)
        tb = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)   # noqa: E731
        q_t, k_t, v_t = tb(c["q"]), tb(k_new), tb(v_new)
        gk_t, gv_t = torch.from_numpy(gk), torch.from_numpy(gv)
        bt_t, sl_t, slot_t = torch.from_numpy(c["bt"]), torch.from_numpy(c["seq_lens"]), torch.from_numpy(last)

        def step():
            REF.write_reference(k_t, v_t, views, slot_t, gk_t, gv_t)
            return REF.attention_reference(q_t, views, bt_t, sl_t, 1, sm, gk_t, gv_t, float(gv[0]))
        # the C port and the reference's torch code agree on this sample (fp64 against fp64)
        port, _ = O.attention(c["q"], cache, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, sm, gk, gv, float(gv[0]))
        agree = float(np.abs(step().numpy() - port).max())
    else:
        kind, agree = "port", None
        lay = O.Layout.slots(PS, KVH, D)
        cache = np.zeros(c["NP"] * 2 * KVH * PS * (D // 2 + D // 16), np.uint8)
        O.write(c["key"], c["val"], cache, lay, c["slots"], gk, gv, True)

        def step():
            O.write(k_new, v_new, cache, lay, last, gk, gv, True)
            O.attention(c["q"], cache, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, sm, gk, gv, float(gv[0]))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    # a step of the whole batch at this rate: the sample's time scaled by its share of the batch's cached tokens
    value = cfg["B"] / (dt * sum(lens_all) / sum(lens))
    sample = (f"{len(rows)} of {cfg['B']} requests ({sum(lens)} of {sum(lens_all)} cached tokens) per step; value scaled "
              "to the whole batch by cached tokens")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong" if cfg.get("sharded") else "weak", "vs_baseline": None, "dtype": "f64",
            "data": "synthetic",
            "config": {"workload": args.workload, **{k: cfg[k] for k in ("B", "HQ", "KVH", "D", "PS")},
                       "context": list(cfg["law"]), "sample": sample},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample,
                             "code": ("the reference's kv_fp4_ref.py (write_reference + attention_reference, torch fp64)"
                                      if kind == "reference" else "C port of the reference's kv_fp4_ref.py (OpenMP)")},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if agree is not None:
        line["cpu_baseline"]["max_abs_vs_c_port"] = agree
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=20261125)
    ap.add_argument("--ref-tokens", type=int, default=100000, help="cached tokens per step of the CPU arm's sample")
    ap.add_argument("--ref-port", action="store_true", help="CPU arm: time the C port even when oracle/_ref is there")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the cpu_baseline leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg (parity keeps a small sample)")
    ap.add_argument("--no-extra", action="store_true", help="skip the roofline legs of configurations 1 and 2")
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
    from horizon_kernels_b200 import kernels as K
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"

    # ---- the decode kernel on configurations 1 and 2 (rank 0 only; their pools are freed before the timed workload)
    extra = {}
    if rank == 0 and not args.no_extra:
        for name in ("c1", "c2"):
            if name == args.workload:
                continue
            wx = setup_workload(name, device, args.seed, 0, 1)
            extra["roofline_" + name] = roofline_record(wx, time_decode_kernel(wx, 20, local), peak, peak_src)
            del wx
            torch.cuda.empty_cache()

    w = setup_workload(args.workload, device, args.seed, rank, world, args.shard)
    B, NBT, batches, pool, impl, layer, builder = w.B, w.NBT, w.batches, w.pool, w.impl, w.layer, w.builder
    HQ, KVH, D, PS = cfg["HQ"], cfg["KVH"], cfg["D"], cfg["PS"]
    step, side = w.step, w.side

    # ---- CUDA graphs of one step per batch (the surface allocates nothing and never synchronises)
    graphs = []
    with torch.cuda.stream(side):
        for i in range(NBT):
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
    # the K timed steps as replay units: chains while a whole chain fits, single steps for the rest
    units, i = [], 0
    while i < args.steps:
        if args.steps - i >= CHAIN and i % NBT == 0:
            units.append((chain_graph, CHAIN))
            i += CHAIN
        else:
            units.append((graphs[i % NBT], 1))
            i += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with sampler:
        # the GPU is kept under the same load before and after the timed steps so that the 20 ms clock samples see it,
        # and long enough before them for the clocks to settle where the power cap leaves them (they sink for a second
        # or two after a cold start: timed too early, the steps would look faster than the kernel timed after them)
        # Ranks reach this point seconds apart (rank 0 timed configurations 1 and 2, the communicator comes up inside
        # the first collective): the barrier HERE absorbs that wait, so that every rank enters the load below at the
        # same moment and the barrier in front of the timed steps waits for milliseconds of skew, not for an idle gap
        # after which the clocks would boost for the few milliseconds the steps take.
        barrier()
        t_end = time.perf_counter() + 2.0
        i = 0
        while time.perf_counter() < t_end:
            graphs[i % NBT].replay()
            i += 1
        # ---- the decode kernel alone (roofline): one leg before the timed steps and one after them (merged below)
        kt = time_decode_kernel(w, min(args.steps, 20), local, seconds=0.2)
        for i in range(args.warmup):
            graphs[i % NBT].replay()
        barrier()
        n_clk0 = len(sampler.samples)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(units) + 1)]
        ev[0].record()
        for j, (g, _) in enumerate(units):
            g.replay()
            ev[j + 1].record()
        barrier()
        ms_total = ev[0].elapsed_time(ev[-1])
        unit_ms = [ev[j].elapsed_time(ev[j + 1]) / n for j, (_, n) in enumerate(units)]
        clk_steps = sorted(sampler.samples[n_clk0:])                 # SM clock samples of the timed steps alone
        kt = merge_timings(kt, time_decode_kernel(w, min(args.steps, 20), local, seconds=0.1))

        # ---- end to end: host inputs -> one pinned H2D copy -> write + decode (graph) -> D2H of the output.
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
        NPK = max(NBT, 2)                               # two sets of buffers even for a single batch (for the
        pack_bt = [batches[i % NBT] for i in range(NPK)]  # leg that keeps two steps in flight)
        packs = [packed(bt) for bt in pack_bt]
        for pk, bt in zip(packs, pack_bt):
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
        # where an end-to-end step spends its time: device-side durations of the three parts (CUDA events, a second
        # loop, not the timed one) and the host wall time of a step
        parts_ms = {"h2d": [], "device": [], "d2h": [], "host_wall": []}
        for i in range(min(args.steps, 2 * REPEATS)):
            pk = packs[i % NBT]
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            t1 = time.perf_counter()
            e[0].record()
            pk.dev.copy_(pk.host, non_blocking=True)
            e[1].record()
            pk.graph.replay()
            e[2].record()
            pk.out_host.copy_(pk.out_dev, non_blocking=True)
            e[3].record()
            torch.cuda.current_stream().synchronize()
            parts_ms["host_wall"].append((time.perf_counter() - t1) * 1e3)
            for k_, a_, b_ in (("h2d", 0, 1), ("device", 1, 2), ("d2h", 2, 3)):
                parts_ms[k_].append(e[a_].elapsed_time(e[b_]))
        # the same steps with two of them in flight (consecutive steps use different buffers and, where the workload
        # has two batches, different batches, as two micro-batches of a serving engine do): copies in, kernels and copies out on three streams chained by events, the host reading
        # step i - 1's result while step i runs. Reported beside the serial figure, never instead of it.
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(NPK)]
        ev_run = [torch.cuda.Event() for _ in range(NPK)]
        ev_out = [torch.cuda.Event() for _ in range(NPK)]

        def piped(n_steps):
            for i in range(n_steps):
                j = i % NPK
                pk = packs[j]
                with torch.cuda.stream(s_in):
                    if i >= NPK:
                        s_in.wait_event(ev_run[j])           # the kernels of step i - NPK have read this buffer
                    pk.dev.copy_(pk.host, non_blocking=True)
                    ev_in[j].record(s_in)
                with torch.cuda.stream(side):
                    side.wait_event(ev_in[j])
                    if i >= NPK:
                        side.wait_event(ev_out[j])           # step i - NPK's output has left the device buffer
                    pk.graph.replay()
                    ev_run[j].record(side)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_run[j])
                    pk.out_host.copy_(pk.out_dev, non_blocking=True)
                    ev_out[j].record(s_out)
                if i >= 1:
                    ev_out[(i - 1) % NPK].synchronize()      # the caller reads the previous step's result
            ev_out[(n_steps - 1) % NPK].synchronize()
        piped(args.warmup)
        barrier()
        t0 = time.perf_counter()
        piped(args.steps)
        barrier()
        piped_s = time.perf_counter() - t0
        t_end = time.perf_counter() + 0.3
        i = 0
        while time.perf_counter() < t_end:
            graphs[i % NBT].replay()
            i += 1
        torch.cuda.synchronize()
    clocks = sampler.summary()

    # ---- max over ranks
    times = torch.tensor([ms_total, e2e_s * 1e3, kt["back_to_back_ms"]["median"], (piped_s or 0.0) * 1e3],
                         dtype=torch.float64, device=device)
    times_max = times.clone()
    if world > 1:
        dist.all_reduce(times_max, op=dist.ReduceOp.MAX)
    ms_total_max, e2e_ms, dec_ms_max, piped_ms = (float(x) for x in times_max.cpu())
    ms_step = ms_total_max / args.steps
    n_req = (B if args.shard else cfg["B"]) if cfg.get("sharded") else B * world   # requests of the whole job per step
    value = n_req / (ms_step * 1e-3)
    e2e_value = n_req / (e2e_ms / args.steps * 1e-3)

    # ---- validation. Every rank runs one more step, then the CPU oracle on three of ITS requests (shortest, median,
    # longest context) over their own cache pages; the GPU outputs of all ranks are gathered with NCCL (the only
    # collective) into request order, and rank 0 compares the gathered rows of every rank's sample with that rank's
    # oracle rows. A wrong partition, gather index or block-table row shows up as an error of order one.
    for i in range(NBT):
        step(i)
    torch.cuda.synchronize()
    status = K.workspace_status(impl._state(device)["ws"])
    bt0 = batches[0]
    order = sorted(range(B), key=lambda r: bt0.lens[r])
    mine = sorted({order[0], order[len(order) // 2], order[-1]}) if B else []
    cores = len(os.sched_getaffinity(0))
    ref_rows, _, _ = oracle_rows(w, bt0, mine, max(1, cores // world))
    gids = [(w.rows[r] if w.rows is not None else rank * B + r) for r in mine]       # request ids of the whole job
    # the end-to-end path (host buffers) and the device-resident path compute the same step: bit-identical outputs
    e2e_equal = bool(torch.equal(packs[0].out_host, bt0.out.cpu()))
    if world > 1:
        from horizon_kernels_b200.sharding import gather_outputs
        n_total = cfg["B"] if cfg.get("sharded") else B * world
        full = gather_outputs(bt0.out, w.rows if w.rows is not None else list(range(rank * B, rank * B + B)), n_total)
        ref_t = torch.zeros((3, HQ, D), dtype=torch.float64, device=device)
        gid_t = torch.full((3,), -1, dtype=torch.int64, device=device)
        ref_t[:len(mine)] = torch.from_numpy(ref_rows).to(device)
        gid_t[:len(mine)] = torch.tensor(gids, device=device)
        refs = [torch.empty_like(ref_t) for _ in range(world)]
        ids = [torch.empty_like(gid_t) for _ in range(world)]
        dist.all_gather(refs, ref_t)
        dist.all_gather(ids, gid_t)
        st = torch.tensor([status, int(e2e_equal)], device=device)
        dist.all_reduce(st, op=dist.ReduceOp.MIN)
        status, e2e_equal = int(st[0]), bool(int(st[1]))
        finite = bool(torch.isfinite(full.float()).all()) and full.shape[0] == n_total
        all_ids = torch.cat(ids)
        keep = all_ids >= 0
        got_s = full[all_ids[keep]].double().cpu().numpy()
        ref_s = torch.cat(refs)[keep].cpu().numpy()
        per_rank = [int((i_ >= 0).sum()) for i_ in ids]
    else:
        finite = bool(torch.isfinite(bt0.out.float()).all())
        got_s = bt0.out[mine].double().cpu().numpy()
        ref_s, per_rank = ref_rows, [len(mine)]

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    roof = roofline_record(w, kt, peak, peak_src)
    if world > 1:                                        # the slowest rank's kernel time next to rank 0's
        roof["kernel_ms_max_over_ranks"] = dec_ms_max
    alg = roof["algorithmic_bytes_per_launch"]
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if cfg.get("sharded") else "weak",
            "vs_baseline": None, "dtype": "f16 mma over e2m1 x e4m3 dequantised values, fp32 softmax and accumulation",
            "data": "synthetic",
            "config": {"workload": args.workload, **{k: cfg[k] for k in ("B", "HQ", "KVH", "D", "PS")},
                       "context": list(cfg["law"]), "pool_pages": int(pool.shape[0]), "per_gpu_batch": B,
                       "parallelism": (f"requests sharded over {world} GPU(s) by cached tokens, no collective on the "
                                       "timed path") if cfg.get("sharded") else f"{world} independent replica(s)",
                       "step": "quantize-on-write of 1 new token per request + paged split-K decode (split sequences "
                               "merged inside the launch), one layer",
                       "l2": ("two batches on disjoint pages alternate, each reads more cache bytes than the L2 holds"
                              if NBT > 1 else "one batch whose cache reads per GPU exceed the L2 several times"),
                       "timing": ("CUDA graphs of the plugin calls (5 steps per batch chained in one graph, like the layers "
                                  "of a model), CUDA events around the K steps, max over ranks; roofline: decode launches "
                                  f"back to back in one graph, CUDA events around a replay, median of 2 x {REPEATS} replays, half of them "
                                  "before and half after the timed steps"),
                       "clocks": "NVML sampled every 20 ms while the same step loops before, during and after the timed steps"},
            "tokens_per_s_per_gpu": value / world,
            "step_samples": {"ms_per_step": stats(unit_ms), "unit": "replay units of the timed region on rank 0",
                             "sm_mhz": clk_steps[len(clk_steps) // 2] if clk_steps else None},
            "roofline": roof, **extra,
            "step_hbm_gbs": alg / (ms_step * 1e-3) / 1e9,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "parts_ms_rank0": {k_: stats(v_)["median"] for k_, v_ in parts_ms.items()},
                    "two_steps_in_flight": {
                        "value": n_req / (piped_ms / args.steps * 1e-3), "unit": "tokens/s",
                        "ms_per_step": piped_ms / args.steps,
                        "how": "consecutive steps use different buffers; copies in, kernels and copies out on three "
                               "streams, the host reads step i - 1's output while step i runs; every step still "
                               "copies its inputs from pinned memory and its output back"}},
            "gpu_launches": 2 * args.steps, "clocks": clocks, "device_status": status, "outputs_finite": finite,
            "e2e_output_equal": e2e_equal,
            "parity": error_record(got_s, ref_s, int(sum(per_rank)), {"requests_per_rank": per_rank,
                                   "sample": "shortest, median and longest context of every rank, through the NCCL gather"
                                   if world > 1 else "shortest, median and longest context"})}

    if world == 1 and not args.no_cpu:
        # ---- CPU baseline on a bounded sample of batch 0 (the oracle is the checker, never the product): requests in
        # batch order until the budget; the whole batch's rate follows from the sample's share of the cached tokens
        _, t1, cores_used = oracle_rows(w, bt0, order[:1], cores)
        rate = bt0.lens[order[0]] / max(t1, 1e-6)                        # cached tokens per second, first estimate
        rows, tok = [], 0
        for r in range(B):
            if (tok + bt0.lens[r] > rate * args.cpu_seconds or len(rows) >= 512) and rows:
                break
            rows.append(r)
            tok += bt0.lens[r]
        ref, secs, cores_used = oracle_rows(w, bt0, rows, cores)
        got = bt0.out[rows].double().cpu().numpy()
        total_tok = sum(bt0.lens)
        line["cpu_baseline"] = {"value": B / (secs * total_tok / tok), "unit": "tokens/s", "cores": cores_used,
                                "kind": "port",
                                "sample": f"{len(rows)} of {B} requests of the same batch ({tok} of {total_tok} cached "
                                          f"tokens), decode only, {secs:.1f} s; scaled to the batch by cached tokens"}
        line["parity_cpu_sample"] = error_record(got, ref, len(rows))
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
