"""Stand-alone timings of the two kernels beside the decode path: quantize-on-write at prefill size and the exact
dequantisation, each on synthetic data, timed with CUDA events. `bench.py` at the repository root measures the decode
step; this module is what the ncu summaries of the other kernels are captured from.

    python -m horizon_kernels_b200.microbench write   [--tokens 32768] [--kvh 8] [--d 128] [--iters 10]
    python -m horizon_kernels_b200.microbench dequant [--tokens 262144] [--kvh 8] [--d 128] [--iters 10] [--f16]
"""
import argparse
import json

import torch

from . import kernels as K
from . import layout as Lt


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def write(a):
    NT, KVH, D, PS = a.tokens, a.kvh, a.d, 16
    g = torch.Generator(device="cuda").manual_seed(1)
    k = torch.randn(NT, KVH, D, generator=g, device="cuda")
    k[:, :, [3, D // 4 + 3, D // 2 + 3, 3 * D // 4 + 3]] *= 20
    k = k.to(torch.bfloat16)
    v = torch.randn(NT, KVH, D, generator=g, device="cuda").to(torch.bfloat16)
    NP = NT // PS + 8
    pool = torch.zeros((NP, 2 * KVH, PS, Lt.slot_bytes(D)), dtype=torch.uint8, device="cuda")
    flat, st = Lt.flat_views(*Lt.slot_views(pool, KVH, D))
    slots = torch.randperm(NP * PS, generator=g, device="cuda")[:NT]
    # the per-tensor scale of the benchmark configuration: amax / (6 * 448), which puts many quotients on a rounding
    # boundary of the 4-bit grid
    gk = torch.full((KVH,), float(k.float().abs().max()) / (6 * 448), device="cuda")
    gv = torch.full((KVH,), float(v.float().abs().max()) / (6 * 448), device="cuda")
    byts = NT * KVH * D * (4 + 1.125) + 8 * NT
    for search in (True, False):
        ms = _time(lambda: K.write(k, v, flat, st, PS, slots, gk, gv, search), a.iters)
        print(json.dumps({"kernel": "write", "tokens": NT, "kv_heads": KVH, "head_dim": D, "search": search,
                          "us": ms * 1e3, "algorithmic_gbs": byts / ms / 1e6}))


def dequant(a):
    NT, KVH, D, PS = a.tokens, a.kvh, a.d, 16
    NP = NT // PS
    pool = torch.randint(0, 120, (NP, 2 * KVH, PS, Lt.slot_bytes(D)), dtype=torch.uint8, device="cuda")
    flat, st = Lt.flat_views(*Lt.slot_views(pool, KVH, D))
    bt = torch.randperm(NP, device="cuda").to(torch.int32)
    dt = torch.float16 if a.f16 else torch.bfloat16
    ok = torch.empty((NT, KVH, D), dtype=dt, device="cuda")
    ov = torch.empty_like(ok)
    ms = _time(lambda: K.dequant_tokens(flat, st, PS, bt, 0, NT, ok, ov), a.iters)
    byts = NT * KVH * D * 2 * (0.5625 + 2)
    print(json.dumps({"kernel": "dequant", "tokens": NT, "kv_heads": KVH, "head_dim": D, "dtype": str(dt),
                      "us": ms * 1e3, "algorithmic_gbs": byts / ms / 1e6}))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["write", "dequant"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--kvh", type=int, default=8)
    ap.add_argument("--d", type=int, default=128, choices=[128, 256])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--f16", action="store_true")
    a = ap.parse_args()
    if a.tokens is None:
        a.tokens = 32768 if a.kernel == "write" else 262144
    {"write": write, "dequant": dequant}[a.kernel](a)


if __name__ == "__main__":
    main()
