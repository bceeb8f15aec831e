"""Stand-alone timings of single kernels on synthetic data, timed with CUDA events: quantize-on-write at prefill size,
the exact dequantisation, and the decode kernel in the variants the benchmark's default workloads do not reach (head
dimension 256, the FP8-key slot, rotated keys). `bench.py` at the repository root measures the decode step; this
module is what the ncu summaries of the other kernels and variants are captured from.

    python -m horizon_kernels_b200.microbench write   [--tokens 32768] [--kvh 8] [--d 128] [--iters 10] [--had] [--k8]
    python -m horizon_kernels_b200.microbench dequant [--tokens 262144] [--kvh 8] [--d 128] [--iters 10] [--f16]
    python -m horizon_kernels_b200.microbench pipes
    python -m horizon_kernels_b200.microbench decode  [--batch 192] [--kvh 2] [--g 8] [--d 256] [--min-len 128]
                                                      [--max-len 32768] [--iters 10] [--had] [--k8] [--nhd] [--ql 1]
"""
import argparse
import json
import math

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


def _pool(NP, KVH, D, PS, k8, nhd=False):
    """an empty page pool in the FP4 slot layout (pages head-major, or positions outermost with nhd) or the FP8-key slot
    layout: flat views, strides and the tensor"""
    if nhd:
        pool = torch.zeros((NP, PS, 2 * KVH, Lt.slot_bytes(D)), dtype=torch.uint8, device="cuda")
        flat, st = Lt.flat_views(*Lt.slot_views(pool.permute(0, 2, 1, 3), KVH, D))
        return flat, st, pool
    if k8:
        pool = torch.zeros((NP, KVH, PS, Lt.K8_SLOT), dtype=torch.uint8, device="cuda")
        flat, st = Lt.k8_flat_views(*Lt.k8_views(pool, D))
    else:
        pool = torch.zeros((NP, 2 * KVH, PS, Lt.slot_bytes(D)), dtype=torch.uint8, device="cuda")
        flat, st = Lt.flat_views(*Lt.slot_views(pool, KVH, D))
    return flat, st, pool


def _token_bytes(D, k8):
    """cache bytes of one token and kv head, keys and values together"""
    return Lt.K8_SLOT if k8 else 2 * Lt.slot_bytes(D)


def write(a):
    NT, KVH, D, PS = a.tokens, a.kvh, a.d, 16
    g = torch.Generator(device="cuda").manual_seed(1)
    k = torch.randn(NT, KVH, D, generator=g, device="cuda")
    k[:, :, [3, D // 4 + 3, D // 2 + 3, 3 * D // 4 + 3]] *= 20
    k = k.to(torch.bfloat16)
    v = torch.randn(NT, KVH, D, generator=g, device="cuda").to(torch.bfloat16)
    NP = NT // PS + 8
    flat, st, _ = _pool(NP, KVH, D, PS, a.k8)
    signs = K.hadamard_signs(D, device="cuda") if a.had else None
    slots = torch.randperm(NP * PS, generator=g, device="cuda")[:NT]
    # the per-tensor scale of the benchmark configuration: amax / (6 * 448), which puts many quotients on a rounding
    # boundary of the 4-bit grid
    gk = torch.full((KVH,), float(k.float().abs().max()) / (6 * 448), device="cuda")
    gv = torch.full((KVH,), float(v.float().abs().max()) / (6 * 448), device="cuda")
    byts = NT * KVH * (D * 4 + _token_bytes(D, a.k8)) + 8 * NT
    for search in (True, False):
        ms = _time(lambda: K.write(k, v, flat, st, PS, slots, gk, gv, search, signs=signs, k8=a.k8), a.iters)
        print(json.dumps({"kernel": "write", "tokens": NT, "kv_heads": KVH, "head_dim": D, "search": search,
                          "rotated": a.had, "k8": a.k8, "us": ms * 1e3, "algorithmic_gbs": byts / ms / 1e6}))


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


def decode(a):
    """One decode step over a hybrid batch: context lengths log-uniform in [min-len, max-len], pages scattered over the
    pool, the cache filled by the write kernel. Every iteration reads the whole cache of the batch once; the batch is
    sized by --batch so that this is several times the L2."""
    B, KVH, G, D, PS = a.batch, a.kvh, a.g, a.d, 16
    g = torch.Generator(device="cuda").manual_seed(2)
    u = torch.rand(B, generator=g, device="cuda").cpu()
    lens = [int(round(math.exp(math.log(a.min_len) + float(x) * (math.log(a.max_len) - math.log(a.min_len)))))
            for x in u]
    pages = [(n + PS - 1) // PS for n in lens]
    tot, MP = sum(pages), max(pages)
    NP = tot + tot // 4 + 8
    flat, st, pool = _pool(NP, KVH, D, PS, a.k8, a.nhd)
    signs = K.hadamard_signs(D, device="cuda") if a.had else None
    perm = torch.randperm(NP, generator=g, device="cuda")[:tot]
    bt = torch.zeros((B, MP), dtype=torch.int32, device="cuda")
    o = 0
    for b, n in enumerate(pages):
        bt[b, :n] = perm[o:o + n].to(torch.int32)
        o += n
    gk = torch.full((KVH,), (1.0 if a.k8 else 1 / 6) * 100.0 / 448, device="cuda")
    gv = torch.full((KVH,), 5.0 / (6 * 448), device="cuda")
    CH = 8192                                      # pages filled per write launch
    for i in range(0, tot, CH):
        pg = perm[i:i + CH]
        n = pg.numel() * PS
        k = torch.randn(n, KVH, D, generator=g, device="cuda")
        k[:, :, [3, D // 4 + 3, D // 2 + 3, 3 * D // 4 + 3]] *= 20
        v = torch.randn(n, KVH, D, generator=g, device="cuda")
        sl = (pg[:, None] * PS + torch.arange(PS, device="cuda")[None, :]).reshape(-1)
        K.write(k.to(torch.bfloat16), v.to(torch.bfloat16), flat, st, PS, sl, gk, gv, False, signs=signs, k8=a.k8)
    ql = a.ql                                      # query tokens per request (1 + draft tokens), causal among themselves
    q = torch.randn(B * ql, KVH * G, D, generator=g, device="cuda").to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qsl = torch.arange(B + 1, dtype=torch.int32, device="cuda") * ql
    out = torch.empty_like(q)
    ws = K.alloc_workspace(B, KVH, G, D, ql, "cuda")
    ms = _time(lambda: K.decode_ragged(q, flat, st, PS, bt, sl, qsl, D ** -0.5, 1.0, gk, gv, ql, out, ws, signs=signs,
                                       k8=a.k8), a.iters)
    if K.workspace_status(ws) != 0 or not bool(torch.isfinite(out.float()).all()):
        raise RuntimeError("decode reported a wait that ran out, or a non-finite output")
    byts = sum(lens) * KVH * _token_bytes(D, a.k8)
    print(json.dumps({"kernel": "decode", "batch": B, "kv_heads": KVH, "group": G, "head_dim": D,
                      "rotated": a.had, "k8": a.k8, "positions_outermost_pages": a.nhd, "query_tokens": ql,
                      "query_rows_per_kv_head": G * ql, "cached_tokens": sum(lens), "cache_mb": byts / 1e6,
                      "us": ms * 1e3, "algorithmic_gbs": byts / ms / 1e6}))


def pipes(a):
    """cycles per warp instruction and SM sub-partition for the instruction kinds of the decode and write kernels
    (hkv_probe_issue_rates in include/hkv.h), at 1, 3 and 4 warps per sub-partition"""
    import ctypes as C
    from . import _lib
    names = ["cvt.rn.f16x2.e2m1x2", "mul.f16x2", "fma.f32", "lop3", "4 cvt + 4 mul.f16x2", "4 cvt + 4 mul + 1 add",
             "4 cvt + 4 mul + 1 add + mma.m16n8k16", "mul.f32", "mul.f32x2", "cvt.rn.satfinite.e2m1x2.f32",
             "cvt.f32.f16", "prmt"]
    per_rep = [8, 8, 8, 8, 8, 9, 10, 8, 8, 8, 8, 8]
    M = len(names)
    nbytes = M * 256 * 8 + 256 * 1024 * 4
    buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for wps in (1, 3, 4):
        _lib.check(_lib.load().hkv_probe_issue_rates(C.c_void_p(buf.data_ptr()), nbytes, wps,
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream)), "hkv_probe_issue_rates")
        torch.cuda.synchronize()
        cyc = buf[:M * 256 * 8].view(torch.int64).view(M, 256)[:, :sms].double().mean(dim=1).cpu().tolist()
        print(json.dumps({"kernel": "pipes", "warps_per_subpartition": wps, "cycles_per_warp_instruction": {
            n: round(c / (2048 * k * wps), 3) for n, c, k in zip(names, cyc, per_rep)},
            "cycles_per_repetition": {n: round(c / (2048 * wps), 2) for n, c in zip(names[4:7], cyc[4:7])}}))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["write", "dequant", "decode", "pipes"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--kvh", type=int, default=None)
    ap.add_argument("--d", type=int, default=None, choices=[128, 256])
    ap.add_argument("--batch", type=int, default=192)
    ap.add_argument("--g", type=int, default=8)
    ap.add_argument("--min-len", type=int, default=128)
    ap.add_argument("--max-len", type=int, default=32768)
    ap.add_argument("--had", action="store_true", help="rotated keys (sign flips + Hadamard transform)")
    ap.add_argument("--k8", action="store_true", help="the FP8-key slot (head_dim 256)")
    ap.add_argument("--ql", type=int, default=1, help="decode: query tokens per request (group x ql rows per kv head)")
    ap.add_argument("--nhd", action="store_true", help="decode: pages with positions outermost (row-copy path)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--f16", action="store_true")
    a = ap.parse_args()
    if a.tokens is None:
        a.tokens = 32768 if a.kernel == "write" else 262144
    if a.kvh is None:
        a.kvh = 2 if a.kernel == "decode" else 8
    if a.d is None:
        a.d = 256 if (a.kernel == "decode" or a.k8) else 128
    {"write": write, "dequant": dequant, "decode": decode, "pipes": pipes}[a.kernel](a)


if __name__ == "__main__":
    main()
