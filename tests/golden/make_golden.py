"""Generates the golden fixtures in this folder by RUNNING THE REFERENCE'S OWN PyTorch implementation of the NVFP4
KV-cache path (nvidia-sm120/horizon_kvfp4/kernels/kv_fp4_ref.py in the reference tree, imported by file path, never
copied) on the deterministic inputs of tests/synth.py.

usage: python tests/golden/make_golden.py <reference_root>

The fixtures pin the CPU oracle (oracle/) and, through it, the CUDA kernels:
  quant.npz      quantize_rows: random / outlier / edge rows, D 128 and 256, several global scales, search on and off
  write.npz      write_reference into garbage-filled caches: region layout (split_views) and the serving slot layout
                 (heads-outer and positions-outer), 10 % skipped slots, non-unit per-head scales
  attention.npz  attention_reference (fp64) for small paged cases incl. partial pages, a 1-token and a 0-token
                 context, GQA 4 / 8 / 6, head_dim 128 / 256, page 16 / 64, 1 and 4 query tokens per request
  config0.npz    the full "batch 4, 32/8 heads, head_dim 128, 2048 tokens, 512 pages" case: sha256 of the cache the
                 reference wrote and its fp64 attention output (inputs regenerate from the seed)
"""
import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import synth  # noqa: E402


def load_ref(root):
    p = os.path.join(root, "nvidia-sm120", "horizon_kvfp4", "kernels", "kv_fp4_ref.py")
    spec = importlib.util.spec_from_file_location("kv_fp4_ref", p)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def slot_views(cache, KVH, D):
    """the serving layout's four [page, pos, head, byte] views of a logical (pages, 2 KVH, PS, slot) cache, as the
    reference's backend builds them (backend.py:286-296)"""
    t = cache.permute(0, 2, 1, 3)
    dd = D // 2
    return t[:, :, :KVH, :dd], t[:, :, :KVH, dd:], t[:, :, KVH:, :dd], t[:, :, KVH:, dd:]


def quant_rows(R):
    out = {}
    for D in (128, 256):
        n = 48
        x = synth.normal(100 + D, (n, D)) * np.exp(synth.normal(200 + D, (n, 1)))
        xo = synth.normal(300 + D, (16, D))
        xo[:, [3, D // 4 + 3, D // 2 + 3, 3 * D // 4 + 3]] *= 20.0
        e = synth.normal(400 + D, (12, D))
        e[0] = 0.0
        e[1] *= 1e-30
        e[2] *= 1e30
        e[3, :16] = 300.0
        e[4, ::2] = -0.0
        e[5] = np.tile(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0,
                                 -6.0]), D // 16)
        e[6] = e[5] * 0.125
        e[7, 5] = -3.0
        e[7, :5] = 0
        e[7, 6:] = 0
        e[8] = 448.0 * 6.0
        e[9] = 1e-3
        x = synth.bf16_bits_to_f32(synth.to_bf16_bits(np.concatenate([x, xo, e])))
        xt = torch.from_numpy(x.copy())
        amax_g = float(np.float32(np.abs(x[:64]).max()) / np.float32(6 * 448))
        gs = [1.0, 0.5, 0.37, amax_g]
        out[f"x{D}"] = x
        out[f"g{D}"] = np.array(gs, np.float32)
        for gi, g in enumerate(gs):
            for search in (0, 1):
                d, s = R.quantize_rows(xt, float(np.float32(g)), bool(search))
                out[f"data{D}_g{gi}_s{search}"] = d.numpy()
                out[f"sf{D}_g{gi}_s{search}"] = s.numpy()
        gr = torch.from_numpy(np.float32(np.exp(synth.normal(500 + D, (x.shape[0],)))))
        d, s = R.quantize_rows(xt, gr, True)
        out[f"grow{D}"] = gr.numpy()
        out[f"data{D}_grow"] = d.numpy()
        out[f"sf{D}_grow"] = s.numpy()
    return out


def write_cases(R):
    out = {}
    for name, KVH, D, PS, NT in (("a", 2, 128, 16, 100), ("b", 4, 256, 64, 70)):
        NP = (NT + PS - 1) // PS + 4
        k = synth.normal(610 + D, (NT, KVH, D)) * 2.0
        k[:, :, [3, D // 2 + 3]] *= 20.0
        v = synth.normal(620 + D, (NT, KVH, D)) * np.exp(0.5 * synth.normal(630 + D, (NT, 1, 1)))
        k[0] = 0
        v[1] = 0
        kb, vb = synth.to_bf16_bits(k), synth.to_bf16_bits(v)
        slots = synth.permutation(640 + D, NP * PS)[:NT].astype(np.int64)
        slots[synth.uniform(650 + D, NT) < 0.1] = -1
        gk = np.array([1.0, 0.5, 2.0, 1.0][:KVH], np.float32)
        gv = np.array([2.0, 0.25, 1.0, 4.0][:KVH], np.float32)
        out.update({f"{name}_key": kb, f"{name}_val": vb, f"{name}_slots": slots, f"{name}_gk": gk, f"{name}_gv": gv,
                    f"{name}_geom": np.array([KVH, D, PS, NP], np.int64)})
        for search in (0, 1):
            c = R.alloc_cache(NP, PS, KVH, D, fill=0xA5)
            R.write_reference(bf16(kb), bf16(vb), R.split_views(c, KVH), torch.from_numpy(slots),
                              torch.from_numpy(gk), torch.from_numpy(gv), None, bool(search))
            out[f"{name}_region_s{search}"] = c.numpy().reshape(-1)
            slot = D // 2 + D // 16
            for lay in ("hnd", "nhd"):
                if lay == "hnd":
                    phys = torch.full((NP, 2 * KVH, PS, slot), 0xA5, dtype=torch.uint8)
                    logical = phys
                else:
                    phys = torch.full((NP, PS, 2 * KVH, slot), 0xA5, dtype=torch.uint8)
                    logical = phys.permute(0, 2, 1, 3)
                R.write_reference(bf16(kb), bf16(vb), slot_views(logical, KVH, D), torch.from_numpy(slots),
                                  torch.from_numpy(gk), torch.from_numpy(gv), None, bool(search))
                out[f"{name}_{lay}_s{search}"] = phys.numpy().reshape(-1)
    return out


def attention_cases(R):
    out = {}
    cases = (("g4", dict(lens=[1, 17, 37, 150, 16, 0], KVH=2, G=4, D=128, PS=16, QL=1), 0x7F),
             ("g8", dict(lens=[5, 64, 200], KVH=2, G=8, D=256, PS=16, QL=1), 0x7F),
             ("g6", dict(lens=[5, 300, 129], KVH=4, G=6, D=256, PS=64, QL=4), 0xAA))
    for i, (name, kw, fill) in enumerate(cases):
        c = synth.paged_case(700 + i, outliers=True, **kw)
        KVH, G, D, PS, QL = kw["KVH"], kw["G"], kw["D"], kw["PS"], kw["QL"]
        gk = np.array([0.5, 2.0, 1.0, 0.25][:KVH], np.float32) * np.float32(0.05)
        gv = np.array([2.0, 0.5, 1.0, 4.0][:KVH], np.float32) * np.float32(0.01)
        cache = R.alloc_cache(c["NP"], PS, KVH, D, fill=fill)
        views = R.split_views(cache, KVH)
        R.write_reference(bf16(c["key"]), bf16(c["val"]), views, torch.from_numpy(c["slots"]), torch.from_numpy(gk),
                          torch.from_numpy(gv), None, True)
        sm = float(D) ** -0.5
        ref = R.attention_reference(bf16(c["q"]), views, torch.from_numpy(c["bt"]), torch.from_numpy(c["seq_lens"]),
                                    QL, sm, torch.from_numpy(gk), torch.from_numpy(gv), v_scale=0.5)
        out.update({f"{name}_cache": cache.numpy().reshape(-1), f"{name}_q": c["q"], f"{name}_bt": c["bt"],
                    f"{name}_seq_lens": c["seq_lens"], f"{name}_qsl": c["qsl"], f"{name}_gk": gk, f"{name}_gv": gv,
                    f"{name}_geom": np.array([KVH, G, D, PS, QL, c["NP"]], np.int64),
                    f"{name}_sm": np.array([sm, 0.5]), f"{name}_ref": ref.numpy()})
    return out


def config0(R):
    """benchmark configuration 0: batch 4, 32 q heads / 8 kv heads, head_dim 128, 2048 cached tokens each, page 16, page table
    a permutation of 512 pages, q / k / v ~ N(0,1) bf16, scale 1/sqrt(128), per-tensor global scale amax/(6*448)."""
    B, KVH, G, D, PS, L = 4, 8, 4, 128, 16, 2048
    c = synth.paged_case(900, [L] * B, KVH, G, D, PS, extra_pages=1)   # its page table is replaced below
    perm = synth.permutation(901, 512).astype(np.int32)          # all 512 pages, page 0 included
    bt = perm.reshape(B, 128)
    slots = np.array([int(bt[b, p // PS]) * PS + p % PS for b in range(B) for p in range(L)], np.int64)
    gk = np.full(KVH, synth.tensor_scale(c["key"]), np.float32)
    gv = np.full(KVH, synth.tensor_scale(c["val"]), np.float32)
    cache = R.alloc_cache(512, PS, KVH, D, fill=0)
    views = R.split_views(cache, KVH)
    R.write_reference(bf16(c["key"]), bf16(c["val"]), views, torch.from_numpy(slots), torch.from_numpy(gk),
                      torch.from_numpy(gv), None, True)
    sm = float(D) ** -0.5
    ref = R.attention_reference(bf16(c["q"]), views, torch.from_numpy(bt), torch.from_numpy(c["seq_lens"]), 1, sm,
                                torch.from_numpy(gk), torch.from_numpy(gv))
    sha = hashlib.sha256(cache.numpy().tobytes()).hexdigest()
    return dict(bt=bt, gk=gk, gv=gv, ref=ref.numpy(), cache_sha256=np.array(sha), sm=np.array([sm]))


def rotation_cases(R):
    """the optional key rotation: the reference's sign vectors, rotate() of bf16 rows in fp32, rotate_q() (one rounding
    to bf16), and caches written with rotated keys (region layout, search on and off)"""
    out = {}
    for D in (128, 256):
        signs = R.hadamard_signs(D)
        x = synth.normal(700 + D, (24, D)) * np.exp(synth.normal(710 + D, (24, 1)))
        x[0] = 0.0
        x[1, 5] = 1e4
        xb = synth.to_bf16_bits(x)
        out[f"signs{D}"] = signs.numpy()
        out[f"x{D}"] = xb
        out[f"rot{D}"] = R.rotate(bf16(xb), signs).numpy()
        out[f"rotq{D}"] = R.rotate_q(bf16(xb), signs).view(torch.int16).numpy().view(np.uint16)
        out[f"scale{D}"] = np.array([R.fwht_scale(D)], np.float32)
        KVH, PS, NT = 2, 16, 50
        NP = (NT + PS - 1) // PS + 2
        k = synth.normal(720 + D, (NT, KVH, D)) * 2.0
        k[:, :, [3, D // 2 + 3]] *= 20.0
        v = synth.normal(730 + D, (NT, KVH, D))
        kb, vb = synth.to_bf16_bits(k), synth.to_bf16_bits(v)
        slots = synth.permutation(740 + D, NP * PS)[:NT].astype(np.int64)
        gk = np.array([0.05, 0.02], np.float32)
        gv = np.array([0.01, 0.03], np.float32)
        out.update({f"w{D}_key": kb, f"w{D}_val": vb, f"w{D}_slots": slots, f"w{D}_gk": gk, f"w{D}_gv": gv,
                    f"w{D}_geom": np.array([KVH, D, PS, NP], np.int64)})
        for search in (0, 1):
            c = R.alloc_cache(NP, PS, KVH, D, fill=0xA5)
            R.write_reference(bf16(kb), bf16(vb), R.split_views(c, KVH), torch.from_numpy(slots),
                              torch.from_numpy(gk), torch.from_numpy(gv), signs, bool(search))
            out[f"w{D}_region_s{search}"] = c.numpy().reshape(-1)
    return out


def k8_cases(R):
    """the K8V4 slot (FP8 keys + FP4 values, 400 bytes at head_dim 256): write_reference_k8's cache bytes and fp64
    attention over gather_k8's dequantised keys and values (the arithmetic of attention_reference)"""
    KVH, G, D, PS = 2, 4, 256, 16
    lens = [70, 16, 301]
    c = synth.paged_case(800, lens, KVH, G, D, PS, outliers=True, ql_list=[1, 2, 1])
    NP = c["NP"]
    gk = np.array([0.05, 0.11], np.float32)
    gv = np.array([0.01, 0.02], np.float32)
    out = {"geom": np.array([KVH, G, D, PS, NP], np.int64), "gk": gk, "gv": gv}
    out.update({k: c[k] for k in ("key", "val", "q", "bt", "slots", "seq_lens", "qsl")})
    sm = D ** -0.5
    for search in (0, 1):
        cache = torch.full((NP, KVH, PS, R.K8_SLOT), 0xA5, dtype=torch.uint8)
        views = R.split_views_k8(cache)
        R.write_reference_k8(bf16(c["key"]), bf16(c["val"]), views, torch.from_numpy(c["slots"]),
                             torch.from_numpy(gk), torch.from_numpy(gv), bool(search))
        out[f"cache_s{search}"] = cache.numpy().reshape(-1)
    q = bf16(c["q"]).double()
    ref = torch.zeros(q.shape, dtype=torch.float64)
    gk64, gv64 = torch.from_numpy(gk).double().view(KVH, 1, 1), torch.from_numpy(gv).double().view(1, KVH, 1)
    for b, L in enumerate(lens):
        K_, V_ = R.gather_k8(views, torch.from_numpy(c["bt"][b]), L)
        q0, q1 = int(c["qsl"][b]), int(c["qsl"][b + 1])
        for t in range(q1 - q0):
            lim = L - (q1 - q0) + t + 1
            qq = q[q0 + t].view(KVH, G, D)
            s_ = torch.einsum("hgd,lhd->hgl", qq, K_[:lim]) * gk64 * sm
            p_ = torch.softmax(s_, dim=-1)
            ref[q0 + t] = torch.einsum("hgl,lhd->hgd", p_, V_[:lim] * gv64).reshape(KVH * G, D)
    out["ref"] = ref.numpy()
    return out


def main():
    root = sys.argv[1]
    R = load_ref(root)
    torch.set_num_threads(8)
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **quant_rows(R))
    np.savez_compressed(os.path.join(HERE, "write.npz"), **write_cases(R))
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **attention_cases(R))
    np.savez_compressed(os.path.join(HERE, "config0.npz"), **config0(R))
    np.savez_compressed(os.path.join(HERE, "rotation.npz"), **rotation_cases(R))
    np.savez_compressed(os.path.join(HERE, "k8v4.npz"), **k8_cases(R))
    for f in ("quant.npz", "write.npz", "attention.npz", "config0.npz", "rotation.npz", "k8v4.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
