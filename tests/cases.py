"""Helpers shared by the GPU parity tests: turn a synthetic paged case (tests/synth.py) into device tensors, run the
CUDA kernels through the host wrappers (which call the C ABI), and run the CPU oracle on the same bytes."""
import numpy as np
import torch

import synth
from horizon_kernels_b200 import kernels as K
from horizon_kernels_b200 import layout as Lt
from oracle import kvfp4 as O


def bf16_tensor(bits: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


class Cache:
    """a device cache in one of the three byte placements, with the views the kernels and the oracle need"""

    def __init__(self, NP, PS, KVH, D, kind="hnd", fill=0, device="cuda"):
        self.NP, self.PS, self.KVH, self.D, self.kind = NP, PS, KVH, D, kind
        slot = Lt.slot_bytes(D)
        if kind == "region":
            self.phys = Lt.alloc_cache(NP, PS, KVH, D, device=device, fill=fill)
            views = Lt.split_views(self.phys, KVH)
            self.olay = O.Layout.region(PS, KVH, D)
        elif kind == "hnd":
            self.phys = torch.full((NP, 2 * KVH, PS, slot), fill, dtype=torch.uint8, device=device)
            views = Lt.slot_views(self.phys, KVH, D)
            self.olay = O.Layout.slots(PS, KVH, D)
        elif kind == "nhd":
            self.phys = torch.full((NP, PS, 2 * KVH, slot), fill, dtype=torch.uint8, device=device)
            views = Lt.slot_views(self.phys.permute(0, 2, 1, 3), KVH, D)
            self.olay = O.Layout.slots(PS, KVH, D, nhd=True)
        else:
            raise ValueError(kind)
        self.flat, self.strides = Lt.flat_views(*views)
        assert tuple(self.strides) == tuple(self.olay.strides()), (self.strides, self.olay.strides())

    def bytes(self) -> np.ndarray:
        return self.phys.detach().cpu().numpy().reshape(-1)

    def load(self, b: np.ndarray):
        self.phys.copy_(torch.from_numpy(b.reshape(self.phys.shape)).to(self.phys.device))


def gpu_write(cache: Cache, key, val, slots, gk, gv, search=True):
    K.write(key, val, cache.flat, cache.strides, cache.PS, slots, gk, gv, search)


def build_decode_case(seed, lens, KVH, G, D, PS, kind="hnd", fill=0x7F, outliers=True, ql_list=None, gscale=None,
                      writer="gpu"):
    """writes the synthetic K / V of a case into a garbage-filled device cache (with the CUDA write kernel, or with the
    oracle when writer == "oracle") and returns everything the decode and the oracle need"""
    c = synth.paged_case(seed, lens, KVH, G, D, PS, outliers=outliers, ql_list=ql_list)
    if gscale is None:
        gk = np.full(KVH, synth.tensor_scale(c["key"]), np.float32)
        gv = np.full(KVH, synth.tensor_scale(c["val"]), np.float32)
    else:
        gk = (np.array([1.0, 0.5, 2.0, 0.25, 1.5, 0.75, 1.25, 3.0][:KVH]) * gscale[0]).astype(np.float32)
        gv = (np.array([2.0, 1.0, 0.5, 4.0, 0.25, 1.5, 3.0, 1.0][:KVH]) * gscale[1]).astype(np.float32)
    cache = Cache(c["NP"], PS, KVH, D, kind, fill)
    dev = cache.phys.device
    if writer == "gpu":
        if c["slots"].size:
            gpu_write(cache, bf16_tensor(c["key"]), bf16_tensor(c["val"]), torch.from_numpy(c["slots"]).to(dev),
                      torch.from_numpy(gk).to(dev), torch.from_numpy(gv).to(dev))
    else:
        host = cache.bytes().copy()
        O.write(c["key"], c["val"], host, cache.olay, c["slots"], gk, gv, True)
        cache.load(host)
    c.update(cache=cache, gk=gk, gv=gv, sm=float(D) ** -0.5)
    return c


def gpu_decode(c, v_scale=1.0, splits=None, out=None, ws=None, qlmax=None):
    cache = c["cache"]
    dev = cache.phys.device
    q = bf16_tensor(c["q"])
    B = len(c["seq_lens"])
    qlmax = int(max(1, (c["qsl"][1:] - c["qsl"][:-1]).max())) if qlmax is None else qlmax
    if out is None:
        out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    if ws is None:
        ws = K.alloc_workspace(B, c["KVH"], c["G"], c["D"], qlmax, dev)
    K.decode_ragged(q, cache.flat, cache.strides, cache.PS, torch.from_numpy(c["bt"]).to(dev),
                    torch.from_numpy(c["seq_lens"]).to(dev), torch.from_numpy(c["qsl"]).to(dev), c["sm"], v_scale,
                    torch.from_numpy(c["gk"]).to(dev), torch.from_numpy(c["gv"]).to(dev), qlmax, out, ws, splits=splits)
    return out, ws


def oracle_decode(c, v_scale=1.0):
    cache = c["cache"]
    out, _ = O.attention(c["q"], cache.bytes(), cache.olay, c["bt"], c["seq_lens"], c["qsl"], c["KVH"], c["sm"],
                         c["gk"], c["gv"], v_scale)
    return out


def errors(got: torch.Tensor, ref: np.ndarray):
    """(max-abs, mean-abs, relative L2) over the rows the oracle wrote"""
    g = got.detach().float().cpu().numpy().astype(np.float64)[:ref.shape[0]]
    m = ~np.isnan(ref)
    d = np.abs(g[m] - ref[m])
    return float(d.max()), float(d.mean()), float(np.linalg.norm(g[m] - ref[m]) / max(np.linalg.norm(ref[m]), 1e-300))


# the tolerances of the task statement, against the reference's dequantise-then-attend result over the same cache
MAX_ABS, MEAN_ABS, REL_L2 = 2e-2, 2e-3, 2.5e-3


def assert_close(got, ref, what=""):
    assert torch.isfinite(got[:ref.shape[0]].float().cpu()[torch.from_numpy(~np.isnan(ref))]).all(), what
    mx, mn, rl = errors(got, ref)
    assert mx <= MAX_ABS and mn <= MEAN_ABS and rl <= REL_L2, (what, mx, mn, rl)
    return mx, mn, rl


def unquantised_attention(c, sm=None):
    """fp64 attention over the UNQUANTISED bf16 keys and values of a synth.paged_case (the "float64 oracle" column of
    the reference's GPU gates, scripts/kernels/kvfp4/test_kvfp4_gpu.py:204-218): what the model would compute without a
    4-bit cache. Token t of a request with ql query tokens and L cached tokens sees keys j < L - ql + t + 1."""
    KVH, G, D = c["KVH"], c["G"], c["D"]
    sm = D ** -0.5 if sm is None else sm
    key, val, q = (O.bf16_to_f32(c[n]).astype(np.float64) for n in ("key", "val", "q"))
    out = np.full(q.shape, np.nan)
    t0 = 0
    for b, L in enumerate(int(x) for x in c["seq_lens"]):
        kb, vb = key[t0:t0 + L], val[t0:t0 + L]
        t0 += L
        q0, q1 = int(c["qsl"][b]), int(c["qsl"][b + 1])
        for t in range(q1 - q0):
            lim = L - (q1 - q0) + t + 1
            if lim <= 0:
                out[q0 + t] = 0.0
                continue
            for h in range(KVH):
                s_ = (q[q0 + t, h * G:(h + 1) * G] @ kb[:lim, h].T) * sm
                p_ = np.exp(s_ - s_.max(axis=1, keepdims=True))
                out[q0 + t, h * G:(h + 1) * G] = (p_ / p_.sum(axis=1, keepdims=True)) @ vb[:lim, h]
    return out
