"""numpy front end of the C oracle (oracle/kvfp4_oracle.c). TEST INFRASTRUCTURE, not product code.

bf16 tensors travel as uint16 bit patterns; caches as flat uint8 arrays plus a Layout that says where the four parts
(K data, K scales, V data, V scales) sit and how they are strided as [page, position, head, byte] views — the same
description the reference kernels take (kv_fp4_ref.py:215-230, kv_fp4_serving.py:873-886 in the reference).
Parity status: pinned by tests/test_oracle.py against vectors generated from the reference's PyTorch code."""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from .build import build

_lib = None


class _CLayout(C.Structure):
    _fields_ = [(n, C.c_longlong) for n in ("kd", "ksf", "vd", "vsf", "dsp", "dst", "dsh", "ssp", "sst", "ssh")] + \
               [("PS", C.c_int), ("k8", C.c_int)]


@dataclass
class Layout:
    """offsets of the four cache parts (bytes from the cache base) and the [page, position, head] byte strides"""
    kd: int
    ksf: int
    vd: int
    vsf: int
    dsp: int
    dst: int
    dsh: int
    ssp: int
    sst: int
    ssh: int
    PS: int
    k8: int = 0

    @staticmethod
    def region(PS: int, KVH: int, D: int) -> "Layout":
        """page = [K data (KVH, PS, D/2) | K scales (KVH, PS, D/16) | V data | V scales]: split_views of the
        reference's torch oracle (kv_fp4_ref.py:215-230)"""
        dd, sd = D // 2, D // 16
        page = 2 * KVH * PS * (dd + sd)
        side = KVH * PS * (dd + sd)
        return Layout(0, KVH * PS * dd, side, side + KVH * PS * dd, page, dd, PS * dd, page, sd, PS * sd, PS)

    @staticmethod
    def slots(PS: int, KVH: int, D: int, nhd: bool = False) -> "Layout":
        """serving layout: logical (pages, 2 KVH, PS, slot) with slot = [D/2 data | D/16 scales], K heads first
        (backend.py:279-300 of the reference); physical order heads-outer (HND) or positions-outer (NHD)"""
        dd, sd = D // 2, D // 16
        slot = dd + sd
        page = 2 * KVH * PS * slot
        if nhd:
            st, sh = 2 * KVH * slot, slot
        else:
            st, sh = slot, PS * slot
        return Layout(0, dd, KVH * sh, KVH * sh + dd, page, st, sh, page, st, sh, PS)

    @staticmethod
    def k8_slots(PS: int, KVH: int, D: int) -> "Layout":
        """K8V4 (kv_fp4_ref.py:283-293): logical (pages, KVH, PS, slot) with slot = [D e4m3 key bytes | D/2 value codes
        | D/16 value scales] (400 bytes at head_dim 256), heads outermost inside a page"""
        slot = D + D // 2 + D // 16
        page = KVH * PS * slot
        return Layout(0, 0, D, D + D // 2, page, slot, PS * slot, page, slot, PS * slot, PS, 1)

    def c(self) -> _CLayout:
        return _CLayout(self.kd, self.ksf, self.vd, self.vsf, self.dsp, self.dst, self.dsh, self.ssp, self.sst,
                        self.ssh, self.PS, self.k8)

    def strides(self):
        return (self.dsp, self.dst, self.dsh, self.ssp, self.sst, self.ssh)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        L.hkvo_attention.restype = C.c_longlong
        L.hkvo_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().hkvo_num_threads())


def set_num_threads(n: int):
    lib().hkvo_set_num_threads(C.c_int(int(n)))


def e4m3_encode(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().hkvo_e4m3_encode_n(_p(x), C.c_longlong(x.size), _p(out))
    return out


def e4m3_decode(c):
    c = np.ascontiguousarray(c, dtype=np.uint8)
    out = np.empty(c.shape, np.float64)
    lib().hkvo_e4m3_decode_n(_p(c), C.c_longlong(c.size), _p(out))
    return out


def e2m1_code(y):
    y = np.ascontiguousarray(y, dtype=np.float32)
    out = np.empty(y.shape, np.uint8)
    lib().hkvo_e2m1_mag_n(_p(y), C.c_longlong(y.size), _p(out))
    return out


def e2m1_value(c):
    c = np.ascontiguousarray(c, dtype=np.uint8)
    out = np.empty(c.shape, np.float32)
    lib().hkvo_e2m1_value_n(_p(c), C.c_longlong(c.size), _p(out))
    return out


def bf16_to_f32(u16):
    return (np.ascontiguousarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize_rows(x, g, search=True):
    """x (..., D) float32, g scalar or array broadcastable to x[..., 0] -> (data (..., D/2), sf (..., D/16)) uint8"""
    x = np.ascontiguousarray(x, dtype=np.float32)
    D = x.shape[-1]
    assert D % 16 == 0
    rows = x.reshape(-1, D)
    gr = np.ascontiguousarray(np.broadcast_to(np.asarray(g, dtype=np.float32), x.shape[:-1]).reshape(-1))
    data = np.empty((rows.shape[0], D // 2), np.uint8)
    sf = np.empty((rows.shape[0], D // 16), np.uint8)
    lib().hkvo_quantize_rows(_p(rows), C.c_longlong(rows.shape[0]), C.c_int(D), _p(gr), C.c_int(int(bool(search))),
                             _p(data), _p(sf))
    return data.reshape(*x.shape[:-1], D // 2), sf.reshape(*x.shape[:-1], D // 16)


def dequantize_rows(data, sf, g=None):
    """(..., D/2), (..., D/16) -> (..., D) float64 = code * e4m3(sf) (* g)"""
    data = np.ascontiguousarray(data, dtype=np.uint8)
    sf = np.ascontiguousarray(sf, dtype=np.uint8)
    D = data.shape[-1] * 2
    n = data.size // (D // 2)
    out = np.empty((n, D), np.float64)
    gp = None
    if g is not None:
        gr = np.ascontiguousarray(np.broadcast_to(np.asarray(g, dtype=np.float64), data.shape[:-1]).reshape(-1))
        gp = _p(gr)
    lib().hkvo_dequantize_rows(_p(data), _p(sf), C.c_longlong(n), C.c_int(D), gp, _p(out))
    return out.reshape(*data.shape[:-1], D)


def fwht_scale(D: int) -> np.float32:
    """D^-0.5 rounded to fp32 (kv_fp4_ref.py:52-54)"""
    return np.float32(1.0 / np.sqrt(np.float64(D)))


def rotate(x, signs):
    """x (..., D) float32 -> fp32 FWHT(x * signs) * D^-0.5 in the reference's butterfly order (kv_fp4_ref.py:83-87)"""
    x = np.ascontiguousarray(x, dtype=np.float32)
    D = x.shape[-1]
    assert D <= 512 and D & (D - 1) == 0
    signs = np.ascontiguousarray(signs, dtype=np.float32)
    out = np.empty_like(x)
    lib().hkvo_rotate_rows(_p(x), C.c_longlong(x.size // D), C.c_int(D), _p(signs), C.c_float(fwht_scale(D)), _p(out))
    return out


def f32_to_bf16_bits(x):
    """round to nearest even, like torch's .to(bfloat16) for finite values"""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def rotate_q(q_bits, signs):
    """bf16 bits of the query the decode consumes when keys are rotated: rotate() rounded once to bf16
    (kv_fp4_ref.py:90-92)"""
    return f32_to_bf16_bits(rotate(bf16_to_f32(q_bits), signs))


def write(key, value, cache, layout: Layout, slots, gk, gv, search=True, signs=None):
    """key / value (NT, KVH, D) uint16 (bf16 bits), C-contiguous; cache flat uint8 (modified in place); slots int64;
    signs (D,) fp32 -> the keys are rotated before they are quantised"""
    key = np.ascontiguousarray(key, dtype=np.uint16)
    value = np.ascontiguousarray(value, dtype=np.uint16)
    NT, KVH, D = key.shape
    slots = np.ascontiguousarray(slots, dtype=np.int64)
    assert slots.shape[0] <= NT and cache.dtype == np.uint8 and cache.flags.c_contiguous
    gk = np.ascontiguousarray(gk, dtype=np.float32)
    gv = np.ascontiguousarray(gv, dtype=np.float32)
    lay = layout.c()
    sg = None if signs is None else np.ascontiguousarray(signs, dtype=np.float32)
    lib().hkvo_write_rot(_p(key), _p(value), C.c_longlong(KVH * D), C.c_longlong(D), C.c_longlong(KVH * D),
                         C.c_longlong(D), _p(cache), C.byref(lay), _p(slots), C.c_longlong(slots.shape[0]), _p(gk),
                         _p(gv), C.c_int(KVH), C.c_int(D), C.c_int(int(bool(search))),
                         None if sg is None else _p(sg), C.c_float(fwht_scale(D)))


def attention(q, cache, layout: Layout, block_tables, seq_lens, query_start_loc, KVH, sm_scale, gk, gv, v_scale=1.0,
              out=None):
    """q (NT, HQ, D) uint16 (bf16 bits) -> (NT, HQ, D) float64. Rows of requests without query tokens keep the value
    they had in `out` (NaN when out is None)."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    NT, HQ, D = q.shape
    G = HQ // KVH
    bt = np.ascontiguousarray(block_tables, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    qsl = np.ascontiguousarray(query_start_loc, dtype=np.int32)
    B = sl.shape[0]
    gk = np.ascontiguousarray(gk, dtype=np.float32)
    gv = np.ascontiguousarray(gv, dtype=np.float32)
    if out is None:
        out = np.full((NT, HQ, D), np.nan, np.float64)
    lay = layout.c()
    n = lib().hkvo_attention(_p(q), _p(cache), C.byref(lay), _p(bt), C.c_int(bt.shape[1]), _p(sl), _p(qsl),
                             C.c_int(B), C.c_int(KVH), C.c_int(G), C.c_int(D), C.c_double(sm_scale), _p(gk), _p(gv),
                             C.c_double(v_scale), _p(out))
    return out, int(n)


def combine(opart, lse, v_scale=1.0):
    """numpy restatement of the fixed-order split merge (kv_fp4_serving.py:518-558 of the reference): opart
    (S, ..., D) float32 normalised partials, lse (S, ...) float32 log2-sum-exp with -inf for empty splits ->
    (..., D) float64"""
    lse = np.asarray(lse, np.float64)
    opart = np.asarray(opart, np.float64)
    mx = lse.max(axis=0)
    w = np.where(np.isneginf(lse), 0.0, np.exp2(lse - np.where(np.isneginf(mx), 0.0, mx)))
    tot = w.sum(axis=0)
    wn = np.where(tot > 0, w / np.where(tot > 0, tot, 1.0), 0.0)
    return (np.where(wn[..., None] > 0, opart, 0.0) * wn[..., None]).sum(axis=0) * v_scale
