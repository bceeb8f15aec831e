"""CPU-side checks of the C-ABI library: it loads, exports every symbol include/hkv.h declares, and rejects
host-detectable misuse with an error code before any CUDA call (nothing is launched here)."""
import ctypes as C
import os
import re

import pytest

from horizon_kernels_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_exports_match_header(lib):
    hdr = open(os.path.join(ROOT, "include", "hkv.h")).read()
    declared = set(re.findall(r"\b(hkv_[a-z_0-9]+)\s*\(", hdr))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.hkv_version() >= 100
    assert lib.hkv_error_string(0) == b"ok" and b"null" in lib.hkv_error_string(-1)


def _strides(*v):
    return (C.c_int64 * 6)(*v)


def test_write_rejects_misuse(lib):
    one = C.c_void_p(0x1000)
    st = _strides(18432, 72, 1152, 18432, 72, 1152)
    args = dict(key=one, val=one, ks=(1024, 128, 1024, 128), parts=(one, one, one, one), st=st, PS=16, slots=one, n=4,
                gk=one, gv=one, KVH=8, D=128)

    def call(**kw):
        a = dict(args, **kw)
        return lib.hkv_write(a["key"], a["val"], *a["ks"], *a["parts"], a["st"], a["PS"], a["slots"], a["n"], a["gk"],
                             a["gv"], a["KVH"], a["D"], 1, None)
    assert call(key=None) == -1
    assert call(slots=None) == -1
    assert call(D=64) == -3
    assert call(D=192) == -3
    assert call(n=-1) == -6
    assert call(n=0) == 0                                    # nothing to do, nothing launched
    assert call(key=C.c_void_p(0x1004)) == -2
    assert call(ks=(1024, 12, 1024, 128)) == -2


def test_decode_rejects_misuse(lib):
    one = C.c_void_p(0x1000)
    st = _strides(18432, 72, 1152, 18432, 72, 1152)
    base = dict(q=one, kd=one, ksf=C.c_void_p(0x1000 + 64), vd=C.c_void_p(0x1000 + 9216),
                vsf=C.c_void_p(0x1000 + 9216 + 64), st=st, PS=16, bt=one, MP=8, sl=one, qsl=one, B=4, KVH=8, G=4, D=128,
                qlmax=1, ws=one, wsb=1 << 20, splits=0, out=one)

    def call(**kw):
        a = dict(base, **kw)
        return lib.hkv_decode(a["q"], a["kd"], a["ksf"], a["vd"], a["vsf"], a["st"], a["PS"], a["bt"], a["MP"], a["sl"],
                              a["qsl"], a["B"], a["KVH"], a["G"], a["D"], a["qlmax"], 0.088, 1.0, one, one, a["ws"],
                              a["wsb"], a["splits"], a["out"], None)
    assert call(q=None) == -1
    assert call(ws=None) == -1
    assert call(D=64) == -3
    assert call(G=65) == -3                                  # more than 64 query rows per kv head
    assert call(qlmax=17) == -3
    assert call(PS=8) == -3
    assert call(PS=24) == -3
    assert call(splits=65) == -4
    assert call(B=-1) == -6
    assert call(B=0) == 0
    assert call(B=100000) == -6
    assert call(st=_strides(18432, 2304, 144, 18432, 1152, 144)) == -3      # scales not behind their token's codes
    assert call(st=_strides(18432, 2300, 144, 18432, 2300, 144)) == -2      # positions-outer rows off the 8-byte grid
    assert call(kd=C.c_void_p(0x1008), ksf=C.c_void_p(0x1008 + 64)) == -2
    assert call(ws=C.c_void_p(0x1010)) == -2


def test_combine_rejects_misuse(lib):
    one = C.c_void_p(0x1000)
    assert lib.hkv_combine(None, 1 << 20, one, 4, 8, 4, 128, 1, 1.0, one, None) == -1
    assert lib.hkv_combine(one, 1 << 20, one, 4, 8, 4, 96, 1, 1.0, one, None) == -3
    assert lib.hkv_combine(one, 1 << 20, one, 0, 8, 4, 128, 1, 1.0, one, None) == 0
    assert lib.hkv_combine(one, 1 << 20, one, 4, 8, 65, 128, 1, 1.0, one, None) == -3


def test_dequant_rejects_misuse(lib):
    one = C.c_void_p(0x1000)
    st = (C.c_int64 * 6)(1152 * 16, 72, 1152, 1152 * 16, 72, 1152)
    f = lib.hkv_dequant

    def call(kd=one, rows=None, cu=None, n_rows=0, start=0, n=4, D=128, KVH=8, ok=one):
        return f(kd, one, one, one, st, 16, one, 4, rows, cu, n_rows, start, n, ok, one, KVH, D, 0, None)
    assert call(kd=None) == -1
    assert call(rows=one) == -1                                # rows without cu
    assert call(rows=one, cu=one, n_rows=0) == -6
    assert call(D=64) == -3
    assert call(KVH=0) == -3
    assert call(n=-1) == -6
    assert call(start=-1) == -6
    assert call(n=0) == 0
    assert call(ok=C.c_void_p(0x1008)) == -2
    assert call(start=60, n=8) == -6                           # positions beyond the 4-page block-table row


def test_set_option_codes(lib):
    assert lib.hkv_set_option(99, 1) == -3
    assert lib.hkv_set_option(1, 2) == -6
    assert lib.hkv_set_option(1, 1) == 0
    assert lib.hkv_set_option(1, 0) == 0


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    from horizon_kernels_b200 import kernels as K
    k = torch.zeros(2, 2, 128, dtype=torch.bfloat16)
    flat = tuple(torch.zeros(16, dtype=torch.uint8) for _ in range(4))
    with pytest.raises(RuntimeError, match="no CPU path"):
        K.write(k, k, flat, (1, 1, 1, 1, 1, 1), 16, torch.zeros(2, dtype=torch.int64), torch.ones(2), torch.ones(2))


def test_python_wrappers_check_dtypes_and_shapes_before_any_launch():
    """a wrong dtype or shape must raise on the host (the C ABI sees raw pointers and could not tell)"""
    import torch
    from horizon_kernels_b200 import kernels as K
    k = torch.zeros(2, 2, 128, dtype=torch.bfloat16)
    flat = tuple(torch.zeros(16, dtype=torch.uint8) for _ in range(4))
    st, slots, g = (1, 1, 1, 1, 1, 1), torch.zeros(2, dtype=torch.int64), torch.ones(2)
    with pytest.raises(TypeError):
        K.write(k.half(), k, flat, st, 16, slots, g, g)                       # fp16 keys
    with pytest.raises(TypeError):
        K.write(k, k, flat, st, 16, slots.int(), g, g)                        # int32 slot ids
    with pytest.raises(ValueError):
        K.write(k, k, flat, st, 16, torch.zeros(3, dtype=torch.int64), g, g)  # more slots than tokens
    with pytest.raises(TypeError):
        K.write(k, k, flat, st, 16, slots, g.double(), g)                     # fp64 scales
    q, out, ws = torch.zeros(2, 8, 128, dtype=torch.bfloat16), torch.zeros(2, 8, 128, dtype=torch.bfloat16), flat[0]
    bt, sl, qsl = torch.zeros(2, 4, dtype=torch.int32), torch.zeros(2, dtype=torch.int32), torch.zeros(3, dtype=torch.int32)
    with pytest.raises(TypeError):
        K.decode_ragged(q, flat, st, 16, bt.long(), sl, qsl, 1.0, 1.0, g, g, 1, out, ws)
    with pytest.raises(ValueError):
        K.decode_ragged(q, flat, st, 16, bt, sl, qsl[:2], 1.0, 1.0, g, g, 1, out, ws)      # B entries instead of B + 1
    with pytest.raises(ValueError):
        K.decode_ragged(q, flat, st, 16, bt, sl, qsl, 1.0, 1.0, g, g, 1, out[:1], ws)      # out shorter than the query
    with pytest.raises(TypeError):
        K.decode_ragged(q.float(), flat, st, 16, bt, sl, qsl, 1.0, 1.0, g, g, 1, out, ws)
    from horizon_kernels_b200 import ops
    hkv = ops.register()
    with pytest.raises((RuntimeError, NotImplementedError)):
        hkv.write(k, k, *flat, list(st), 16, slots, g, g, True)                # CPU tensors: no implementation
