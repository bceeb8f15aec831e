"""hkv_decode_noalloc, the decode entry point for callers that cannot allocate device memory (a runtime that starts
after the serving process has given all GPU memory to its pool, or code running while cudaMalloc is forbidden): it
must give the same output as hkv_decode + hkv_combine with a caller-provided workspace, on two calls in a row that
share its built-in scratch. Called through the C ABI. This file sorts last on purpose: if it fails, a run that stops
at the first failure has already run everything else."""
import ctypes as C

import numpy as np
import pytest
import torch

from cases import assert_close, bf16_tensor, build_decode_case, gpu_decode, oracle_decode
from horizon_kernels_b200 import _lib

pytestmark = pytest.mark.gpu


def call_noalloc(c, out, v_scale=1.0, splits=0):
    cache = c["cache"]
    dev = cache.phys.device
    q = bf16_tensor(c["q"])
    bt, sl, qsl = (torch.from_numpy(c[k]).to(dev) for k in ("bt", "seq_lens", "qsl"))
    gk, gv = torch.from_numpy(c["gk"]).to(dev), torch.from_numpy(c["gv"]).to(dev)
    kd, ksf, vd, vsf = cache.flat
    st = (C.c_int64 * 6)(*cache.strides)
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    rc = _lib.load().hkv_decode_noalloc(p(q), p(kd), p(ksf), p(vd), p(vsf), st, cache.PS, p(bt), bt.shape[1], p(sl), p(qsl),
                                        len(c["seq_lens"]), c["KVH"], c["G"], c["D"], 1, c["sm"], v_scale, p(gk), p(gv),
                                        splits, p(out), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc


@pytest.mark.parametrize("D,KVH,G", [(128, 8, 4), (256, 2, 8)])
def test_noalloc_matches_workspace_entry_points(D, KVH, G):
    for seed, lens in ((4100, [3000, 17, 900, 64, 5000]), (4101, [40000, 1, 333])):      # two calls in a row
        c = build_decode_case(seed + D, lens, KVH, G, D, 16)
        want, _ = gpu_decode(c, v_scale=0.5)
        torch.cuda.synchronize()
        got = torch.full_like(want, float("nan"))
        assert call_noalloc(c, got, v_scale=0.5) == 0
        assert_close(got, oracle_decode(c, v_scale=0.5))
        # same kernels, same partitioning: the two paths agree to the last bit, well inside the tests' tolerance
        assert torch.equal(got, want)


def test_noalloc_rejects_what_does_not_fit_or_is_unsupported():
    c = build_decode_case(4200, [100], 2, 4, 128, 16)
    out = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda")
    L = _lib.load()
    assert call_noalloc(c, out, splits=65) == -4
    assert b"scratch" in L.hkv_error_string(-9)
    c2 = dict(c, G=65)                                            # more than 64 query rows per kv head
    assert call_noalloc(c2, out) == -3
