"""The torch custom ops (torch.ops.hkv.write / decode / combine) give the same bytes and outputs as the host wrappers."""
import numpy as np
import pytest
import torch

from cases import Cache, assert_close, bf16_tensor, build_decode_case, gpu_decode, oracle_decode
from horizon_kernels_b200 import kernels as K
from horizon_kernels_b200 import ops

pytestmark = pytest.mark.gpu


def test_custom_ops_match_wrappers():
    hkv = ops.register()
    c = build_decode_case(5100, [700, 33, 2500], 8, 4, 128, 16)          # cache written through kernels.write
    cache = c["cache"]
    dev = cache.phys.device
    # write through the op into a second cache: same bytes
    other = Cache(cache.NP, cache.PS, cache.KVH, cache.D, "hnd", fill=0x7F)
    gk, gv = torch.from_numpy(c["gk"]).to(dev), torch.from_numpy(c["gv"]).to(dev)
    hkv.write(bf16_tensor(c["key"]), bf16_tensor(c["val"]), *other.flat, list(other.strides), other.PS,
              torch.from_numpy(c["slots"]).to(dev), gk, gv, True)
    assert torch.equal(other.phys, cache.phys)
    want, _ = gpu_decode(c)
    q = bf16_tensor(c["q"])
    out = torch.full_like(want, float("nan"))
    ws = K.alloc_workspace(3, 8, 4, 128, 1, dev)
    bt, sl, qsl = (torch.from_numpy(c[k]).to(dev) for k in ("bt", "seq_lens", "qsl"))
    hkv.decode(q, *cache.flat, list(cache.strides), cache.PS, bt, sl, qsl, c["sm"], 1.0, gk, gv, 1, ws, 0, out)
    hkv.combine(ws, qsl, 8, 4, 128, 1, 1.0, out)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert_close(out, oracle_decode(c))
    with pytest.raises((RuntimeError, NotImplementedError)):
        hkv.combine(ws.cpu(), qsl.cpu(), 8, 4, 128, 1, 1.0, out.cpu())          # no CPU implementation
