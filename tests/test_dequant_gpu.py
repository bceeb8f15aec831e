"""GPU parity of the exact dequantisation kernel (hkv_dequant, through the Python wrappers with the reference's
signatures `dequant_tokens` / `dequant_multi`, kv_fp4_serving.py:918 and :1008) against the oracle's dequantize_rows
(pinned to the reference's by tests/test_oracle.py) over the same cache bytes: bit-equal in bf16 and in fp16."""
import numpy as np
import pytest
import torch

from cases import build_decode_case
from horizon_kernels_b200 import kernels as K
from oracle import kvfp4 as O

pytestmark = pytest.mark.gpu


def oracle_rows(c, b, positions, side):
    """dequantised (len(positions), KVH, D) fp32 rows of request b, read from the cache bytes like the oracle does"""
    cache, lay = c["cache"], c["cache"].olay
    raw = cache.bytes()
    KVH, D, PS = c["KVH"], c["D"], cache.PS
    base_d, base_s = (lay.vd, lay.vsf) if side else (lay.kd, lay.ksf)
    out = np.zeros((len(positions), KVH, D), np.float32)
    for i, p in enumerate(positions):
        page, pos = int(c["bt"][b, p // PS]), p % PS
        for h in range(KVH):
            od = base_d + page * lay.dsp + pos * lay.dst + h * lay.dsh
            os_ = base_s + page * lay.ssp + pos * lay.sst + h * lay.ssh
            out[i, h] = O.dequantize_rows(raw[od:od + D // 2][None], raw[os_:os_ + D // 16][None])[0]
    return out


@pytest.mark.parametrize("D,KVH,PS,kind", [(128, 8, 16, "hnd"), (256, 2, 16, "hnd"), (128, 3, 32, "nhd"),
                                           (256, 4, 64, "region"), (128, 2, 16, "region")])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dequant_tokens_matches_oracle(D, KVH, PS, kind, dtype):
    lens = [200, 77, 16]
    c = build_decode_case(5000 + D + KVH, lens, KVH, 4, D, PS, kind=kind, gscale=(0.05, 0.01))
    cache = c["cache"]
    bt = torch.from_numpy(c["bt"]).cuda()
    for b, (start, n) in enumerate([(0, 200), (5, 61), (15, 1)]):
        ok = torch.full((n + 3, KVH, D), 9.0, dtype=dtype, device="cuda")
        ov = torch.full((n + 3, KVH, D), 9.0, dtype=dtype, device="cuda")
        k, v = K.dequant_tokens(cache.flat, cache.strides, PS, bt[b].contiguous(), start, n, ok, ov)
        pos = list(range(start, start + n))
        assert np.array_equal(k.float().cpu().numpy(), oracle_rows(c, b, pos, 0))
        assert np.array_equal(v.float().cpu().numpy(), oracle_rows(c, b, pos, 1))
        assert (ok[n:] == 9.0).all() and (ov[n:] == 9.0).all()         # rows past n are untouched


def test_dequant_multi_packs_requests():
    KVH, D, PS = 4, 128, 16
    lens = [50, 300, 7, 129]
    c = build_decode_case(5100, lens, KVH, 4, D, PS)
    cache = c["cache"]
    bt = torch.from_numpy(c["bt"]).cuda()
    rows = [3, 1, 2]                                                      # any order, any subset
    cu = np.concatenate([[0], np.cumsum([lens[r] for r in rows])]).astype(np.int32)
    n = int(cu[-1])
    ok = torch.zeros((n, KVH, D), dtype=torch.bfloat16, device="cuda")
    ov = torch.zeros_like(ok)
    K.dequant_multi(cache.flat, cache.strides, PS, bt, torch.tensor(rows, dtype=torch.int32, device="cuda"),
                    torch.from_numpy(cu).cuda(), len(rows), n, ok, ov)
    for i, r in enumerate(rows):
        pos = list(range(lens[r]))
        assert np.array_equal(ok[cu[i]:cu[i + 1]].float().cpu().numpy(), oracle_rows(c, r, pos, 0))
        assert np.array_equal(ov[cu[i]:cu[i + 1]].float().cpu().numpy(), oracle_rows(c, r, pos, 1))


def test_dequant_round_trip_of_grid_values():
    """values on the E2M1 grid times a power-of-two block scale survive write -> dequant exactly (times 1 / g)"""
    KVH, D, PS, NT = 2, 128, 16, 64
    grid = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -.5, -1, -1.5, -2, -3, -4, -6, 6.0])
    idx = torch.randint(0, 16, (NT, KVH, D), generator=torch.Generator().manual_seed(3))
    x = grid[idx]
    x[..., 15::16] = 6.0                                                  # every block's amax is 6: scale code of 1.0 * g
    from horizon_kernels_b200 import layout as Lt
    pool = torch.zeros((NT // PS, 2 * KVH, PS, Lt.slot_bytes(D)), dtype=torch.uint8, device="cuda")
    flat, st = Lt.flat_views(*Lt.slot_views(pool, KVH, D))
    g = torch.ones(KVH, device="cuda")
    xb = x.to(torch.bfloat16).cuda()
    K.write(xb, xb, flat, st, PS, torch.arange(NT, dtype=torch.int64, device="cuda"), g, g, True)
    ok = torch.empty((NT, KVH, D), dtype=torch.float16, device="cuda")
    ov = torch.empty_like(ok)
    K.dequant_tokens(flat, st, PS, torch.arange(NT // PS, dtype=torch.int32, device="cuda"), 0, NT, ok, ov)
    assert torch.equal(ok.float().cpu(), x) and torch.equal(ov.float().cpu(), x)


def test_dequant_misuse_raises():
    c = build_decode_case(5200, [40], 2, 4, 128, 16)
    cache = c["cache"]
    bt = torch.from_numpy(c["bt"]).cuda()
    ok = torch.empty((40, 2, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(TypeError):
        K.dequant_tokens(cache.flat, cache.strides, 16, bt[0].contiguous(), 0, 40, ok, ok.half())
    with pytest.raises(ValueError):
        K.dequant_tokens(cache.flat, cache.strides, 16, bt[0].contiguous(), 0, 41, ok, torch.empty_like(ok))
    from horizon_kernels_b200 import _lib
    with pytest.raises(_lib.HkvError, match="unsupported"):          # the K8V4 slot exists at head_dim 256 only
        K.dequant_tokens(cache.flat, cache.strides, 16, bt[0].contiguous(), 0, 40, ok, torch.empty_like(ok), k8=True)
