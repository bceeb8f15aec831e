"""The K8V4 slot on the GPU (FP8 keys + FP4 values, 400 bytes per token and kv head at head_dim 256; reference:
kv_fp4_ref.py:283-321, `HORIZON_KVFP4_K8`): write byte-equal to the reference's write_reference_k8 fixture and to the
oracle, decode within the task's tolerance of fp64 attention over the same cache, dequantisation exact."""
import os

import numpy as np
import pytest
import torch

import synth
from cases import assert_close, bf16_tensor
from horizon_kernels_b200 import kernels as K
from horizon_kernels_b200 import layout as Lt
from oracle import kvfp4 as O

pytestmark = pytest.mark.gpu
D = 256


def k8_cache(NP, KVH, PS, fill):
    phys = torch.full((NP, KVH, PS, Lt.K8_SLOT), fill, dtype=torch.uint8, device="cuda")
    flat, st = Lt.k8_flat_views(*Lt.k8_views(phys, D))
    lay = O.Layout.k8_slots(PS, KVH, D)
    assert tuple(st) == tuple(lay.strides())
    return phys, flat, st, lay


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("search", [0, 1])
def test_k8_write_golden(golden_dir, search):
    z = np.load(os.path.join(golden_dir, "k8v4.npz"))
    KVH, G, D_, PS, NP = (int(v) for v in z["geom"])
    phys, flat, st, lay = k8_cache(NP, KVH, PS, 0xA5)
    K.write(bf16_tensor(z["key"]), bf16_tensor(z["val"]), flat, st, PS, dev(z["slots"]), dev(z["gk"]), dev(z["gv"]),
            bool(search), k8=True)
    assert np.array_equal(phys.cpu().numpy().reshape(-1), z[f"cache_s{search}"])


def test_k8_decode_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "k8v4.npz"))
    KVH, G, D_, PS, NP = (int(v) for v in z["geom"])
    phys, flat, st, lay = k8_cache(NP, KVH, PS, 0)
    phys.copy_(dev(z["cache_s1"]).view(phys.shape))
    q = bf16_tensor(z["q"])
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = K.alloc_workspace(len(z["seq_lens"]), KVH, G, D, 2, "cuda")
    K.decode_ragged(q, flat, st, PS, dev(z["bt"]), dev(z["seq_lens"]), dev(z["qsl"]), D ** -0.5, 1.0, dev(z["gk"]),
                    dev(z["gv"]), 2, out, ws, k8=True)
    assert K.workspace_status(ws) == 0
    assert_close(out, z["ref"])


@pytest.mark.parametrize("KVH,G,lens,qls", [(2, 8, [3000, 17, 640, 0, 129], [1, 1, 1, 1, 1]),
                                            (4, 4, [20000, 500], [2, 1]), (1, 16, [257], [1])])
def test_k8_write_decode_dequant_match_oracle(KVH, G, lens, qls):
    PS = 16
    c = synth.paged_case(1300 + KVH, lens, KVH, G, D, PS, outliers=True, ql_list=qls)
    gk = np.full(KVH, synth.tensor_scale(c["key"]) * 6, np.float32)       # keys span the e4m3 range
    gv = np.full(KVH, synth.tensor_scale(c["val"]), np.float32)
    phys, flat, st, lay = k8_cache(c["NP"], KVH, PS, 0x7F)
    K.write(bf16_tensor(c["key"]), bf16_tensor(c["val"]), flat, st, PS, dev(c["slots"]), dev(gk), dev(gv), True,
            k8=True)
    want = np.full(phys.numel(), 0x7F, np.uint8)
    O.write(c["key"], c["val"], want, lay, c["slots"], gk, gv, True)
    assert np.array_equal(phys.cpu().numpy().reshape(-1), want)
    # decode (several passes when G * ql > 8), also with a capped number of partitions
    q = bf16_tensor(c["q"])
    qlmax = max(qls)
    ref, _ = O.attention(c["q"], want, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, D ** -0.5, gk, gv, 0.5)
    ws = K.alloc_workspace(len(lens), KVH, G, D, qlmax, "cuda")
    for splits in (None, 1):
        out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
        K.decode_ragged(q, flat, st, PS, dev(c["bt"]), dev(c["seq_lens"]), dev(c["qsl"]), D ** -0.5, 0.5, dev(gk),
                        dev(gv), qlmax, out, ws, splits=splits, k8=True)
        assert K.workspace_status(ws) == 0
        assert_close(out, ref, f"splits {splits}")
    # dequantisation of request 0's first tokens: keys are the e4m3 values, values code * scale
    n = min(lens[0], 300)
    ok = torch.empty((n, KVH, D), dtype=torch.float16, device="cuda")
    ov = torch.empty_like(ok)
    K.dequant_tokens(flat, st, PS, dev(c["bt"][0]), 0, n, ok, ov, k8=True)
    e4 = O.e4m3_decode(np.arange(128, dtype=np.uint8))
    raw = want.reshape(phys.shape)
    for i in range(0, n, 37):
        page, pos = int(c["bt"][0, i // PS]), i % PS
        for h in range(KVH):
            slot = raw[page, h, pos]
            kb = slot[:D]
            assert np.array_equal(ok[i, h].float().cpu().numpy(), np.where(kb & 0x80, -1.0, 1.0) * e4[kb & 0x7F])
            assert np.array_equal(ov[i, h].float().cpu().numpy(),
                                  O.dequantize_rows(slot[D:D + D // 2][None], slot[D + D // 2:][None])[0])


def test_k8_misuse():
    phys, flat, st, lay = k8_cache(4, 2, 16, 0)
    k = torch.zeros(4, 2, 128, dtype=torch.bfloat16, device="cuda")       # head_dim 128 has no K8V4 slot
    with pytest.raises(Exception):
        K.write(k, k, flat, st, 16, torch.arange(4, device="cuda"), torch.ones(2, device="cuda"),
                torch.ones(2, device="cuda"), True, k8=True)
    k = torch.zeros(4, 2, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        K.write(k, k, flat, st, 16, torch.arange(4, device="cuda"), torch.ones(2, device="cuda"),
                torch.ones(2, device="cuda"), True, signs=torch.ones(256, device="cuda"), k8=True)
