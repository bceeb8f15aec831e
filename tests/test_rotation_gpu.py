"""The optional Hadamard key rotation on the GPU (reference: kv_fp4_ref.py:31-35, :55-92, :233-241 and the fused
rotation of kv_fp4_serving.py:146-189, :621-641): the write kernel's rotated keys are byte-equal to the reference's
write_reference(signs=...) fixture and to the oracle, and the decode kernel, given the UNROTATED query, matches fp64
attention of the rotated bf16 query (rotate_q) over the rotated cache."""
import os

import numpy as np
import pytest
import torch

import synth
from cases import Cache, assert_close, bf16_tensor, unquantised_attention
from horizon_kernels_b200 import kernels as K
from oracle import kvfp4 as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [128, 256])
@pytest.mark.parametrize("search", [0, 1])
def test_rotated_write_golden(golden_dir, D, search):
    z = np.load(os.path.join(golden_dir, "rotation.npz"))
    KVH, D_, PS, NP = (int(v) for v in z[f"w{D}_geom"])
    cache = Cache(NP, PS, KVH, D, "region", fill=0xA5)
    signs = torch.from_numpy(z[f"signs{D}"]).cuda()
    assert torch.equal(signs.cpu(), K.hadamard_signs(D))
    K.write(bf16_tensor(z[f"w{D}_key"]), bf16_tensor(z[f"w{D}_val"]), cache.flat, cache.strides, PS,
            torch.from_numpy(z[f"w{D}_slots"]).cuda(), torch.from_numpy(z[f"w{D}_gk"]).cuda(),
            torch.from_numpy(z[f"w{D}_gv"]).cuda(), bool(search), signs=signs)
    assert np.array_equal(cache.bytes(), z[f"w{D}_region_s{search}"])


@pytest.mark.parametrize("KVH,D,NT,kind", [(8, 128, 5000, "hnd"), (2, 128, 300, "hnd"), (1, 256, 4100, "nhd"),
                                           (3, 256, 77, "hnd")])
def test_rotated_write_matches_oracle(KVH, D, NT, kind):
    """prefill-sized and small launches, kv-head counts that put key and value rows into one warp, skipped slots and a
    grid whose last block is partly out of range"""
    PS = 16
    NP = (NT + PS - 1) // PS + 2
    k = synth.normal(900 + NT, (NT, KVH, D)) * 2.0
    k[:, :, [3, D // 2 + 3]] *= 20.0
    v = synth.normal(901 + NT, (NT, KVH, D))
    kb, vb = synth.to_bf16_bits(k), synth.to_bf16_bits(v)
    slots = synth.permutation(902 + NT, NP * PS)[:NT].astype(np.int64)
    slots[::13] = -1
    gk = np.full(KVH, synth.tensor_scale(kb), np.float32)
    gv = np.full(KVH, synth.tensor_scale(vb), np.float32)
    signs = K.hadamard_signs(D)
    cache = Cache(NP, PS, KVH, D, kind, fill=0x33)
    K.write(bf16_tensor(kb), bf16_tensor(vb), cache.flat, cache.strides, PS, torch.from_numpy(slots).cuda(),
            torch.from_numpy(gk).cuda(), torch.from_numpy(gv).cuda(), True, signs=signs.cuda())
    want = np.full(cache.phys.numel(), 0x33, np.uint8)
    O.write(kb, vb, want, cache.olay, slots, gk, gv, True, signs=signs.numpy())
    assert np.array_equal(cache.bytes(), want)


@pytest.mark.parametrize("KVH,G,D,qls", [(8, 4, 128, [1, 1, 1]), (2, 8, 256, [1, 1, 1]), (2, 4, 128, [2, 1, 2])])
def test_rotated_decode_matches_oracle(KVH, G, D, qls):
    lens = [700, 33, 2100]
    PS = 16
    c = synth.paged_case(950 + D + G, lens, KVH, G, D, PS, outliers=True, ql_list=qls)
    gk = np.full(KVH, synth.tensor_scale(c["key"]) * 0.5, np.float32)       # rotated keys are smaller than the outliers
    gv = np.full(KVH, synth.tensor_scale(c["val"]), np.float32)
    signs = K.hadamard_signs(D)
    cache = Cache(c["NP"], PS, KVH, D, "hnd", fill=0x7F)
    dev = cache.phys.device
    K.write(bf16_tensor(c["key"]), bf16_tensor(c["val"]), cache.flat, cache.strides, PS,
            torch.from_numpy(c["slots"]).to(dev), torch.from_numpy(gk).to(dev), torch.from_numpy(gv).to(dev), True,
            signs=signs.to(dev))
    sm = D ** -0.5
    NT = c["q"].shape[0]
    out = torch.full((NT, KVH * G, D), float("nan"), dtype=torch.bfloat16, device=dev)
    qlmax = max(qls)
    ws = K.alloc_workspace(len(lens), KVH, G, D, qlmax, dev)
    K.decode_ragged(bf16_tensor(c["q"]), cache.flat, cache.strides, PS, torch.from_numpy(c["bt"]).to(dev),
                    torch.from_numpy(c["seq_lens"]).to(dev), torch.from_numpy(c["qsl"]).to(dev), sm, 1.0,
                    torch.from_numpy(gk).to(dev), torch.from_numpy(gv).to(dev), qlmax, out, ws, signs=signs.to(dev))
    assert K.workspace_status(ws) == 0
    # the oracle: fp64 attention of the rotated bf16 query over the same (rotated) cache bytes
    q_rot = O.rotate_q(c["q"], signs.numpy())
    ref, _ = O.attention(q_rot, cache.bytes(), cache.olay, c["bt"], c["seq_lens"], c["qsl"], KVH, sm, gk, gv, 1.0)
    assert_close(out, ref)
    # the rotation leaves the model's math unchanged (q' . k' = q . k): the result stays close to fp64 attention over
    # the UNQUANTISED bf16 keys and values; what remains is the 4-bit quantisation error of this outlier-heavy case
    true = unquantised_attention(c, sm)
    err = np.abs(out.float().cpu().numpy().astype(np.float64) - true)
    assert np.mean(err) < 0.25, np.mean(err)
