"""The plugin surface end to end on the GPU: HorizonFp4Impl.do_kv_cache_update + forward with metadata from
HorizonFp4Builder, on a vLLM-shaped (blocks, 2*KVH, PS, slot) cache, against the CPU oracle
(reference call path: nvidia-sm120/horizon_kvfp4/backend.py:389-436)."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

os.environ["HORIZON_KVFP4_STANDALONE"] = "1"
import synth  # noqa: E402
from cases import assert_close, bf16_tensor  # noqa: E402
from horizon_kernels_b200 import backend as BE  # noqa: E402
from horizon_kernels_b200 import layout as Lt  # noqa: E402
from oracle import kvfp4 as O  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nhd", [False, True])
@pytest.mark.parametrize("KVH,G,D,PS", [(8, 4, 128, 16), (2, 8, 256, 16), (4, 2, 128, 64)])
def test_update_then_forward_matches_oracle(KVH, G, D, PS, nhd):
    """both page orders the backend advertises: head-major (LBHNC) and positions-outermost (LBNHC) physical pages behind
    the same logical (blocks, 2 * KVH, PS, slot) view"""
    lens = [300, 17, 2049, 64]
    c = synth.paged_case(31 + D + PS, lens, KVH, G, D, PS, outliers=True)
    dev = torch.device("cuda")
    B, HQ = len(lens), KVH * G
    kscale, vscale = 0.04, 0.009
    layer = SimpleNamespace(_k_scale_float=kscale, _v_scale_float=vscale, layer_name="model.layers.3.self_attn.attn")
    impl = BE.HorizonFp4Impl(HQ, D, D ** -0.5, num_kv_heads=KVH, kv_cache_dtype="nvfp4", max_num_seqs=16)
    if nhd:
        phys = torch.full((c["NP"], PS, 2 * KVH, Lt.slot_bytes(D)), 0x7F, dtype=torch.uint8, device=dev)
        kv_cache = phys.permute(0, 2, 1, 3)
    else:
        phys = kv_cache = Lt.alloc_cache(c["NP"], PS, KVH, D, device=dev, fill=0x7F)
    # prefill-style write of every cached token as flat (T, KVH * D) tensors, the shape vLLM passes
    key = bf16_tensor(c["key"]).view(-1, KVH * D)
    val = bf16_tensor(c["val"]).view(-1, KVH * D)
    impl.do_kv_cache_update(layer, key, val, kv_cache, torch.from_numpy(c["slots"]).to(dev))
    want = np.full(kv_cache.numel(), 0x7F, np.uint8)
    lay = O.Layout.slots(PS, KVH, D, nhd=nhd)
    gk = np.full(KVH, kscale, np.float32)
    gv = np.full(KVH, vscale, np.float32)
    O.write(c["key"], c["val"], want, lay, c["slots"], gk, gv, True)
    assert np.array_equal(phys.cpu().numpy().reshape(-1), want)

    qsl = torch.from_numpy(c["qsl"])
    cam = SimpleNamespace(num_reqs=B, num_actual_tokens=B, query_start_loc=qsl.to(dev), query_start_loc_cpu=qsl,
                          seq_lens=torch.from_numpy(c["seq_lens"]).to(dev),
                          block_table_tensor=torch.from_numpy(c["bt"]).to(dev),
                          slot_mapping=torch.zeros(B, dtype=torch.int64, device=dev), seq_lens_cpu_upper_bound=None)
    meta = BE.HorizonFp4Builder().build(0, cam)
    query = bf16_tensor(c["q"]).view(B, HQ * D)
    output = torch.full((B + 2, HQ * D), 5.0, dtype=torch.bfloat16, device=dev)      # padded, as under CUDA graphs
    ret = impl.forward(layer, query, None, None, kv_cache, meta, output)
    assert ret is output
    ref, _ = O.attention(c["q"], want, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, D ** -0.5, gk, gv, vscale)
    scale = 1.0 / vscale                            # the output carries the extra v_scale factor: compare at unit scale
    assert_close(output[:B].view(B, HQ, D).float() * scale, ref * scale)
    assert (output[B:] == 5.0).all()


@pytest.mark.parametrize("chunk,pf16", [("65536", "1"), ("160", "1"), ("96", "0")])
@pytest.mark.parametrize("KVH,G,D,PS", [(8, 4, 128, 16), (2, 8, 256, 16)])
def test_mixed_step_with_prefill_rows(KVH, G, D, PS, chunk, pf16, monkeypatch):
    """a step with decode rows (1 query token) and prefill rows over a cached prefix (37 and 300 query tokens): the
    decode kernel serves the former and leaves the latter untouched, the dequantise + attention path serves the latter;
    both against the oracle with the reference's causal window"""
    # (prefill contexts are dequantised in chunks merged by a running log-sum-exp: the small chunk sizes cut the 700-token
    # context into several chunks that do not end on page boundaries; compute dtype fp16 or bf16)
    monkeypatch.setenv("HORIZON_KVFP4_CHUNK", chunk)
    monkeypatch.setenv("HORIZON_KVFP4_PF16", pf16)
    lens = [300, 37, 2049, 64, 700]
    qls = [1, 37, 1, 1, 300]
    c = synth.paged_case(77 + D, lens, KVH, G, D, PS, outliers=True, ql_list=qls)
    dev = torch.device("cuda")
    B, HQ, NT = len(lens), KVH * G, sum(qls)
    kscale, vscale = 0.04, 0.5
    layer = SimpleNamespace(_k_scale_float=kscale, _v_scale_float=vscale, layer_name="model.layers.0.self_attn.attn")
    impl = BE.HorizonFp4Impl(HQ, D, D ** -0.5, num_kv_heads=KVH, kv_cache_dtype="nvfp4", max_num_seqs=16)
    kv_cache = Lt.alloc_cache(c["NP"], PS, KVH, D, device=dev, fill=0x7F)
    impl.do_kv_cache_update(layer, bf16_tensor(c["key"]).view(-1, KVH * D), bf16_tensor(c["val"]).view(-1, KVH * D),
                            kv_cache, torch.from_numpy(c["slots"]).to(dev))
    qsl = torch.from_numpy(c["qsl"])
    cam = SimpleNamespace(num_reqs=B, num_actual_tokens=NT, query_start_loc=qsl.to(dev), query_start_loc_cpu=qsl,
                          seq_lens=torch.from_numpy(c["seq_lens"]).to(dev),
                          block_table_tensor=torch.from_numpy(c["bt"]).to(dev),
                          slot_mapping=torch.zeros(NT, dtype=torch.int64, device=dev),
                          seq_lens_cpu_upper_bound=torch.from_numpy(c["seq_lens"]))
    meta = BE.HorizonFp4Builder().build(0, cam)
    assert [r[0] for r in meta.prefill_rows] == [1, 4] and meta.has_decode and meta.qlmax == 1
    query = bf16_tensor(c["q"]).view(NT, HQ * D)
    output = torch.full((NT, HQ * D), 5.0, dtype=torch.bfloat16, device=dev)
    impl.forward(layer, query, None, None, kv_cache, meta, output)
    lay = O.Layout.slots(PS, KVH, D)
    gk = np.full(KVH, kscale, np.float32)
    gv = np.full(KVH, vscale, np.float32)
    ref, _ = O.attention(c["q"], kv_cache.cpu().numpy().reshape(-1), lay, c["bt"], c["seq_lens"], c["qsl"], KVH,
                         D ** -0.5, gk, gv, 1.0)
    # like the reference, the decode path multiplies by the V scale twice (gv and bmm2_scale are both
    # layer._v_scale_float, backend.py:431) and the prefill path once (backend.py:523-541): compare at unit scale
    from cases import errors
    got = output.view(NT, HQ, D).float() / vscale
    want = ref / vscale
    dec = np.zeros(NT, bool)
    for b in range(B):
        if qls[b] == 1:
            dec[int(c["qsl"][b])] = True
    got[torch.from_numpy(dec).to(dev)] /= vscale
    assert_close(got[torch.from_numpy(dec).to(dev)], want[dec], "decode rows")
    # prefill rows go through a library bf16 attention (probabilities rounded to bf16): the reference's own gate,
    # relative L2, holds; the absolute error scales with the outputs, which reach the values' outliers here
    mx, mn, rl = errors(got[torch.from_numpy(~dec).to(dev)], want[~dec])
    assert rl <= 2.5e-3 and mn <= 2e-3 and mx <= 6e-2, (mx, mn, rl)


def test_rotation_option_end_to_end(monkeypatch):
    """HORIZON_KVFP4_HAD=1: do_kv_cache_update writes rotated keys, forward rotates the queries of decode rows inside the
    kernel and of prefill rows in torch; both against fp64 attention of rotate_q(q) over the rotated cache"""
    monkeypatch.setenv("HORIZON_KVFP4_HAD", "1")
    from horizon_kernels_b200 import kernels as K
    KVH, G, D, PS = 4, 4, 128, 16
    lens, qls = [500, 90, 64], [1, 30, 1]
    c = synth.paged_case(88, lens, KVH, G, D, PS, outliers=True, ql_list=qls)
    dev = torch.device("cuda")
    B, HQ, NT = len(lens), KVH * G, sum(qls)
    kscale, vscale = 0.02, 1.0
    layer = SimpleNamespace(_k_scale_float=kscale, _v_scale_float=vscale, layer_name="model.layers.1.self_attn.attn")
    impl = BE.HorizonFp4Impl(HQ, D, D ** -0.5, num_kv_heads=KVH, kv_cache_dtype="nvfp4", max_num_seqs=8)
    assert impl.had
    kv_cache = Lt.alloc_cache(c["NP"], PS, KVH, D, device=dev, fill=0x7F)
    impl.do_kv_cache_update(layer, bf16_tensor(c["key"]), bf16_tensor(c["val"]), kv_cache,
                            torch.from_numpy(c["slots"]).to(dev))
    lay = O.Layout.slots(PS, KVH, D)
    gk, gv = np.full(KVH, kscale, np.float32), np.full(KVH, vscale, np.float32)
    signs = K.hadamard_signs(D).numpy()
    want = np.full(kv_cache.numel(), 0x7F, np.uint8)
    O.write(c["key"], c["val"], want, lay, c["slots"], gk, gv, True, signs=signs)
    assert np.array_equal(kv_cache.cpu().numpy().reshape(-1), want)
    qsl = torch.from_numpy(c["qsl"])
    cam = SimpleNamespace(num_reqs=B, num_actual_tokens=NT, query_start_loc=qsl.to(dev), query_start_loc_cpu=qsl,
                          seq_lens=torch.from_numpy(c["seq_lens"]).to(dev),
                          block_table_tensor=torch.from_numpy(c["bt"]).to(dev),
                          slot_mapping=torch.zeros(NT, dtype=torch.int64, device=dev),
                          seq_lens_cpu_upper_bound=torch.from_numpy(c["seq_lens"]))
    meta = BE.HorizonFp4Builder().build(0, cam)
    output = torch.zeros((NT, HQ * D), dtype=torch.bfloat16, device=dev)
    impl.forward(layer, bf16_tensor(c["q"]).view(NT, HQ * D), None, None, kv_cache, meta, output)
    ref, _ = O.attention(O.rotate_q(c["q"], signs), want, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, D ** -0.5, gk,
                         gv, 1.0)
    from cases import errors
    mx, mn, rl = errors(output.view(NT, HQ, D), ref)
    assert rl <= 2.5e-3 and mn <= 2e-3 and mx <= 6e-2, (mx, mn, rl)


def test_k8v4_option_end_to_end(monkeypatch):
    """HORIZON_KVFP4_K8=1: a (blocks, KVH, PS, 400) cache, FP8 keys and FP4 values through do_kv_cache_update + forward
    (decode rows and a prefill row) against the oracle"""
    monkeypatch.setenv("HORIZON_KVFP4_K8", "1")
    KVH, G, D, PS = 2, 8, 256, 16
    lens, qls = [500, 90, 64], [1, 30, 1]
    c = synth.paged_case(99, lens, KVH, G, D, PS, outliers=True, ql_list=qls)
    dev = torch.device("cuda")
    B, HQ, NT = len(lens), KVH * G, sum(qls)
    kscale, vscale = 0.25, 1.0
    layer = SimpleNamespace(_k_scale_float=kscale, _v_scale_float=vscale, layer_name="model.layers.2.self_attn.attn")
    impl = BE.HorizonFp4Impl(HQ, D, D ** -0.5, num_kv_heads=KVH, kv_cache_dtype="nvfp4", max_num_seqs=8)
    assert impl.k8
    kv_cache = torch.full((c["NP"], KVH, PS, 400), 0x7F, dtype=torch.uint8, device=dev)
    impl.do_kv_cache_update(layer, bf16_tensor(c["key"]), bf16_tensor(c["val"]), kv_cache,
                            torch.from_numpy(c["slots"]).to(dev))
    lay = O.Layout.k8_slots(PS, KVH, D)
    gk, gv = np.full(KVH, kscale, np.float32), np.full(KVH, vscale, np.float32)
    want = np.full(kv_cache.numel(), 0x7F, np.uint8)
    O.write(c["key"], c["val"], want, lay, c["slots"], gk, gv, True)
    assert np.array_equal(kv_cache.cpu().numpy().reshape(-1), want)
    qsl = torch.from_numpy(c["qsl"])
    cam = SimpleNamespace(num_reqs=B, num_actual_tokens=NT, query_start_loc=qsl.to(dev), query_start_loc_cpu=qsl,
                          seq_lens=torch.from_numpy(c["seq_lens"]).to(dev),
                          block_table_tensor=torch.from_numpy(c["bt"]).to(dev),
                          slot_mapping=torch.zeros(NT, dtype=torch.int64, device=dev),
                          seq_lens_cpu_upper_bound=torch.from_numpy(c["seq_lens"]))
    meta = BE.HorizonFp4Builder().build(0, cam)
    output = torch.zeros((NT, HQ * D), dtype=torch.bfloat16, device=dev)
    impl.forward(layer, bf16_tensor(c["q"]).view(NT, HQ * D), None, None, kv_cache, meta, output)
    ref, _ = O.attention(c["q"], want, lay, c["bt"], c["seq_lens"], c["qsl"], KVH, D ** -0.5, gk, gv, 1.0)
    from cases import errors
    mx, mn, rl = errors(output.view(NT, HQ, D), ref)
    assert rl <= 2.5e-3 and mn <= 2e-3 and mx <= 6e-2, (mx, mn, rl)
