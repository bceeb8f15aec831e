"""Host logic of the vLLM plugin surface, exercised with duck-typed stand-ins for vLLM's objects (no vLLM import, no
GPU): capability answers, constructor checks, and the metadata builder's split into decode and prefill rows
(reference: nvidia-sm120/horizon_kvfp4/backend.py:84-181)."""
import os
from types import SimpleNamespace

import pytest
import torch

os.environ["HORIZON_KVFP4_STANDALONE"] = "1"
from horizon_kernels_b200 import backend as BE  # noqa: E402


def test_backend_capabilities():
    B = BE.HorizonFp4Backend
    assert B.get_name() == "CUSTOM"
    assert B.accept_output_buffer and not B.forward_includes_kv_cache_update
    assert B.supported_dtypes == [torch.bfloat16] and B.supported_kv_cache_dtypes == ["nvfp4"]
    assert B.get_supported_head_sizes() == [128, 256]
    assert B.get_supported_kernel_block_sizes() == [16, 32, 64]
    assert B.supports_kv_cache_dtype("nvfp4") and not B.supports_kv_cache_dtype("fp8")
    assert B.supports_attn_type("decoder") and not B.supports_attn_type("encoder")
    assert B.get_impl_cls() is BE.HorizonFp4Impl and B.get_builder_cls() is BE.HorizonFp4Builder


def test_customize_spec_sets_two_slots_per_kv_head(monkeypatch):
    from dataclasses import dataclass
    monkeypatch.delenv("HORIZON_KVFP4_K8", raising=False)

    @dataclass
    class Spec:
        head_size: int
        head_size_v: int
        num_kv_heads: int
        kv_quant_mode: object
        state_content_bytes: object = None
        num_head_slots: object = None
    s = BE.HorizonFp4Backend.customize_spec(Spec(128, 128, 8, SimpleNamespace(is_nvfp4=True)))
    assert s.num_head_slots == 16 and s.state_content_bytes == 72
    s = BE.HorizonFp4Backend.customize_spec(Spec(256, 256, 2, SimpleNamespace(is_nvfp4=True)))
    assert s.num_head_slots == 4 and s.state_content_bytes == 144
    untouched = Spec(128, 128, 8, SimpleNamespace(is_nvfp4=False))
    assert BE.HorizonFp4Backend.customize_spec(untouched) is untouched
    with pytest.raises(ValueError):
        BE.HorizonFp4Backend.customize_spec(Spec(64, 64, 8, SimpleNamespace(is_nvfp4=True)))
    monkeypatch.setenv("HORIZON_KVFP4_K8", "1")                       # K8V4: one 400-byte slot per kv head
    s = BE.HorizonFp4Backend.customize_spec(Spec(256, 256, 2, SimpleNamespace(is_nvfp4=True)))
    assert s.num_head_slots == 2 and s.state_content_bytes == 400
    with pytest.raises(ValueError):
        BE.HorizonFp4Backend.customize_spec(Spec(128, 128, 8, SimpleNamespace(is_nvfp4=True)))
    with pytest.raises(ValueError):
        BE.HorizonFp4Impl(32, 128, 0.1, num_kv_heads=8, kv_cache_dtype="nvfp4")


def test_impl_constructor_checks():
    I = BE.HorizonFp4Impl
    ok = I(32, 128, 0.088, num_kv_heads=8, kv_cache_dtype="nvfp4")
    assert ok.G == 4 and ok.qlmax == 1
    with pytest.raises(ValueError):
        I(32, 64, 0.1, num_kv_heads=8, kv_cache_dtype="nvfp4")
    with pytest.raises(ValueError):
        I(32, 128, 0.1, num_kv_heads=8, kv_cache_dtype="fp8")
    with pytest.raises(ValueError):
        I(32, 128, 0.1, num_kv_heads=8, kv_cache_dtype="nvfp4", sliding_window=128)
    with pytest.raises(ValueError):
        I(32, 128, 0.1, num_kv_heads=8, kv_cache_dtype="nvfp4", sinks=torch.zeros(1))
    assert I(32, 128, 0.1, num_kv_heads=2, kv_cache_dtype="nvfp4").G == 16     # 16 query rows per kv head: two passes
    assert I(32, 128, 0.1, num_kv_heads=8, kv_cache_dtype="nvfp4", num_speculative_tokens=3).qlmax == 4
    with pytest.raises(ValueError):
        I(128, 128, 0.1, num_kv_heads=1, kv_cache_dtype="nvfp4")           # 128 query rows per kv head


def cam(qsl, seq_lens, MP=4):
    n = len(seq_lens)
    return SimpleNamespace(num_reqs=n, num_actual_tokens=qsl[-1], query_start_loc=torch.tensor(qsl, dtype=torch.int32),
                           query_start_loc_cpu=torch.tensor(qsl, dtype=torch.int32),
                           seq_lens=torch.tensor(seq_lens, dtype=torch.int32),
                           block_table_tensor=torch.zeros((n + 2, MP), dtype=torch.int32),
                           slot_mapping=torch.arange(qsl[-1], dtype=torch.int64), seq_lens_cpu_upper_bound=None)


def test_builder_splits_decode_and_prefill_rows():
    b = BE.HorizonFp4Builder()
    m = b.build(0, cam([0, 1, 2, 3], [10, 20, 30]))
    assert m.num_reqs == 3 and m.has_decode and m.prefill_rows == [] and m.qlmax == 1 and m.decode_threshold == 1
    assert m.block_table.shape[0] == 3 and m.query_start_loc.shape[0] == 4
    m = b.build(0, cam([0, 1, 9, 9, 10], [10, 200, 5, 30]))            # a prefill chunk and a padding request
    assert m.has_decode and m.prefill_rows == [(1, 1, 9, 200)]
    spec_cfg = SimpleNamespace(speculative_config=SimpleNamespace(num_speculative_tokens=1))
    b2 = BE.HorizonFp4Builder(vllm_config=spec_cfg)
    m = b2.build(0, cam([0, 2, 4, 5], [10, 20, 30]))
    assert m.decode_threshold == 2 and m.qlmax == 2 and m.prefill_rows == []


def test_profiling_run_returns_output_and_output_quantisation_is_refused():
    impl = BE.HorizonFp4Impl(32, 128, 0.088, num_kv_heads=8, kv_cache_dtype="nvfp4")
    out = torch.zeros(4, 32 * 128, dtype=torch.bfloat16)
    assert impl.forward(None, out, None, None, None, None, out) is out
    m = BE.HorizonFp4Builder().build(0, cam([0, 1, 9], [10, 200]))
    assert m.prefill_rows == [(1, 1, 9, 200)] and m.has_decode
    with pytest.raises(ValueError):
        impl.forward(None, out, None, None, None, m, out, output_scale=torch.ones(1))


def test_register_is_gated(monkeypatch):
    import horizon_kernels_b200
    monkeypatch.delenv("HORIZON_KVFP4", raising=False)
    horizon_kernels_b200.register()                       # does nothing, imports nothing
