"""horizon_kernels_b200: the NVFP4 KV-cache attention path of Horizon-Tech-doo/horizon-kernels
(`nvidia-sm120/horizon_kvfp4`) rebuilt for NVIDIA B200 (sm_100a): quantize-on-write, paged split-K decode and the
log-sum-exp combine as hand-written CUDA behind a C ABI (include/hkv.h), plus the vLLM plugin surface.

`register()` is the vLLM general-plugin entry point: with HORIZON_KVFP4=1 it registers HorizonFp4Backend as vLLM's CUSTOM
attention backend (select it with `--attention-backend CUSTOM --kv-cache-dtype nvfp4`); without the switch it does
nothing (reference: nvidia-sm120/horizon_kvfp4/__init__.py:38-42)."""
import os

__all__ = ["register"]


def register():
    if os.environ.get("HORIZON_KVFP4", "0") != "1":
        return
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    register_backend(AttentionBackendEnum.CUSTOM, "horizon_kernels_b200.backend.HorizonFp4Backend")
