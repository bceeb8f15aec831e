"""vLLM attention-backend surface for the NVFP4 KV cache on B200: the drop-in for the reference's
`nvidia-sm120/horizon_kvfp4/backend.py` (class and method names, argument meaning and error behaviour follow it).

  HorizonFp4Backend   static capabilities: bf16 activations, "nvfp4" cache dtype, head sizes 128 / 256, page sizes
                      16 / 32 / 64, 2 * KVH head slots of D/2 + D/16 bytes per token (reference backend.py:84-130)
  HorizonFp4Metadata  per-step tensors (reference backend.py:133-144)
  HorizonFp4Builder   builds the metadata from vLLM's CommonAttentionMetadata (reference backend.py:147-181)
  HorizonFp4Impl      do_kv_cache_update -> CUDA quantize-on-write; forward -> CUDA split-K decode + combine
                      (reference backend.py:189-436)

The classes derive from vLLM's base classes when vLLM has already been imported by the process (that is, when vLLM
loads this plugin); otherwise from small stand-ins, so the surface can be exercised and benchmarked without importing
vLLM. Rows with more query tokens than the decode threshold (prefill over a cached prefix) take the exact
dequantisation kernel, chunk by chunk, followed by torch matmuls with a running log-sum-exp (library attention, as the
reference uses FlashInfer's FA2 and merge_state there, backend.py:517-543); that path is eager and outside the timed
hot path. There is no fallback to another backend.
"""
import os
import sys
from dataclasses import dataclass, replace
from typing import ClassVar

import torch

from . import kernels as K
from .layout import flat_views, k8_flat_views, k8_slot_bytes, k8_views, slot_bytes, slot_views

HEAD_SIZES = (128, 256)
PAGE_SIZES = (16, 32, 64)
MAX_ROWS = 64                     # query rows per kv head, G * (1 + draft tokens): eight per pass over the cache
_STATE = {}                       # per device: decode workspace


def _env(name, default):
    return os.environ.get(name, default)


def _vllm_bases():
    """vLLM's base classes when vLLM is loaded in this process, else None"""
    if "vllm" not in sys.modules or _env("HORIZON_KVFP4_STANDALONE", "0") == "1":
        return None
    try:
        from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadata,
                                               AttentionMetadataBuilder, AttentionType)
        return dict(AttentionBackend=AttentionBackend, AttentionCGSupport=AttentionCGSupport,
                    AttentionImpl=AttentionImpl, AttentionMetadata=AttentionMetadata,
                    AttentionMetadataBuilder=AttentionMetadataBuilder, AttentionType=AttentionType)
    except Exception:  # noqa: BLE001  (an older or newer vLLM without these names: fall back to the stand-ins)
        return None


class _StandInType:
    DECODER = "decoder"


class _StandInCG:
    UNIFORM_BATCH = "UNIFORM_BATCH"


class _StandInBuilderBase:
    reorder_batch_threshold = 1

    def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None):
        self.kv_cache_spec, self.layer_names, self.vllm_config, self.device = kv_cache_spec, layer_names, vllm_config, device

    def _init_reorder_batch_threshold(self, threshold, supports_spec_as_decode=False):
        spec = getattr(self.vllm_config, "speculative_config", None) if self.vllm_config is not None else None
        n = (getattr(spec, "num_speculative_tokens", 0) or 0) if spec is not None else 0
        self.reorder_batch_threshold = threshold + n if supports_spec_as_decode else threshold


def _build_classes():
    vb = _vllm_bases()
    BackendBase = vb["AttentionBackend"] if vb else object
    ImplBase = vb["AttentionImpl"] if vb else object
    MetaBase = vb["AttentionMetadata"] if vb else object
    BuilderBase = vb["AttentionMetadataBuilder"] if vb else _StandInBuilderBase
    AttentionType = vb["AttentionType"] if vb else _StandInType
    CGSupport = vb["AttentionCGSupport"] if vb else _StandInCG

    class HorizonFp4Backend(BackendBase):
        accept_output_buffer: bool = True
        forward_includes_kv_cache_update: bool = False
        supported_dtypes: ClassVar[list] = [torch.bfloat16]
        supported_kv_cache_dtypes: ClassVar[list] = ["nvfp4"]

        @classmethod
        def customize_spec(cls, spec):
            """2 * KVH head slots of D/2 + D/16 bytes per token (reference backend.py:91-97)"""
            if getattr(spec, "state_content_bytes", None) is not None or not spec.kv_quant_mode.is_nvfp4:
                return spec
            if spec.head_size not in HEAD_SIZES or spec.head_size_v != spec.head_size:
                raise ValueError(f"horizon_kvfp4 needs head_dim in {HEAD_SIZES}, got {spec.head_size}")
            if _env("HORIZON_KVFP4_K8", "0") == "1":          # FP8 keys + FP4 values: one 400-byte slot per kv head
                if spec.head_size != 256:
                    raise ValueError("the K8V4 slot (HORIZON_KVFP4_K8) exists at head_dim 256 only")
                return replace(spec, num_head_slots=spec.num_kv_heads, state_content_bytes=k8_slot_bytes(256))
            return replace(spec, num_head_slots=2 * spec.num_kv_heads, state_content_bytes=slot_bytes(spec.head_size))

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_supported_kernel_block_sizes():
            return list(PAGE_SIZES)

        @classmethod
        def supported_kv_cache_layouts(cls):
            """both page orders of the reference (backend.py:107-110): head-major pages (a head's 16-token tile is one
            contiguous run, fetched with one bulk copy: the fast path) first, positions-outermost pages second (fetched
            row by row). The K8V4 slot is served head-major only."""
            both = _env("HORIZON_KVFP4_K8", "0") != "1"
            try:
                if _vllm_bases() is None:
                    raise RuntimeError("not inside vLLM")
                from vllm.v1.kv_cache_interface import KVCacheLayout
                return (KVCacheLayout.LBHNC, KVCacheLayout.LBNHC) if both else (KVCacheLayout.LBHNC,)
            except Exception:  # noqa: BLE001
                return ("LBHNC", "LBNHC") if both else ("LBHNC",)

        @classmethod
        def get_supported_head_sizes(cls):
            return list(HEAD_SIZES)

        @classmethod
        def supports_kv_cache_dtype(cls, kv_cache_dtype) -> bool:
            return kv_cache_dtype == "nvfp4"

        @classmethod
        def supports_attn_type(cls, attn_type) -> bool:
            return attn_type == AttentionType.DECODER

        @staticmethod
        def get_impl_cls():
            return HorizonFp4Impl

        @staticmethod
        def get_builder_cls():
            return HorizonFp4Builder

    @dataclass
    class HorizonFp4Metadata(MetaBase):
        num_reqs: int
        num_actual_tokens: int
        query_start_loc: torch.Tensor          # (num_reqs + 1,) int32, device
        seq_lens: torch.Tensor                 # (num_reqs,) int32, device (exact)
        block_table: torch.Tensor              # (num_reqs, max_blocks) int32, device
        slot_mapping: torch.Tensor
        has_decode: bool                       # some request has <= decode_threshold query tokens
        prefill_rows: list                     # [(row, q0, q1, seq_len)] of requests with more query tokens
        decode_threshold: int
        qlmax: int = 1                         # decode kernel variant: smallest of 1 / 2 / 4 / 8 >= the longest decode row

    class HorizonFp4Builder(BuilderBase):
        _cudagraph_support: ClassVar = CGSupport.UNIFORM_BATCH
        supports_draft_decode_metadata_update: bool = True

        def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None):
            super().__init__(kv_cache_spec, layer_names, vllm_config, device)
            self._init_reorder_batch_threshold(1, supports_spec_as_decode=True)

        def build(self, common_prefix_len, common_attn_metadata, fast_build=False, **kwargs):
            """reference backend.py:157-177: device tensors sliced to the step's requests; rows are split on the CPU
            copy of query_start_loc into decode rows (<= threshold tokens) and prefill rows"""
            cam = common_attn_metadata
            n = cam.num_reqs
            thr = int(self.reorder_batch_threshold or 1)
            qsl = cam.query_start_loc_cpu[: n + 1].tolist()
            qlens = [qsl[i + 1] - qsl[i] for i in range(n)]
            rows = [i for i in range(n) if qlens[i] > thr]
            dec = [q for q in qlens if 0 < q <= thr]
            mx = max(dec) if dec else 1
            qlmax = next((c for c in (1, 2, 4, 8) if c >= mx and c <= thr), thr)
            prefill_rows = []
            if rows:
                ub = getattr(cam, "seq_lens_cpu_upper_bound", None)
                if ub is None:
                    ub = cam.seq_lens[:n].cpu()
                prefill_rows = [(i, qsl[i], qsl[i + 1], int(ub[i])) for i in rows]
            return HorizonFp4Metadata(
                num_reqs=n, num_actual_tokens=cam.num_actual_tokens, query_start_loc=cam.query_start_loc[: n + 1],
                seq_lens=cam.seq_lens[:n], block_table=cam.block_table_tensor[:n], slot_mapping=cam.slot_mapping,
                has_decode=len(rows) < n, prefill_rows=prefill_rows, decode_threshold=thr, qlmax=qlmax)

        def update_draft_decode_metadata(self, metadata) -> None:
            pass

    class HorizonFp4Impl(ImplBase):
        supports_quant_query_input: bool = False
        can_return_lse_for_decode: bool = False

        def __init__(self, num_heads, head_size, scale, num_kv_heads=None, alibi_slopes=None, sliding_window=None,
                     kv_cache_dtype="auto", logits_soft_cap=None, attn_type=AttentionType.DECODER,
                     kv_sharing_target_layer_name=None, **kwargs):
            # the reference asserts the same feature set (backend.py:196-200); here misuse raises
            if head_size not in HEAD_SIZES:
                raise ValueError(f"horizon_kvfp4 needs head_dim in {HEAD_SIZES}, got {head_size}")
            if kv_cache_dtype != "nvfp4":
                raise ValueError(f"horizon_kvfp4 serves kv_cache_dtype 'nvfp4' only, got {kv_cache_dtype!r}")
            if alibi_slopes is not None or sliding_window is not None or logits_soft_cap:
                raise ValueError("alibi, sliding windows and logit soft caps are not supported")
            if kv_sharing_target_layer_name is not None:
                raise ValueError("KV sharing is not supported")
            if kwargs.get("sinks") is not None:
                raise ValueError("attention sinks are not supported")
            if attn_type != AttentionType.DECODER:
                raise ValueError("decoder self-attention only")
            self.num_heads = num_heads
            self.head_size = head_size
            self.scale = float(scale)
            self.num_kv_heads = num_kv_heads or num_heads
            self.kv_cache_dtype = kv_cache_dtype
            self.attn_type = attn_type
            self.kv_sharing_target_layer_name = None
            self.sliding_window = None
            self.G = self.num_heads // self.num_kv_heads
            # HORIZON_KVFP4_K8=1: the K8V4 slot (FP8 keys, FP4 values; reference backend.py:50-54, :211-212)
            self.k8 = _env("HORIZON_KVFP4_K8", "0") == "1"
            if self.k8 and (head_size != 256 or _env("HORIZON_KVFP4_HAD", "0") == "1"):
                raise ValueError("HORIZON_KVFP4_K8 needs head_dim 256 and keeps FP8 keys: the rotation must be off")
            # HORIZON_KVFP4_HAD=1: keys are written rotated (Hadamard) and queries rotated inside the decode kernel
            # (reference backend.py:214-222, kv_fp4_ref.py:31-35)
            self.had = _env("HORIZON_KVFP4_HAD", "0") == "1"
            self._signs = None
            self.search = _env("HORIZON_KVFP4_SEARCH", "1") == "1"
            self.cps = int(_env("HORIZON_KVFP4_CPS", "0"))        # splits per (request, kv head); 0 = fill the GPU
            # prefill rows (backend.py:229, :16-25 of the reference): fp16 compute dtype, context chunk in tokens
            self.pf16 = _env("HORIZON_KVFP4_PF16", "1") == "1"
            self.prefill_chunk = max(16, int(_env("HORIZON_KVFP4_CHUNK", "65536")))
            self._gk = self._gv = None
            self._views = None
            nspec, max_reqs = 0, int(kwargs.get("max_num_seqs", 0) or 0)
            try:
                if _vllm_bases() is None:
                    raise RuntimeError("not inside vLLM")
                from vllm.config import get_current_vllm_config
                cfg = get_current_vllm_config()
                spec = cfg.speculative_config
                nspec = (spec.num_speculative_tokens or 0) if spec is not None else 0
                max_reqs = max_reqs or cfg.scheduler_config.max_num_seqs
            except Exception:  # noqa: BLE001  (outside a vLLM engine: keyword arguments or defaults)
                nspec = int(kwargs.get("num_speculative_tokens", 0) or 0)
            self.qlmax = 1 + nspec
            if self.G * self.qlmax > MAX_ROWS:
                raise ValueError(f"G * (1 + draft tokens) = {self.G * self.qlmax} exceeds {MAX_ROWS} query rows per kv head")
            self.max_reqs = max_reqs or 1024

        # -------------------------------------------------------------------------------------------- helpers
        def _state(self, device):
            """one zeroed decode workspace per device, allocated on first use outside graph capture
            (reference backend.py:263-277)"""
            key = (str(device), self.num_kv_heads, self.G, self.head_size, self.qlmax)
            st = _STATE.get(key)
            if not _STATE.get("options"):
                # vLLM writes seq_lens and query_start_loc once per step, before the first layer runs, so the decode
                # kernel may read them ahead of its launch dependency (HORIZON_KVFP4_EARLY_META=0 turns this off)
                K.set_option(K.OPT_EARLY_METADATA, 0 if os.environ.get("HORIZON_KVFP4_EARLY_META", "1") == "0" else 1)
                _STATE["options"] = True
            if st is None or st["max_reqs"] < self.max_reqs:
                st = _STATE[key] = {"ws": K.alloc_workspace(self.max_reqs, self.num_kv_heads, self.G, self.head_size,
                                                            self.qlmax, device), "max_reqs": self.max_reqs}
            return st

        def _cache_views(self, kv_cache: torch.Tensor):
            """(num_blocks, 2*KVH, PS, slot) uint8 logical view -> flat parts + strides, memoised on the cache's
            address and strides (reference backend.py:279-300)"""
            v = self._views
            if v is not None and v[0] == kv_cache.data_ptr() and v[1] == tuple(kv_cache.stride()):
                return v[2]
            if self.k8:                                           # (blocks, KVH, PS, 400)
                if kv_cache.shape[1] != self.num_kv_heads:
                    raise ValueError(f"K8V4 cache must have one slot per kv head, got shape {tuple(kv_cache.shape)}")
                flat, strides = k8_flat_views(*k8_views(kv_cache, self.head_size))
            else:
                views = slot_views(kv_cache, self.num_kv_heads, self.head_size)
                flat, strides = flat_views(*views)
            out = dict(flat=flat, strides=strides, PS=kv_cache.shape[2])
            self._views = (kv_cache.data_ptr(), tuple(kv_cache.stride()), out)
            return out

        def _scales(self, layer, device):
            if self._gk is None:
                self._gk = torch.full((self.num_kv_heads,), float(layer._k_scale_float), device=device)
                self._gv = torch.full((self.num_kv_heads,), float(layer._v_scale_float), device=device)
            return self._gk, self._gv

        def _rot(self, device):
            """the rotation's sign vector on the device (None without HORIZON_KVFP4_HAD)"""
            if not self.had:
                return None
            if self._signs is None or self._signs.device != device:
                self._signs = K.hadamard_signs(self.head_size, device=device)
            return self._signs

        def process_weights_after_loading(self, act_dtype):
            """the kernels are compiled ahead of time; only the workspace is made here, outside any CUDA graph"""
            if torch.cuda.is_available():
                self._state(torch.device("cuda", torch.cuda.current_device()))

        # ---------------------------------------------------------------------------------------------- write
        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            """reference backend.py:389-403"""
            v = self._cache_views(kv_cache)
            gk, gv = self._scales(layer, key.device)
            D = self.head_size
            k3 = key.view(key.shape[0], self.num_kv_heads, D) if key.dim() == 2 else key
            v3 = value.view(value.shape[0], self.num_kv_heads, D) if value.dim() == 2 else value
            K.write(k3, v3, v["flat"], v["strides"], v["PS"], slot_mapping, gk, gv, self.search,
                    signs=self._rot(key.device), k8=self.k8)

        # -------------------------------------------------------------------------------------------- forward
        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                    output_block_scale=None):
            """reference backend.py:410-436"""
            if attn_metadata is None:                 # profiling run
                return output
            if output_scale is not None or output_block_scale is not None:
                raise ValueError("fused output quantisation is not supported")
            m = attn_metadata
            T = m.num_actual_tokens
            st = self._state(query.device)
            v = self._cache_views(kv_cache)
            gk, gv = self._scales(layer, query.device)
            q = query[:T]
            if q.dim() == 2:
                q = q.view(T, self.num_heads, self.head_size)
            if not q.is_contiguous():
                q = q.contiguous()
            out = output.view(output.shape[0], self.num_heads, self.head_size) if output.dim() == 2 else output
            if m.has_decode and m.num_reqs > 0:
                K.decode_ragged(q, v["flat"], v["strides"], v["PS"], m.block_table, m.seq_lens, m.query_start_loc,
                                self.scale, float(layer._v_scale_float), gk, gv, m.qlmax, out, st["ws"],
                                splits=self.cps or None, signs=self._rot(q.device), k8=self.k8)
            if m.prefill_rows:
                self._prefill_rows(layer, q, v, m, out)
            return output

        def _prefill_rows(self, layer, q, v, m, out):
            """requests with more query tokens than the decode threshold: the request's context (the new tokens were
            written by do_kv_cache_update) is dequantised exactly in chunks of HORIZON_KVFP4_CHUNK tokens (65,536, the
            reference's chunk: backend.py:16-25, :519-543) and attended chunk by chunk with a running log-sum-exp, so
            the memory held per request is bounded by the chunk, not by the context. Causal window of the reference:
            query token t of ql sees keys j < L - ql + t + 1. Compute dtype fp16 (HORIZON_KVFP4_PF16=1, the reference's
            default, backend.py:229: code * scale is exact in fp16) or bf16. The global scales are folded into the
            softmax scale and the output like the reference's sm / vs. Eager torch matmuls (a library path, as the
            reference calls FlashInfer there), outside the timed decode path."""
            sm = self.scale * float(layer._k_scale_float)
            vs = float(layer._v_scale_float)
            KVH, G, D = self.num_kv_heads, self.G, self.head_size
            dt = torch.float16 if self.pf16 else torch.bfloat16
            CH = self.prefill_chunk
            dev = q.device
            for row, q0, q1, L in m.prefill_rows:
                ql = q1 - q0
                if ql <= 0 or L <= 0:
                    continue
                qi = q[q0:q1]
                if self.had:                                                     # the cached keys are rotated
                    qi = K.rotate(qi, self._rot(dev)).to(torch.bfloat16)
                # (KVH, G * ql, D): row g * ql + t of a kv head is query head g, token t
                qh = qi.view(ql, KVH, G, D).permute(1, 2, 0, 3).reshape(KVH, G * ql, D).to(dt)
                lim = (L - ql + 1 + torch.arange(ql, device=dev)).repeat(G)      # keys visible to every row
                n_ch = min(CH, L)
                kk = torch.empty((n_ch, KVH, D), dtype=dt, device=dev)
                vv = torch.empty_like(kk)
                # query rows per block so that one block's scores stay near 256 MB
                QB = max(1, min(G * ql, (256 << 20) // max(1, KVH * n_ch * 4)))
                acc = torch.zeros((KVH, G * ql, D), dtype=torch.float32, device=dev)
                mx = torch.full((KVH, G * ql, 1), float("-inf"), dtype=torch.float32, device=dev)
                den = torch.zeros((KVH, G * ql, 1), dtype=torch.float32, device=dev)
                bt_row = m.block_table[row].contiguous()
                for c0 in range(0, L, CH):
                    n = min(CH, L - c0)
                    K.dequant_tokens(v["flat"], v["strides"], v["PS"], bt_row, c0, n, kk, vv, k8=self.k8)
                    kt = kk[:n].permute(1, 2, 0)                                 # (KVH, D, n)
                    # (KVH, n, D); the value product always takes fp16 operands: the dequantised values are exact in it
                    # and the probabilities lie in [0, 1]; both products accumulate and return fp32
                    vt = vv[:n].permute(1, 0, 2).to(torch.float16)
                    pos = c0 + torch.arange(n, device=dev)
                    for r0 in range(0, G * ql, QB):
                        r1 = min(G * ql, r0 + QB)
                        s_ = torch.bmm(qh[:, r0:r1], kt, out_dtype=torch.float32) * sm   # (KVH, rows, n), fp32 accumulate and output
                        s_.masked_fill_(pos[None, None, :] >= lim[None, r0:r1, None], float("-inf"))
                        nm = torch.maximum(mx[:, r0:r1], s_.amax(dim=-1, keepdim=True))
                        nm_safe = torch.where(torch.isinf(nm), torch.zeros_like(nm), nm)
                        p_ = torch.exp(s_ - nm_safe)
                        al = torch.exp(mx[:, r0:r1] - nm_safe)
                        den[:, r0:r1] = den[:, r0:r1] * al + p_.sum(dim=-1, keepdim=True)
                        acc[:, r0:r1] = acc[:, r0:r1] * al + torch.bmm(p_.to(torch.float16), vt, out_dtype=torch.float32)
                        mx[:, r0:r1] = nm
                o = acc / den.clamp_min(1e-30) * vs
                out[q0:q1].copy_(o.view(KVH, G, ql, D).permute(2, 0, 1, 3).reshape(ql, KVH * G, D).to(out.dtype))

    return dict(HorizonFp4Backend=HorizonFp4Backend, HorizonFp4Metadata=HorizonFp4Metadata,
                HorizonFp4Builder=HorizonFp4Builder, HorizonFp4Impl=HorizonFp4Impl)


_CLASSES = None


def __getattr__(name):
    """the four classes are created on first access, so that they pick vLLM's bases when vLLM is what imports them"""
    global _CLASSES
    if name in ("HorizonFp4Backend", "HorizonFp4Metadata", "HorizonFp4Builder", "HorizonFp4Impl"):
        if _CLASSES is None:
            _CLASSES = _build_classes()
        return _CLASSES[name]
    raise AttributeError(name)
