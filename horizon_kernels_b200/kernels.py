"""Host wrappers of the three CUDA kernels, with the call signatures of the reference's serving module
(nvidia-sm120/horizon_kvfp4/kernels/kv_fp4_serving.py): `write`, `decode_ragged`, `flat_views`, `plan_splits`.

The wrappers only marshal pointers, sizes and the current CUDA stream into the C ABI (include/hkv.h). They allocate
nothing and never synchronise, so calls can be captured in a CUDA graph. There is no CPU or PyTorch fallback."""
import ctypes as C

import torch

from . import _lib
from .layout import flat_views  # noqa: F401  (re-exported: part of the reference's API)

LOG2E = 1.4426950408889634
_SMS = {}


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _need_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("hkv kernels need CUDA tensors: there is no CPU path")


def num_sms(device=None) -> int:
    d = torch.cuda.current_device() if device is None else torch.device(device).index
    if d not in _SMS:
        _SMS[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _SMS[d]


def plan_splits(B: int, KVH: int, ctas_per_sm: int = 4, max_splits: int = 64, sms: int = None) -> int:
    """splits per (request, kv head); depends on the batch size only, so it is safe under CUDA graphs
    (reference: kv_fp4_serving.py:889-891)"""
    sms = num_sms() if sms is None else sms
    return max(1, min(max_splits, sms * ctas_per_sm // max(1, B * KVH)))


def workspace_bytes(B: int, KVH: int, G: int, D: int, qlmax: int = 1) -> int:
    n = int(_lib.load().hkv_decode_workspace_bytes(B, KVH, G, D, qlmax))
    if n == 0:
        raise _lib.HkvError(-3, "hkv_decode_workspace_bytes")
    return n


def alloc_workspace(B: int, KVH: int, G: int, D: int, qlmax: int = 1, device="cuda") -> torch.Tensor:
    """zeroed uint8 workspace for decode batches of up to B requests; allocate once, outside graph capture
    (reference: backend.py:263-277)"""
    with torch.cuda.device(device):
        return torch.zeros(workspace_bytes(B, KVH, G, D, qlmax), dtype=torch.uint8, device=device)


SIGN_SEED = 0x6B7634              # the reference's seed of the rotation's sign vector (kv_fp4_ref.py:49)


def hadamard_signs(D: int, seed: int = SIGN_SEED, device=None) -> torch.Tensor:
    """the reference's fixed random +-1 per channel (kv_fp4_ref.py:57-60): the same vector must serve q and k"""
    g = torch.Generator().manual_seed(seed)
    s = (torch.randint(0, 2, (D,), generator=g) * 2 - 1).to(torch.float32)
    return s if device is None else s.to(device)


def rotate(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """fp32 FWHT(x * signs) * D^-0.5 over the last dimension, butterflies in the stage order h = 1, 2, .., D / 2
    (kv_fp4_ref.py:63-87). A torch helper for eager paths (prefill queries); the kernels rotate in registers."""
    D = x.shape[-1]
    y = (x.float() * signs.to(x.device, torch.float32)).reshape(-1, D)
    h = 1
    while h < D:
        v = y.view(-1, D // (2 * h), 2, h)
        y = torch.stack((v[:, :, 0] + v[:, :, 1], v[:, :, 0] - v[:, :, 1]), dim=2).reshape(-1, D)
        h *= 2
    scale = float(torch.tensor(1.0 / (D ** 0.5), dtype=torch.float32))
    return (y * scale).view(x.shape)


def _check_scales(gk, gv, KVH):
    for t in (gk, gv):
        if t.dtype != torch.float32 or t.shape != (KVH,) or not t.is_contiguous():
            raise TypeError("gk / gv must be contiguous fp32 tensors with one entry per kv head")


def _check_signs(signs, D):
    if signs is None:
        return
    _need_cuda(signs)
    if signs.dtype != torch.float32 or signs.shape != (D,) or not signs.is_contiguous():
        raise TypeError("signs must be a contiguous fp32 tensor of head_dim entries")


def write(key, value, flat, strides, PS, slot_mapping, gk, gv, search=True, signs=None, k8=False):
    """key / value (NT, KVH, D) bf16 views (any token / head strides, last dim contiguous); slot_mapping (NSL,) int64,
    slot < 0 skipped, tokens beyond NSL untouched; flat / strides from flat_views; gk / gv (KVH,) fp32.
    signs (D,) fp32 of +-1 on the device: the keys are rotated (FWHT(k * signs) * D^-0.5 in fp32) before they are
    quantised. Bit-exact to the reference's write_reference (kv_fp4_ref.py:233-245). Signature of
    kv_fp4_serving.py:994."""
    if k8 and signs is not None:
        raise ValueError("the K8V4 slot keeps FP8 keys: no rotation")
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise TypeError("key / value must be bf16")
    if key.dim() != 3 or value.shape != key.shape:
        raise ValueError("key / value must be (tokens, kv heads, head_dim) tensors of one shape")
    if key.stride(-1) != 1 or value.stride(-1) != 1:
        raise ValueError("key / value need a contiguous last dimension")
    if slot_mapping.dtype != torch.int64 or slot_mapping.dim() != 1 or not slot_mapping.is_contiguous():
        raise TypeError("slot_mapping must be contiguous int64")
    if slot_mapping.shape[0] > key.shape[0]:
        raise ValueError("more slots than tokens")
    _check_scales(gk, gv, key.shape[1])
    _need_cuda(key, value, slot_mapping, gk, gv, *flat)
    _check_signs(signs, key.shape[2])
    KVH, D = key.shape[1], key.shape[2]
    kd, ksf, vd, vsf = flat
    st = (C.c_int64 * 6)(*strides)
    args = (_ptr(key), _ptr(value), key.stride(0), key.stride(1), value.stride(0), value.stride(1), _ptr(kd), _ptr(ksf),
            _ptr(vd), _ptr(vsf), st, int(PS), _ptr(slot_mapping), slot_mapping.shape[0], _ptr(gk), _ptr(gv), KVH, D,
            int(bool(search)))
    with torch.cuda.device(key.device):
        if k8:                  # flat = (key bytes, unused, value codes, value scales)
            rc = _lib.load().hkv_write_k8(*args[:6], _ptr(kd), _ptr(vd), _ptr(vsf), *args[10:], _stream())
        elif signs is None:
            rc = _lib.load().hkv_write(*args, _stream())
        else:
            rc = _lib.load().hkv_write_rot(*args, _ptr(signs), _stream())
    _lib.check(rc, "hkv_write")


def decode_ragged(query, flat, strides, PS, block_tables, seq_lens, query_start_loc, bmm1_scale, bmm2_scale, gk, gv,
                  qlmax, out, workspace, splits=None, nst=None, ncw=None, min_chunk=None, tw=None, signs=None,
                  k8=False):
    """query (NT, HQ, D) bf16 contiguous; block_tables (B, MP) int32; seq_lens (B,) int32; query_start_loc (B + 1,)
    int32; out (>= NT, HQ, D) bf16, rows of requests without (or with more than qlmax) query tokens are left
    untouched; workspace from alloc_workspace. out = softmax(q k^T * bmm1_scale * gk) v * gv * bmm2_scale.
    The workspace must have been zero-filled once (alloc_workspace does).
    `splits` bounds the number of stream partitions to B * KVH * splits; the tuning arguments of the reference
    (nst, ncw, min_chunk, tw) are accepted and ignored. signs (D,) fp32 of +-1 on the device: the keys in the cache
    were written rotated, and the kernel rotates the UNROTATED query it is given the same way.
    Signature of kv_fp4_serving.py:894-895."""
    if k8 and signs is not None:
        raise ValueError("the K8V4 slot keeps FP8 keys: no rotation")
    if query.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise TypeError("query / out must be bf16")
    if query.dim() != 3 or out.dim() != 3 or out.shape[1:] != query.shape[1:] or out.shape[0] < query.shape[0]:
        raise ValueError("query (tokens, heads, head_dim); out (>= tokens, heads, head_dim)")
    if not query.is_contiguous() or not out.is_contiguous():
        raise ValueError("query / out must be contiguous")
    for t in (block_tables, seq_lens, query_start_loc):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise TypeError("block_tables / seq_lens / query_start_loc must be contiguous int32")
    if block_tables.dim() != 2 or seq_lens.shape != (block_tables.shape[0],) or \
            query_start_loc.shape != (block_tables.shape[0] + 1,):
        raise ValueError("block_tables (B, MP); seq_lens (B,); query_start_loc (B + 1,)")
    B, MP = block_tables.shape
    KVH = gk.shape[0]
    HQ, D = query.shape[1], query.shape[2]
    _check_scales(gk, gv, KVH)
    if HQ % KVH:
        raise ValueError("query heads must be a multiple of the kv heads")
    G = HQ // KVH
    _need_cuda(query, block_tables, seq_lens, query_start_loc, gk, gv, out, workspace, *flat)
    _check_signs(signs, query.shape[2])
    S = 0 if splits is None else int(splits)
    kd, ksf, vd, vsf = flat
    st = (C.c_int64 * 6)(*strides)
    wsb = workspace.numel() * workspace.element_size()
    L = _lib.load()
    with torch.cuda.device(query.device):
        s = _stream()
        args = (_ptr(query), _ptr(kd), _ptr(ksf), _ptr(vd), _ptr(vsf), st, int(PS), _ptr(block_tables), MP,
                _ptr(seq_lens), _ptr(query_start_loc), B, KVH, G, D, int(qlmax), float(bmm1_scale), float(bmm2_scale),
                _ptr(gk), _ptr(gv), _ptr(workspace), wsb, S)
        if k8:
            rc = L.hkv_decode_k8(args[0], args[1], *args[3:], _ptr(out), s)
        elif signs is None:
            rc = L.hkv_decode(*args, _ptr(out), s)
        else:
            rc = L.hkv_decode_rot(*args, _ptr(signs), _ptr(out), s)
        _lib.check(rc, "hkv_decode")          # (split sequences are merged inside the launch: `out` is complete)
    return out


def _dequant(flat, strides, PS, block_tables, MP, rows, cu, n_rows, start, n_tokens, out_k, out_v, k8):
    _need_cuda(block_tables, out_k, out_v, *flat)
    if out_k.dtype not in (torch.bfloat16, torch.float16) or out_v.dtype != out_k.dtype:
        raise TypeError("out_k / out_v must both be bf16 or both fp16")
    if not out_k.is_contiguous() or not out_v.is_contiguous() or out_k.shape != out_v.shape:
        raise ValueError("out_k / out_v must be contiguous (n, KVH, D) tensors of one shape")
    if out_k.shape[0] < n_tokens:
        raise ValueError("output buffers shorter than the number of tokens")
    if block_tables.dtype != torch.int32 or not block_tables.is_contiguous():
        raise TypeError("block tables must be contiguous int32")
    KVH, D = out_k.shape[1], out_k.shape[2]
    kd, ksf, vd, vsf = flat
    st = (C.c_int64 * 6)(*strides)
    tail = (st, int(PS), _ptr(block_tables), int(MP), None if rows is None else _ptr(rows),
            None if cu is None else _ptr(cu), int(n_rows), int(start), int(n_tokens), _ptr(out_k), _ptr(out_v), KVH, D,
            int(out_k.dtype == torch.float16))
    with torch.cuda.device(out_k.device):
        if k8:
            rc = _lib.load().hkv_dequant_k8(_ptr(kd), _ptr(vd), _ptr(vsf), *tail, _stream())
        else:
            rc = _lib.load().hkv_dequant(_ptr(kd), _ptr(ksf), _ptr(vd), _ptr(vsf), *tail, _stream())
    _lib.check(rc, "hkv_dequant")


def dequant_tokens(flat, strides, PS, block_table_row, start, n, out_k, out_v, k8=False):
    """positions [start, start + n) of one request (its block-table row, int32) -> out_k / out_v[:n], (n, KVH, D) bf16
    or fp16 by the output dtype: e2m1 * e4m3, exact, no global scale. Signature of kv_fp4_serving.py:918."""
    if block_table_row.dim() != 1:
        raise ValueError("block_table_row is the 1-D block-table row of one request")
    if (start + n + PS - 1) // PS > block_table_row.shape[0]:
        raise ValueError("positions beyond the block-table row")
    _dequant(flat, strides, PS, block_table_row, block_table_row.shape[0], None, None, 0, start, n, out_k, out_v, k8)
    return out_k[:n], out_v[:n]


def dequant_multi(flat, strides, PS, block_tables, rows, cu, n_rows, n_tokens, out_k, out_v, k8=False):
    """full contexts of requests rows[r] (int32, device), packed: out_k / out_v[cu[r]:cu[r + 1]] = request rows[r];
    cu (n_rows + 1,) int32 device with cu[n_rows] == n_tokens. Exact, no global scale.
    Signature of kv_fp4_serving.py:1008."""
    _need_cuda(rows, cu)
    for t in (rows, cu):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise TypeError("rows / cu must be contiguous int32")
    if block_tables.dim() != 2 or cu.shape[0] < n_rows + 1 or rows.shape[0] < n_rows:
        raise ValueError("block_tables (B, MP); rows (>= n_rows,); cu (>= n_rows + 1,)")
    _dequant(flat, strides, PS, block_tables, block_tables.shape[1], rows, cu, n_rows, 0, n_tokens, out_k, out_v, k8)


OPT_EARLY_METADATA = 1


def set_option(option: int, value: int) -> None:
    """process-wide library options (include/hkv.h `hkv_set_option`). OPT_EARLY_METADATA = 1 tells the decode kernel that
    seq_lens and query_start_loc are older than the kernel launched just before it, as they are in a serving engine."""
    _lib.check(_lib.load().hkv_set_option(int(option), int(value)), "hkv_set_option")


def workspace_status(workspace) -> int:
    """device status word of the last launches (0 = ok); synchronises, for tests and debugging"""
    st = C.c_int(0)
    with torch.cuda.device(workspace.device):
        rc = _lib.load().hkv_workspace_status(_ptr(workspace), C.byref(st), _stream())
    _lib.check(rc, "hkv_workspace_status")
    return int(st.value)
