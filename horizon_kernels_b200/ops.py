"""torch custom ops over the C ABI: `torch.ops.hkv.write`, `torch.ops.hkv.decode`, `torch.ops.hkv.combine`.

The ops are thin: they pass the tensors' device pointers, the strides and the current CUDA stream to `libhkv.so`
(include/hkv.h) and mutate their output arguments in place, like the reference's TileLang-launched kernels mutate the
cache and the output buffer (kv_fp4_serving.py:994-1005, :894-915 in the reference). Registering them with torch lets
graph-capturing front ends (torch.compile, vLLM's piecewise graphs) treat the launches as opaque mutating ops. There is
a CUDA implementation only: calling an op with CPU tensors raises. `combine` is kept for the reference's three-launch
sequence; the merge of split sequences runs inside `decode`, so it launches nothing.
"""
import ctypes as C

import torch

from . import _lib
from . import kernels as K

_REGISTERED = False


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr())


def _strides6(strides):
    if len(strides) != 6:
        raise ValueError("strides must be (data page, data position, data head, scale page, scale position, scale head)")
    return tuple(int(x) for x in strides)


def register():
    """defines the hkv::* ops once per process; returns torch.ops.hkv"""
    global _REGISTERED
    if _REGISTERED:
        return torch.ops.hkv
    lib = torch.library.Library("hkv", "DEF")
    lib.define("write(Tensor key, Tensor value, Tensor(a!) k_data, Tensor(b!) k_sf, Tensor(c!) v_data, Tensor(d!) v_sf, "
               "int[] strides, int page_size, Tensor slot_mapping, Tensor gk, Tensor gv, bool search) -> ()")
    lib.define("decode(Tensor query, Tensor k_data, Tensor k_sf, Tensor v_data, Tensor v_sf, int[] strides, int page_size, "
               "Tensor block_tables, Tensor seq_lens, Tensor query_start_loc, float sm_scale, float v_scale, Tensor gk, "
               "Tensor gv, int qlmax, Tensor(a!) workspace, int splits, Tensor(b!) out) -> ()")
    lib.define("combine(Tensor(a!) workspace, Tensor query_start_loc, int num_kv_heads, int group, int head_dim, int qlmax, "
               "float v_scale, Tensor(b!) out) -> ()")

    # the implementations go through the host wrappers of kernels.py, so dtypes, contiguity and shapes are checked
    # once, in one place, before any pointer reaches the C ABI
    def write(key, value, k_data, k_sf, v_data, v_sf, strides, page_size, slot_mapping, gk, gv, search):
        K.write(key, value, (k_data, k_sf, v_data, v_sf), _strides6(strides), int(page_size), slot_mapping, gk, gv,
                bool(search))

    def decode(query, k_data, k_sf, v_data, v_sf, strides, page_size, block_tables, seq_lens, query_start_loc, sm_scale,
               v_scale, gk, gv, qlmax, workspace, splits, out):
        if block_tables.dim() != 2 or query_start_loc.shape[0] != block_tables.shape[0] + 1 or \
                seq_lens.shape[0] != block_tables.shape[0]:
            raise ValueError("block_tables (B, MP), seq_lens (B,), query_start_loc (B + 1,)")
        K.decode_ragged(query, (k_data, k_sf, v_data, v_sf), _strides6(strides), int(page_size), block_tables, seq_lens,
                        query_start_loc, float(sm_scale), float(v_scale), gk, gv, int(qlmax), out, workspace,
                        splits=int(splits) or None)

    def combine(workspace, query_start_loc, num_kv_heads, group, head_dim, qlmax, v_scale, out):
        K._need_cuda(workspace, query_start_loc, out)
        with torch.cuda.device(out.device):
            rc = _lib.load().hkv_combine(_p(workspace), workspace.numel() * workspace.element_size(), _p(query_start_loc),
                                         query_start_loc.shape[0] - 1, int(num_kv_heads), int(group), int(head_dim),
                                         int(qlmax), float(v_scale), _p(out), _stream())
        _lib.check(rc, "hkv_combine")

    lib.impl("write", write, "CUDA")
    lib.impl("decode", decode, "CUDA")
    lib.impl("combine", combine, "CUDA")
    register._lib = lib                       # keep the Library object alive
    _REGISTERED = True
    return torch.ops.hkv
