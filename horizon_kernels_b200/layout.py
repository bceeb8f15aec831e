"""Page geometry of the NVFP4 KV cache and the strided views the kernels address it through.

Per (token, kv head, side): D/2 bytes of E2M1 codes (element 2j in the low nibble of byte j) followed or accompanied by
D/16 E4M3 block scales. Two byte placements exist in the reference and both are accepted here:

  region layout   one page = [K codes (KVH, PS, D/2) | K scales (KVH, PS, D/16) | V codes | V scales]
                  (reference: kv_fp4_ref.py:205-230 `alloc_cache` / `split_views`)
  slot layout     logical (pages, 2*KVH, PS, slot), slot = [D/2 codes | D/16 scales], heads [0, KVH) = K and
                  [KVH, 2*KVH) = V; physically heads-outer or positions-outer inside a page
                  (reference: backend.py:279-300 `_cache_views`)

Every part is handed to the kernels as a [page, position, head, byte] view: a base pointer and three byte strides.
"""
import torch

BLOCK = 16


def slot_bytes(D: int) -> int:
    return D // 2 + D // BLOCK


def page_bytes(PS: int, KVH: int, D: int) -> int:
    return 2 * KVH * PS * slot_bytes(D)


def alloc_cache(num_pages: int, PS: int, KVH: int, D: int, device="cpu", fill: int = 0) -> torch.Tensor:
    """uint8 (num_pages, 2*KVH, PS, D/2 + D/16): the shape vLLM gives an NVFP4 cache of one layer"""
    return torch.full((num_pages, 2 * KVH, PS, slot_bytes(D)), fill, dtype=torch.uint8, device=device)


def split_views(cache: torch.Tensor, KVH: int):
    """region layout: (k_data, k_sf, v_data, v_sf) as [page, position, head, byte] views of a contiguous
    (pages, 2*KVH, PS, slot) cache"""
    NP, H2, PS, full = cache.shape
    if H2 != 2 * KVH or not cache.is_contiguous():
        raise ValueError("split_views needs a contiguous (pages, 2*KVH, PS, slot) cache")
    dd = full * 8 // 9
    sd = full - dd
    PB = cache.stride(0)
    side = KVH * PS * full
    base = cache.storage_offset()
    views = []
    for s in range(2):
        b0 = base + s * side
        views.append(torch.as_strided(cache, (NP, PS, KVH, dd), (PB, dd, PS * dd, 1), b0))
        views.append(torch.as_strided(cache, (NP, PS, KVH, sd), (PB, sd, PS * sd, 1), b0 + KVH * PS * dd))
    return tuple(views)


def slot_views(kv_cache: torch.Tensor, KVH: int, D: int):
    """slot layout: kv_cache is the LOGICAL (pages, 2*KVH, PS, slot) uint8 view (any physical order of the middle
    dimensions) -> (k_data, k_sf, v_data, v_sf) as [page, position, head, byte] views"""
    if kv_cache.dtype != torch.uint8 or kv_cache.shape[1] != 2 * KVH or kv_cache.shape[3] != slot_bytes(D):
        raise ValueError(f"expected uint8 (pages, {2 * KVH}, PS, {slot_bytes(D)}), got {tuple(kv_cache.shape)}")
    t = kv_cache.permute(0, 2, 1, 3)
    dd = D // 2
    return t[:, :, :KVH, :dd], t[:, :, :KVH, dd:], t[:, :, KVH:, :dd], t[:, :, KVH:, dd:]


def flat_views(k_data, k_sf, v_data, v_sf):
    """[page, position, head, byte] views -> (four flat uint8 tensors starting at each view's first byte, six byte
    strides (data page, position, head, scale page, position, head)). Same contract as the reference's `flat_views`
    (kv_fp4_serving.py:873-886)."""
    def flat(v):
        u = v.view(torch.uint8)
        n = u.untyped_storage().nbytes() - u.storage_offset()
        return torch.as_strided(u, (n,), (1,), u.storage_offset())
    if k_data.stride() != v_data.stride() or k_sf.stride() != v_sf.stride():
        raise ValueError("K and V views must share their strides")
    st = tuple(int(x) for x in (*k_data.stride()[:3], *k_sf.stride()[:3]))
    return (flat(k_data), flat(k_sf), flat(v_data), flat(v_sf)), st


K8_SLOT = 400                    # K8V4 slot at head_dim 256: [256 e4m3 key bytes | 128 value codes | 16 value scales]


def k8_slot_bytes(D: int) -> int:
    return D + D // 2 + D // 16


def k8_views(kv_cache: torch.Tensor, D: int = 256):
    """K8V4 cache, logical (pages, KVH, PS, slot) uint8 -> (kd, vd, vsf) as [page, position, head, byte] views: key
    bytes, value codes, value scales (reference `split_views_k8`, kv_fp4_ref.py:290-293)"""
    if kv_cache.dtype != torch.uint8 or kv_cache.dim() != 4 or kv_cache.shape[3] != k8_slot_bytes(D):
        raise ValueError(f"K8V4 cache must be uint8 (pages, KVH, PS, {k8_slot_bytes(D)})")
    t = kv_cache.permute(0, 2, 1, 3)
    return t[..., :D], t[..., D:D + D // 2], t[..., D + D // 2:]


def k8_flat_views(kd, vd, vsf):
    """(kd, vd, vsf) views -> the four-entry `flat` tuple and six strides the kernel wrappers take; the key-scale entry
    is a placeholder (the value scales again), as in the reference's backend (backend.py:287-291)"""
    (fk, fs, fv, fvs), st = flat_views(kd, vsf, vd, vsf)
    return (fk, fvs, fv, fvs), st
